"""GPU parity of the tcgen05 GEMM against the CPU oracle, through the C ABI.

Tolerance: |c - c32| <= 1e-2 + 1e-2 * |c32| against the oracle's fp32-accumulated result (the
stated bound), and the reference's own tighter acceptance bound atol = 1e-2 * sqrt(K / 1024),
rtol = 2e-3 (operators/GEMMTC.py:51-63; bf16 uses one bf16 ulp, 1.6e-2, as rtol)."""

import ctypes
import math

import numpy as np
import pytest

import oracle
from util import bits_to_torch, torch_to_bits

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def native():
    from deca_b200 import native as n

    n.lib()
    return n


def make_ab(M, N, K, dtype, seed=2):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.rand(M, K, generator=g) * 2 - 1
    b = torch.rand(K, N, generator=g) * 2 - 1
    return oracle.to_bits(a.numpy(), dtype), oracle.to_bits(b.numpy(), dtype)


def run_native(native, dtype, a_bits, b_bits, cfg=None):
    M, K = a_bits.shape
    N = b_bits.shape[1]
    a, b = bits_to_torch(a_bits, dtype), bits_to_torch(b_bits, dtype)
    buf = torch.full((M + 2, N), 7.0, dtype=a.dtype, device="cuda")
    c = buf[1 : M + 1]
    ccfg = None
    if cfg is not None:
        ccfg = ctypes.byref(native.GemmCfg(cfg.get("BM", 128), cfg.get("BN", 256), 64, cfg.get("stages", 4), cfg.get("raster", 8),
                                           cfg.get("epi_smem", 1), 1, cfg.get("acc_bufs", 2)))
    st = native.lib().deca_gemm16(native.DTYPE_CODE[dtype], a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, ccfg,
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st == 0, native.status_string(st)
    assert native.last_device_status() == (0, 0, 0)
    assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
    return torch_to_bits(c)


def check(dtype, a_bits, b_bits, c_bits):
    K = a_bits.shape[1]
    _, c32 = oracle.gemm16(a_bits, b_bits, dtype, want_f32=True)
    got = oracle.from_bits(c_bits, dtype)
    err = np.abs(got - c32)
    assert np.all(err <= 1e-2 + 1e-2 * np.abs(c32)), f"max err {err.max()}"
    atol, rtol = 1e-2 * math.sqrt(max(K, 64) / 1024), (2e-3 if dtype == "float16" else 1.6e-2)
    assert np.all(err <= atol + rtol * np.abs(c32)), f"max err {err.max()} (reference bound)"


SHAPES = [(128, 256, 64), (128, 256, 128), (128, 64, 512), (256, 512, 256), (384, 768, 320), (64, 80, 96),
          (200, 264, 136), (1, 8, 8), (1000, 1000, 1000), (130, 2056, 72), (2048, 256, 64),
          (256, 192, 128), (136, 448, 200)]  # N a whole number of 64-column blocks that the tile width does not divide


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_default_config_matches_oracle(native, dtype, shape):
    M, N, K = shape
    a, b = make_ab(M, N, K, dtype)
    check(dtype, a, b, run_native(native, dtype, a, b))


CONFIGS = [
    dict(BN=64, stages=2, acc_bufs=1, epi_smem=0), dict(BN=64, stages=8, acc_bufs=2), dict(BN=128, stages=3, raster=1),
    dict(BN=128, stages=6, acc_bufs=1), dict(BN=256, stages=2, epi_smem=0), dict(BN=256, stages=3, acc_bufs=1),
    dict(BN=256, stages=4, raster=2), dict(BN=128, stages=4, epi_smem=0, raster=16),
    dict(BM=256, BN=256, stages=3, acc_bufs=1), dict(BM=256, BN=256, stages=2, acc_bufs=1, epi_smem=0, raster=1),
    dict(BM=256, BN=128, stages=4, acc_bufs=2), dict(BM=256, BN=128, stages=4, acc_bufs=1, raster=3),
]


@pytest.mark.parametrize("cfg", CONFIGS, ids=lambda c: ",".join(f"{k}={v}" for k, v in c.items()))
def test_configs_match_oracle(native, cfg):
    # the last two: N is a whole number of 64-column blocks (B loaded by one three-dimensional copy per
    # tile) that the tile width does not divide, so the copy's last blocks lie outside the tensor
    for shape in ((640, 768, 448), (300, 520, 200), (1280, 1024, 128), (256, 192, 128), (136, 448, 200)):
        a, b = make_ab(*shape, "float16", seed=7)
        check("float16", a, b, run_native(native, "float16", a, b, cfg))
    a, b = make_ab(520, 264, 328, "bfloat16", seed=8)
    check("bfloat16", a, b, run_native(native, "bfloat16", a, b, cfg))


def test_golden_vector(native, golden):
    """A, B and the fp32 result of the reference's own GEMMTC.reference."""
    c = oracle.from_bits(run_native(native, "float16", golden["gemm_a"], golden["gemm_b"]), "float16")
    ref = golden["gemm_c32"]
    assert np.all(np.abs(c - ref) <= 2.5e-3 + 2e-3 * np.abs(ref))  # GEMMTC(64, 80, 96).tolerance


@pytest.mark.parametrize("size", [4096])
def test_full_size_against_torch_and_oracle(native, size):
    """The benchmark shape: every element against torch's fp32 GEMM of the same inputs (the
    reference's acceptance test), sampled rows against the oracle, linearity, determinism."""
    from deca_b200.operators import GEMMTC

    M = N = K = size
    g = torch.Generator(device="cpu").manual_seed(2)
    a = (torch.rand(M, K, generator=g) * 2 - 1).half().cuda()
    b = (torch.rand(K, N, generator=g) * 2 - 1).half().cuda()
    op = GEMMTC(M, N, K)
    c = op(a, b)
    torch.cuda.synchronize()
    ref = op.reference((a, b))
    atol, rtol = op.tolerance
    assert torch.all((c.float() - ref).abs() <= atol + rtol * ref.abs())
    assert torch.all((c.float() - ref).abs() <= 1e-2 + 1e-2 * ref.abs())
    assert torch.equal(op(a, b), c)
    rows = torch.randint(0, M, (8,), generator=torch.Generator().manual_seed(0)).cuda()
    check("float16", torch_to_bits(a[rows]), torch_to_bits(b), torch_to_bits(c[rows]))
    # linearity: (2A) B == 2 (A B) exactly (scaling by two is exact in fp16 and fp32) wherever
    # the result is a normal fp16 number (subnormal results round on a fixed absolute grid)
    c2 = op((a * 2).half(), b)
    normal = c.float().abs() >= 2.0**-13
    assert torch.equal(c2.float()[normal], (c.float() * 2)[normal])


def test_argument_errors(native):
    L = native.lib()
    a = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    b = torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    c = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(0)
    assert L.deca_gemm16(0, None, b.data_ptr(), c.data_ptr(), 128, 64, 64, None, st) == -1
    assert L.deca_gemm16(0, a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, 64, 64, None, st) == -2
    assert L.deca_gemm16(0, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 60, 64, None, st) == -3
    assert L.deca_gemm16(0, a.data_ptr() + 2, b.data_ptr(), c.data_ptr(), 64, 64, 64, None, st) == -3
    assert L.deca_gemm16(3, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 64, 64, None, st) == -5
    bad = native.GemmCfg(128, 96, 64, 4, 8, 1, 1, 2)
    assert L.deca_gemm16(0, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 64, 64, ctypes.byref(bad), st) == -4
    bad = native.GemmCfg(128, 256, 64, 8, 8, 1, 1, 2)  # 8 stages of 48 KB do not fit shared memory
    assert L.deca_gemm16(0, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 64, 64, ctypes.byref(bad), st) == -4
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------- stream-K mode
def run_stream_k(native, dtype, a, b, cfg_tuple, launches=2):
    """C through deca_gemm16_ws with stream_k = 1; the same zeroed workspace serves every launch."""
    M, K = a.shape
    N = b.shape[1]
    BM, BN, stages, raster, acc = cfg_tuple
    ccfg = native.GemmCfg(BM, BN, 64, stages, raster, 1, 1, acc, 1)
    L = native.lib()
    nbytes = ctypes.c_size_t(0)
    assert L.deca_gemm16_workspace_bytes(native.DTYPE_CODE[dtype], M, N, K, ctypes.byref(ccfg), ctypes.byref(nbytes)) == 0
    ws = torch.zeros(max(nbytes.value, 256), dtype=torch.uint8, device="cuda")
    outs = []
    for _ in range(launches):
        buf = torch.full((M + 2, N), 7.0, dtype=a.dtype, device="cuda")
        c = buf[1 : M + 1]
        st = L.deca_gemm16_ws(native.DTYPE_CODE[dtype], a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, ctypes.byref(ccfg),
                              ws.data_ptr(), nbytes.value, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert st == 0, native.status_string(st)
        assert native.last_device_status() == (0, 0, 0)
        assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
        outs.append(torch_to_bits(c))
    if nbytes.value:
        flags = ws[: 148 * 16].view(torch.int32)
        assert int(flags.abs().sum().item()) == 0, "ready flags not cleared by the launch"
    return outs, nbytes.value


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape,cfg", [
    ((4096, 4096, 512), (256, 256, 3, 8, 1)),    # 256 tiles on 148 SMs: every tile in the split region
    ((2048, 2048, 1024), (128, 256, 4, 8, 2)),   # 128 tiles: fewer tiles than SMs, 16 k blocks each
    ((1280, 1280, 1024), (128, 128, 4, 4, 2)),   # 100 tiles
    ((2560, 2560, 256), (128, 128, 3, 4, 2)),    # 400 tiles: one whole wave, then 252 tiles split
    ((1000, 1096, 520), (128, 128, 3, 2, 2)),    # partial tiles in M, N and K
    ((256, 256, 4096), (128, 128, 4, 1, 2)),     # 4 tiles, 64 k blocks each: many CTAs per tile
])
def test_stream_k_matches_oracle_and_plain_kernel(native, dtype, shape, cfg):
    M, N, K = shape
    a_bits, b_bits = make_ab(M, N, K, dtype, seed=5)
    a, b = bits_to_torch(a_bits, dtype), bits_to_torch(b_bits, dtype)
    outs, nbytes = run_stream_k(native, dtype, a, b, cfg)
    assert nbytes > 0, "the shape was meant to be split"
    assert np.array_equal(outs[0], outs[1]), "two launches on one workspace differ"
    check(dtype, a_bits, b_bits, outs[0])
    BM, BN, stages, raster, acc = cfg
    plain = run_native(native, dtype, a_bits, b_bits, dict(BM=BM, BN=BN, stages=stages, raster=raster, acc_bufs=acc))
    # split tiles are summed in another order in fp32: after rounding to 16 bits nearly all agree
    assert np.mean(plain == outs[0]) > 0.98


def test_stream_k_not_applied_and_argument_errors(native):
    L = native.lib()
    ccfg = native.GemmCfg(256, 256, 64, 3, 8, 1, 1, 1, 1)
    n = ctypes.c_size_t(123)
    assert L.deca_gemm16_workspace_bytes(native.F16, 8192, 8192, 8192, ctypes.byref(ccfg), ctypes.byref(n)) == 0
    assert n.value == 0  # 1024 tiles fill 6.9 waves: nothing to split
    a = torch.zeros(512, 2048, dtype=torch.float16, device="cuda")
    b = torch.zeros(2048, 512, dtype=torch.float16, device="cuda")
    c = torch.zeros(512, 512, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    small = native.GemmCfg(128, 128, 64, 3, 1, 1, 1, 2, 1)
    assert L.deca_gemm16(native.F16, a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 512, 2048, ctypes.byref(small), st) == -4
    assert L.deca_gemm16_workspace_bytes(native.F16, 512, 512, 512, ctypes.byref(small), ctypes.byref(n)) == 0
    assert n.value == 0  # 16 tiles of 8 k blocks: too little work per CTA to split
    assert L.deca_gemm16_workspace_bytes(native.F16, 512, 512, 2048, ctypes.byref(small), ctypes.byref(n)) == 0
    assert n.value == 256 * 4 + 64 * 128 * 128 * 4  # 64 CTAs: flags (rounded to 256 bytes) + one fp32 tile each
    ws = torch.zeros(n.value, dtype=torch.uint8, device="cuda")
    args = (native.F16, a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 512, 2048, ctypes.byref(small))
    assert L.deca_gemm16_ws(*args, None, 0, st) == -1
    assert L.deca_gemm16_ws(*args, ws.data_ptr(), n.value - 1, st) == -2
    assert L.deca_gemm16_ws(*args, ws.data_ptr() + 16, n.value, st) == -3
    assert L.deca_gemm16_ws(*args, ws.data_ptr(), n.value, st) == 0
    bad = native.GemmCfg(128, 128, 64, 3, 1, 1, 1, 2, 2)
    assert L.deca_gemm16_check_config(native.F16, 512, 512, 512, ctypes.byref(bad)) == -4
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)


def test_stream_k_through_the_operator(native):
    from deca_b200.kernels.gemm_b200 import GemmConfig, stream_k_plan
    from deca_b200.operators import GEMMTC

    op = GEMMTC(2048, 2048, 2048)
    cfg = GemmConfig(BM=256, BN=256, stages=3, raster=8, acc_bufs=1, stream_k=True)
    assert stream_k_plan(cfg, 2048, 2048, 2048) == (148, 0, 64 * 32)
    a, b = op.make_inputs()
    ref = op.reference((a, b))
    out = op(a, b, cfg=cfg)
    out2 = op(a, b, cfg=cfg)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    atol, rtol = op.tolerance
    assert torch.allclose(out.float(), ref.float(), atol=atol, rtol=rtol)
    assert native.last_device_status() == (0, 0, 0)


# ---------------------------------------------------------------------------- CTA pairs (cta_group::2)
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape,stages,raster", [
    ((512, 256, 64), 2, 1),       # one pair tile, one k block
    ((1024, 512, 512), 3, 2),
    ((1000, 520, 264), 4, 8),     # partial tiles in M, N and K; the odd CTA's rows partly outside M
    ((300, 256, 128), 3, 1),      # the odd CTA's 256 rows mostly outside M
    ((2048, 4096, 1024), 4, 8),   # 64 pair tiles: one wave
    ((8192, 2048, 256), 3, 4),    # 128 pair tiles: every pair runs more than one tile
])
def test_cta_pair_kernel_matches_oracle(native, dtype, shape, stages, raster):
    run_cta_pair_case(native, dtype, shape, 256, 256, stages, raster, 1)


@pytest.mark.parametrize("tile", [(128, 256, 4, 2), (128, 128, 6, 2), (256, 128, 4, 2), (128, 256, 3, 1), (128, 128, 8, 1)],
                         ids=lambda t: "x".join(map(str, t)))
@pytest.mark.parametrize("shape", [(256, 128, 64), (1000, 520, 264), (1024, 1024, 512), (4096, 384, 256)],
                         ids=lambda s: "x".join(map(str, s)))
def test_cta_pair_smaller_tiles(native, shape, tile):
    BM, BN, stages, acc = tile
    run_cta_pair_case(native, "float16", shape, BM, BN, stages, 4, acc)


def run_cta_pair_case(native, dtype, shape, BM, BN, stages, raster, acc):
    M, N, K = shape
    a_bits, b_bits = make_ab(M, N, K, dtype, seed=7)
    a, b = bits_to_torch(a_bits, dtype), bits_to_torch(b_bits, dtype)
    buf = torch.full((M + 2, N), 7.0, dtype=a.dtype, device="cuda")
    c = buf[1 : M + 1]
    ccfg = native.GemmCfg(BM, BN, 64, stages, raster, 1, 2, acc, 0)
    L = native.lib()
    assert L.deca_gemm16_check_config(native.DTYPE_CODE[dtype], M, N, K, ctypes.byref(ccfg)) == 0
    for _ in range(2):
        st = L.deca_gemm16(native.DTYPE_CODE[dtype], a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, ctypes.byref(ccfg),
                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert st == 0, native.status_string(st)
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)
    assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
    got = torch_to_bits(c)
    check(dtype, a_bits, b_bits, got)
    # same k order per element as the one-CTA kernel: identical bits
    plain = run_native(native, dtype, a_bits, b_bits, dict(BM=128, BN=128, stages=3, raster=raster, acc_bufs=2))
    assert np.array_equal(got, plain)


def test_cta_pair_config_rules(native):
    L = native.lib()

    def rc(*fields):
        return L.deca_gemm16_check_config(native.F16, 4096, 4096, 4096, ctypes.byref(native.GemmCfg(*fields)))

    assert rc(256, 256, 64, 4, 8, 1, 2, 1, 0) == 0
    assert rc(128, 256, 64, 4, 8, 1, 2, 2, 0) == 0   # 128 rows per CTA, two accumulators
    assert rc(128, 128, 64, 8, 8, 1, 2, 2, 0) == 0
    assert rc(128, 64, 64, 4, 8, 1, 2, 2, 0) == -4   # 128 or 256 columns
    assert rc(256, 256, 64, 5, 8, 1, 2, 1, 0) == -4  # five stages do not fit
    assert rc(256, 256, 64, 3, 8, 0, 2, 1, 0) == -4  # staged epilogue only
    assert rc(256, 256, 64, 3, 8, 1, 2, 2, 0) == -4  # one accumulator (all 512 columns)
    assert rc(256, 256, 64, 3, 8, 1, 2, 1, 1) == -4  # no stream-K
    assert rc(256, 256, 64, 3, 8, 1, 3, 1, 0) == -4


# ---------------------------------------------------------------------------- fp16 accumulation
@pytest.mark.parametrize("shape,tile", [((640, 768, 448), (128, 256, 4, 2)), ((1280, 1024, 1024), (256, 256, 3, 1)),
                                        ((300, 520, 4096), (128, 128, 6, 2)), ((256, 256, 16), (128, 64, 2, 2))],
                         ids=lambda v: "x".join(map(str, v)))
def test_fp16_accumulate_mode(native, shape, tile):
    """``acc_f16``: the tensor cores accumulate in fp16 (the reference's ``acc_f16`` configs,
    gemm_tir.py:52-58).  Bound: the reference's tolerance for that mode against the fp32 result,
    atol = 2e-3 * K, rtol = 1e-2 (operators/GEMMTC.py:60-62).  The mode must be a real one: with a
    deep K its results differ from the fp32-accumulating kernel's and are less accurate, while one
    16-deep step (a single MMA per output) gives the same sum up to the last bit of its rounding."""
    M, N, K = shape
    BM, BN, stages, acc = tile
    a_bits, b_bits = make_ab(M, N, K, "float16", seed=12)
    a, b = bits_to_torch(a_bits, "float16"), bits_to_torch(b_bits, "float16")
    out = {}
    for f16 in (0, 1):
        buf = torch.full((M + 2, N), 7.0, dtype=torch.float16, device="cuda")
        ccfg = native.GemmCfg(BM, BN, 64, min(stages, max(2, -(-K // 64))), 2, 1, 1, acc, 0, f16)
        rc = native.lib().deca_gemm16(native.F16, a.data_ptr(), b.data_ptr(), buf[1 : M + 1].data_ptr(), M, N, K,
                                      ctypes.byref(ccfg), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert rc == 0, native.status_string(rc)
        assert native.last_device_status() == (0, 0, 0)
        assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
        out[f16] = oracle.from_bits(torch_to_bits(buf[1 : M + 1]), "float16")
    _, c32 = oracle.gemm16(a_bits, b_bits, "float16", want_f32=True)
    err32, err16 = np.abs(out[0] - c32), np.abs(out[1] - c32)
    assert np.all(err16 <= 2e-3 * K + 1e-2 * np.abs(c32)), f"max err {err16.max()}"
    if K == 16:
        # one 16-deep step per output: the same sum, rounded to fp16 by the tensor core instead of by
        # the epilogue (the two roundings may differ in the last bit)
        assert np.all(np.abs(out[0] - out[1]) <= 2.0 ** (np.floor(np.log2(np.maximum(np.abs(c32), 2.0**-14))) - 10))
        assert np.mean(out[0] == out[1]) > 0.9
    else:
        assert err16.max() > err32.max() and np.mean(out[0] != out[1]) > 0.05, "the mode changed nothing"
        # each of the K / 16 partial sums is rounded to fp16 once: a random walk of half-ulp steps
        assert err16.max() <= 8.0 * math.sqrt(K / 16) * 2.0**-11 * max(1.0, np.abs(c32).max())


def test_fp16_accumulate_operator_and_rules(native):
    from deca_b200.kernels.gemm_b200 import GemmConfig
    from deca_b200.operators import GEMMTC

    M, N, K = 512, 512, 2048
    g = torch.Generator(device="cpu").manual_seed(3)
    a = (torch.rand(M, K, generator=g) * 2 - 1).half().cuda()
    b = (torch.rand(K, N, generator=g) * 2 - 1).half().cuda()
    op = GEMMTC(M, N, K, acc="fp16", acc_splits=1)
    assert op.describe() == "GEMMTC(M=512, N=512, K=2048, float16, acc=fp16x1)"
    c = op(a, b)
    torch.cuda.synchronize()
    ref = op.reference((a, b))
    atol, rtol = op.tolerance
    assert torch.all((c.float() - ref).abs() <= atol + rtol * ref.abs())
    assert not torch.equal(c, GEMMTC(M, N, K)(a, b))
    L = native.lib()
    rc = lambda dt, cfg: L.deca_gemm16_check_config(dt, M, N, K, ctypes.byref(cfg))  # noqa: E731
    assert rc(native.F16, native.GemmCfg(128, 256, 64, 4, 8, 1, 1, 2, 0, 1)) == 0
    assert rc(native.BF16, native.GemmCfg(128, 256, 64, 4, 8, 1, 1, 2, 0, 1)) == -4   # fp16 inputs only
    assert rc(native.F16, native.GemmCfg(128, 256, 64, 4, 8, 1, 2, 2, 0, 1)) == -4    # not on CTA pairs
    assert rc(native.F16, native.GemmCfg(128, 256, 64, 4, 8, 1, 1, 2, 1, 1)) == -4    # not with stream-K
    assert rc(native.F16, native.GemmCfg(128, 256, 64, 4, 8, 1, 1, 2, 0, 2)) == -4
    with pytest.raises(AssertionError):
        GEMMTC(M, N, K, dtype="bfloat16", acc="fp16")
    assert not op.is_valid(GemmConfig()) and op.is_valid(GemmConfig(acc_f16=True))


@pytest.mark.parametrize("shape,tile", [((2304, 640, 192), (128, 128, 3, 2)), ((4096, 1024, 256), (256, 256, 3, 1)),
                                        ((1000, 520, 136), (128, 64, 2, 2)), ((8192, 768, 128), (128, 256, 2, 2))],
                         ids=lambda v: "x".join(map(str, v)))
def test_column_band_tile_order(native, shape, tile):
    """``raster_n``: the tiles are walked in groups of tile columns down M instead of tile rows along
    N.  Only the order changes, so every output bit equals the row-group order's, for group widths
    that divide the tile grid, do not divide it, and exceed it."""
    M, N, K = shape
    BM, BN, stages, acc = tile
    a_bits, b_bits = make_ab(M, N, K, "float16", seed=15)
    a, b = bits_to_torch(a_bits, "float16"), bits_to_torch(b_bits, "float16")

    def run(raster, along_n):
        buf = torch.full((M + 2, N), 7.0, dtype=torch.float16, device="cuda")
        ccfg = native.GemmCfg(BM, BN, 64, stages, raster, 1, 1, acc, raster_n=along_n)
        rc = native.lib().deca_gemm16(native.F16, a.data_ptr(), b.data_ptr(), buf[1 : M + 1].data_ptr(), M, N, K,
                                      ctypes.byref(ccfg), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert rc == 0, native.status_string(rc)
        assert native.last_device_status() == (0, 0, 0)
        assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
        return torch_to_bits(buf[1 : M + 1])

    want = run(4, 0)
    check("float16", a_bits, b_bits, want)
    for raster in (1, 2, 3, 8, 64):
        assert np.array_equal(run(raster, 1), want), f"raster={raster}"
    pair = native.GemmCfg(128, 256, 64, 4, 4, 1, 2, 2, raster_n=1)
    assert native.lib().deca_gemm16_check_config(native.F16, M, N, K, ctypes.byref(pair)) == -4
