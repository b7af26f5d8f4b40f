"""GPU parity of the row-wise kernels against the CPU oracle, through the C ABI.

Tolerance: 1e-3 relative against the oracle's fp32 value (see util.rowwise_allowed for the
rounding terms), and at most one 16-bit ulp against the oracle's rounded output."""

import ctypes

import numpy as np
import pytest

import oracle
from util import bits_to_torch, rowwise_allowed, torch_to_bits, ulp

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def native():
    from deca_b200 import native as n

    n.lib()
    return n


def make_x(M, N, dtype, seed=1, scale=3.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = scale * torch.randn(M, N, generator=g)
    w = 1.0 + 0.1 * torch.randn(N, generator=g)
    return oracle.to_bits(x.numpy(), dtype), oracle.to_bits(w.numpy(), dtype)


def run_native(native, op, dtype, x_bits, w_bits, cfg=None, eps=1e-6):
    """Calls deca_rowwise on device copies; the output sits between two canary rows."""
    M, N = x_bits.shape
    x = bits_to_torch(x_bits, dtype)
    w = bits_to_torch(w_bits, dtype) if w_bits is not None else None
    buf = torch.full((M + 2, N), 7.0, dtype=x.dtype, device="cuda")
    y = buf[1 : M + 1]
    ccfg = None
    if cfg is not None:
        ccfg = ctypes.byref(native.RowCfg(cfg["tpr"], cfg.get("rpb", 1), cfg.get("vec", 8),
                                          native.ROW_MODE_CODE[cfg.get("mode", "reg")], cfg.get("unroll", 1),
                                          int(cfg.get("hint", False))))
    st = native.lib().deca_rowwise(
        native.ROW_OP_CODE[op], native.DTYPE_CODE[dtype], x.data_ptr(), w.data_ptr() if w is not None else None,
        y.data_ptr(), M, N, ctypes.c_float(eps), ccfg, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st == 0, native.status_string(st)
    assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
    return torch_to_bits(y)


def check(op, dtype, x_bits, w_bits, y_bits, eps=1e-6):
    if op == "softmax":
        ref_bits, ref32 = oracle.softmax(x_bits, dtype, want_f32=True)
    else:
        ref_bits, ref32 = oracle.rmsnorm(x_bits, w_bits, eps, dtype, want_f32=True)
    got = oracle.from_bits(y_bits, dtype)
    err = np.abs(got - ref32)
    allowed = rowwise_allowed(ref32, dtype, op)
    assert np.all(err <= allowed), f"max excess x{(err / allowed).max():.2f}"
    ref = oracle.from_bits(ref_bits, dtype)
    assert np.all(np.abs(got - ref) <= ulp(ref, dtype) * (1.0001 if op == "softmax" else 2.0001))
    assert np.mean(y_bits == ref_bits) > (0.97 if op == "softmax" else 0.99)
    if op == "rmsnorm":  # all but the rare rounding-boundary elements meet the plain 1e-3 bound
        assert np.mean(err <= rowwise_allowed(ref32, dtype)) > 0.995


SHAPES = [(4, 4096), (3, 1000), (5, 8), (148 * 3, 1024), (64, 8192), (8, 32000), (2, 128256), (16, 2048), (7, 4104),
          (6, 1002), (9, 50), (3, 4098), (2, 2)]  # the last four: rows that are only a multiple of 2 long


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("op", ["softmax", "rmsnorm"])
@pytest.mark.parametrize("shape", SHAPES)
def test_default_config_matches_oracle(native, op, dtype, shape):
    x, w = make_x(*shape, dtype)
    y = run_native(native, op, dtype, x, w if op == "rmsnorm" else None)
    check(op, dtype, x, w, y)


CONFIGS = [
    dict(tpr=32, rpb=4), dict(tpr=64, rpb=1), dict(tpr=128, rpb=2, hint=True), dict(tpr=256, rpb=4),
    dict(tpr=512, rpb=2), dict(tpr=1024, rpb=1), dict(tpr=128, rpb=1, vec=4), dict(tpr=256, rpb=1, vec=4, hint=True),
    dict(tpr=128, mode="twopass", unroll=1), dict(tpr=128, mode="twopass", unroll=2, hint=True),
    dict(tpr=64, mode="twopass", unroll=4, rpb=4), dict(tpr=256, mode="twopass", unroll=4, vec=4),
    dict(tpr=128, mode="tma", rpb=4, unroll=4), dict(tpr=32, mode="tma", rpb=8, unroll=2),
    dict(tpr=512, mode="tma", rpb=1, unroll=3), dict(tpr=256, mode="tma", rpb=2, unroll=1),
    dict(tpr=128, mode="tma", rpb=3, unroll=2), dict(tpr=64, mode="tma", rpb=4, unroll=2),
    dict(tpr=64, mode="tma", rpb=5, unroll=2),
]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("op", ["softmax", "rmsnorm"])
@pytest.mark.parametrize("cfg", CONFIGS, ids=lambda c: ",".join(f"{k}={v}" for k, v in c.items()))
def test_configs_match_oracle(native, op, dtype, cfg):
    from deca_b200.kernels.rowwise_b200 import RowConfig, check_config

    pycfg = RowConfig(cfg["tpr"], cfg.get("rpb", 1), cfg.get("vec", 8), cfg.get("mode", "reg"), cfg.get("unroll", 1),
                      cfg.get("hint", False))
    ran = 0
    for shape in ((8, 4096), (4, 5000), (1500, 1024) if cfg.get("mode") == "tma" else (12, 1024)):
        try:  # a config that the validity rules reject for a shape is skipped, as the tuner does
            check_config(pycfg, op, *shape, dtype)
        except AssertionError:
            continue
        ran += 1
        x, w = make_x(*shape, dtype, seed=5)
        y = run_native(native, op, dtype, x, w if op == "rmsnorm" else None, cfg)
        check(op, dtype, x, w, y)
    assert ran >= 1


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_golden_vectors(native, golden, dtype):
    """Against the outputs of the reference's own torch code, with the reference's tolerance
    (operators/Rowwise.py:15-20)."""
    for tag in ("hid", "ragged", "vocab"):
        x = golden[f"row_{tag}_{dtype}_x"]
        ref = oracle.from_bits(golden[f"row_{tag}_{dtype}_softmax"], dtype)
        got = oracle.from_bits(run_native(native, "softmax", dtype, x, None), dtype)
        rtol = 1e-2 if dtype == "float16" else 3e-2
        assert np.all(np.abs(got - ref) <= 1e-5 + rtol * np.abs(ref))
        assert np.all(np.abs(got - ref) <= ulp(ref, dtype) * 1.0001)
        if tag == "vocab":
            continue
        w = golden[f"row_{tag}_{dtype}_w"]
        ref = oracle.from_bits(golden[f"row_{tag}_{dtype}_rmsnorm"], dtype)
        got = oracle.from_bits(run_native(native, "rmsnorm", dtype, x, w), dtype)
        tol = 1e-2 if dtype == "float16" else 3e-2
        assert np.all(np.abs(got - ref) <= tol + tol * np.abs(ref))
        assert np.all(np.abs(got - ref) <= 1.5 * ulp(ref, dtype))


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_full_size_properties(native, dtype):
    """The benchmark shape X[16384, 4096]: size-independent properties on every row, the
    oracle on a sample of rows, and bit-identical reruns."""
    M, N = 16384, 4096
    g = torch.Generator(device="cpu").manual_seed(1)
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
    x = (3.0 * torch.randn(M, N, generator=g)).to(tdt).cuda()
    w = (1.0 + 0.1 * torch.randn(N, generator=g)).to(tdt).cuda()
    from deca_b200.operators import RMSNorm, Softmax

    sm, rn = Softmax(M, N, dtype), RMSNorm(M, N, dtype, 1e-6)
    y = sm(x)
    torch.cuda.synchronize()
    yf = y.float()
    assert torch.all(yf >= 0)
    assert torch.allclose(yf.sum(-1), torch.ones(M, device="cuda"), atol=4e-3 if dtype == "float16" else 2e-2)
    assert torch.equal(yf.argmax(-1), x.float().argmax(-1)) or torch.all(
        x.float().gather(1, yf.argmax(-1, keepdim=True)) == x.float().max(-1, keepdim=True).values)
    # softmax is invariant to a per-row shift that is exact in the 16-bit type
    assert torch.equal(sm(x), y)
    z = rn(x, w)
    torch.cuda.synchronize()
    assert torch.equal(rn(x, w), z)
    # RMSNorm is homogeneous of degree 0 in x for power-of-two scales (eps aside)
    z2 = rn((x.float() * 2).to(tdt), w)
    assert (z2.float() - z.float()).abs().max().item() <= 2e-2 * z.float().abs().max().item()
    rows = torch.randint(0, M, (48,), generator=torch.Generator().manual_seed(0))
    xb, wb = torch_to_bits(x[rows.cuda()]), torch_to_bits(w)
    check("softmax", dtype, xb, None, torch_to_bits(y[rows.cuda()]))
    check("rmsnorm", dtype, xb, wb, torch_to_bits(z[rows.cuda()]))
    # and the reference's own acceptance test: eager torch within its tolerance table
    for op, out, inputs in ((sm, y, (x,)), (rn, z, (x, w))):
        ref = op.reference(inputs).float()
        atol, rtol = op.tolerance
        assert torch.all((out.float() - ref).abs() <= atol + rtol * ref.abs())


def test_no_wait_timed_out(native):
    """The bounded waits of the bulk-copy kernels never ran out in the runs above."""
    x, w = make_x(2048, 4096, "float16", seed=9)
    y = run_native(native, "softmax", "float16", x, None, dict(tpr=128, mode="tma", rpb=4, unroll=4))
    check("softmax", "float16", x, None, y)
    assert native.last_device_status(clear=False) == (0, 0, 0)


def test_edge_values(native):
    """Rows with -inf entries, constant rows and a large dynamic range."""
    N = 1024
    x = np.zeros((4, N), np.float32)
    x[0, :] = 5.0
    x[1, :] = -np.inf
    x[1, 7] = 1.0
    x[2, :] = np.linspace(-60000, 60000, N)
    x[3, ::2] = -np.inf
    for dtype in ("float16", "bfloat16"):
        xb = oracle.to_bits(x, dtype)
        y = oracle.from_bits(run_native(native, "softmax", dtype, xb, None), dtype)
        ref = oracle.from_bits(oracle.softmax(xb, dtype), dtype)
        assert np.all(np.abs(y - ref) <= ulp(ref, dtype) * 1.0001)
        assert y[1, 7] == 1.0 and y[1].sum() == 1.0


def test_argument_errors(native):
    L = native.lib()
    x = torch.zeros(8, 64, dtype=torch.float16, device="cuda")
    y = torch.empty_like(x)
    st = ctypes.c_void_p(0)
    f = ctypes.c_float(1e-6)
    assert L.deca_rowwise(0, 0, None, None, y.data_ptr(), 8, 64, f, None, st) == -1
    assert L.deca_rowwise(1, 0, x.data_ptr(), None, y.data_ptr(), 8, 64, f, None, st) == -1
    assert L.deca_rowwise(0, 0, x.data_ptr(), None, y.data_ptr(), 0, 64, f, None, st) == -2
    assert L.deca_rowwise(0, 0, x.data_ptr() + 2, None, y.data_ptr(), 4, 64, f, None, st) == -3
    assert L.deca_rowwise(0, 7, x.data_ptr(), None, y.data_ptr(), 8, 64, f, None, st) == -5
    bad = native.RowCfg(48, 1, 8, 0, 1, 0)
    assert L.deca_rowwise(0, 0, x.data_ptr(), None, y.data_ptr(), 8, 64, f, ctypes.byref(bad), st) == -4
    bad = native.RowCfg(32, 3, 8, 0, 1, 0)  # rows_per_block does not divide M
    assert L.deca_rowwise(0, 0, x.data_ptr(), None, y.data_ptr(), 8, 64, f, ctypes.byref(bad), st) == -4
    torch.cuda.synchronize()


# ------------------------------------------------------------------ row statistics (fp32 path)
def run_native_stats(native, op, dtype, x_bits, w_bits, cfg=None, eps=1e-6):
    """deca_rowwise_stats: the outputs plus the two fp32 statistics per row the kernel reduced to."""
    M, N = x_bits.shape
    x = bits_to_torch(x_bits, dtype)
    w = bits_to_torch(w_bits, dtype) if w_bits is not None else None
    y = torch.empty_like(x)
    stats = torch.full((M, 2), float("nan"), dtype=torch.float32, device="cuda")
    ccfg = None
    if cfg is not None:
        ccfg = ctypes.byref(native.RowCfg(cfg["tpr"], cfg.get("rpb", 1), cfg.get("vec", 8),
                                          native.ROW_MODE_CODE[cfg.get("mode", "reg")], cfg.get("unroll", 1),
                                          int(cfg.get("hint", False))))
    st = native.lib().deca_rowwise_stats(
        native.ROW_OP_CODE[op], native.DTYPE_CODE[dtype], x.data_ptr(), w.data_ptr() if w is not None else None,
        y.data_ptr(), stats.data_ptr(), M, N, ctypes.c_float(eps), ccfg,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st == 0, native.status_string(st)
    return torch_to_bits(y), stats.cpu().numpy()


STATS_CONFIGS = [None, dict(tpr=64, rpb=2), dict(tpr=256, mode="twopass", unroll=2), dict(tpr=128, vec=4, hint=True)]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("cfg", STATS_CONFIGS, ids=lambda c: "default" if c is None else ",".join(f"{k}={v}" for k, v in c.items()))
def test_rmsnorm_fp32_statistic_and_exact_rounding(native, dtype, cfg):
    """The only fp32 quantity of RMSNorm is r = rsqrt(mean(x^2) + eps): it must match an exact
    (float64) computation to 1e-3 relative -- it does to 5e-6 -- and, given the kernel's own r, EVERY
    output bit must follow from the reference's rounding sequence dt(f32(dt(x * r)) * w)
    (rowwise_tir.py:340-350).  This is the 1e-3 bound without any 16-bit rounding term."""
    eps = 1e-6
    for shape, scale in (((512, 4096), 3.0), ((34, 1000), 0.01), ((8, 16384), 40.0)):
        x_bits, w_bits = make_x(*shape, dtype, seed=13, scale=scale)
        y_bits, stats = run_native_stats(native, "rmsnorm", dtype, x_bits, w_bits, cfg, eps)
        assert np.array_equal(y_bits, run_native(native, "rmsnorm", dtype, x_bits, w_bits, cfg, eps)), "same kernel, same bits"
        x32, w32 = oracle.from_bits(x_bits, dtype), oracle.from_bits(w_bits, dtype)
        x64 = x32.astype(np.float64)
        r_exact = 1.0 / np.sqrt((x64 * x64).mean(axis=1) + eps)
        r = stats[:, 0]
        assert np.all(np.abs(r - r_exact) <= 5e-6 * r_exact), f"rsqrt off by {(np.abs(r - r_exact) / r_exact).max():.2e}"
        assert np.all(np.abs(stats[:, 1] - (x64 * x64).sum(axis=1)) <= 5e-6 * (x64 * x64).sum(axis=1))
        normed = oracle.from_bits(oracle.to_bits(x32 * r[:, None].astype(np.float32), dtype), dtype)
        want_bits = oracle.to_bits(normed * w32[None, :], dtype)
        assert np.array_equal(y_bits, want_bits), f"{np.mean(y_bits != want_bits):.2e} of the outputs differ"


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("cfg", STATS_CONFIGS, ids=lambda c: "default" if c is None else ",".join(f"{k}={v}" for k, v in c.items()))
def test_softmax_fp32_statistics_and_rounding(native, dtype, cfg):
    """Softmax reduces a row to (max * log2 e, 1 / sum of exponentials): the first is exact, the second
    must match a float64 computation to 1e-3 relative (it does to 1e-5); given them, every output is
    the correctly rounded 16-bit value of exp2(x * log2 e - max * log2 e) / sum up to the 2^-22
    accuracy of the hardware exponential (rowwise_tir.py:279-300)."""
    for shape, scale in (((512, 4096), 3.0), ((34, 1000), 0.3), ((4, 32000), 6.0)):
        if cfg is not None and cfg.get("mode", "reg") == "reg" and shape[1] > 32 * cfg["tpr"] * cfg.get("vec", 8):
            continue  # the row does not fit this config's registers
        x_bits, _ = make_x(*shape, dtype, seed=17, scale=scale)
        y_bits, stats = run_native_stats(native, "softmax", dtype, x_bits, None, cfg)
        assert np.array_equal(y_bits, run_native(native, "softmax", dtype, x_bits, None, cfg))
        assert_softmax_follows_stats(x_bits, y_bits, stats, dtype)


def assert_softmax_follows_stats(x_bits, y_bits, stats, dtype):
    """Row max * log2(e) exact, 1 / sum within 1e-5 of float64, and every output the correctly rounded
    16-bit value of exp2(x * log2 e - max * log2 e) / sum up to the fp32 accuracy of the exponential."""
    x32 = oracle.from_bits(x_bits, dtype)
    log2e = np.float32(1.4426950408889634)
    ml = x32.max(axis=1) * log2e
    assert np.array_equal(stats[:, 0], ml), "row max * log2(e) is an exact fp32 product"
    x64 = x32.astype(np.float64)
    s_exact = np.exp2(x64 * float(log2e) - ml.astype(np.float64)[:, None]).sum(axis=1)
    inv = stats[:, 1].astype(np.float64)
    assert np.all(np.abs(inv * s_exact - 1.0) <= 1e-5), f"1/sum off by {np.abs(inv * s_exact - 1).max():.2e}"
    arg = (x32 * log2e - ml[:, None]).astype(np.float64)  # fma in the kernel: within half an fp32 ulp of this
    y_exact = np.exp2(arg) * inv[:, None]
    got = oracle.from_bits(y_bits, dtype).astype(np.float64)
    # half a 16-bit ulp of rounding + the fp32 error of the exponential and of its argument
    slack = 0.5 * ulp(y_exact, dtype) * 1.0001 + 1e-5 * y_exact + (3e-8 if dtype == "float16" else 0.0)
    assert np.all(np.abs(got - y_exact) <= slack), f"max excess x{(np.abs(got - y_exact) / slack).max():.3f}"


def test_stats_argument_errors(native):
    L = native.lib()
    x = torch.zeros(8, 1024, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(0)
    eps = ctypes.c_float(1e-6)
    assert L.deca_rowwise_stats(0, 0, x.data_ptr(), None, x.data_ptr(), None, 8, 1024, eps, None, st) == -1
    stats = torch.zeros(8, 2, device="cuda")
    tma = native.RowCfg(128, 2, 8, native.ROW_TMA, 2, 0)
    assert L.deca_rowwise_stats(0, 0, x.data_ptr(), None, x.data_ptr(), stats.data_ptr(), 8, 1024, eps, ctypes.byref(tma), st) == -5
    torch.cuda.synchronize()


# ------------------------------------------------------------------ cluster mode (long rows, one pass)
CLUSTER_CASES = [((64, 32000), dict(tpr=512, mode="cluster", unroll=2, hint=True)),
                 ((64, 32000), dict(tpr=256, mode="cluster", unroll=4)),
                 ((16, 128256), dict(tpr=512, mode="cluster", unroll=8, hint=True)),
                 ((16, 128256), dict(tpr=1024, mode="cluster", unroll=4, vec=4)),
                 ((32, 65536), dict(tpr=1024, mode="cluster", unroll=8)),
                 ((9, 16392), dict(tpr=256, mode="cluster", unroll=2)),      # slices end inside a vector stride
                 ((5, 1000), dict(tpr=32, mode="cluster", unroll=4)),        # short rows: most CTAs nearly idle
                 ((3, 24), dict(tpr=32, mode="cluster", unroll=8, vec=2))]   # more CTAs than vectors


@pytest.mark.parametrize("op", ["softmax", "rmsnorm"])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape,cfg", CLUSTER_CASES, ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else ",".join(f"{k}={x}" for k, x in v.items()))
def test_cluster_mode_matches_oracle(native, op, dtype, shape, cfg):
    """A thread-block cluster shares a row: each CTA caches a slice in registers and the row maximum /
    sums are combined through distributed shared memory.  Same arithmetic as the register mode: checked
    against the oracle, and the fp32 row statistics against float64."""
    x_bits, w_bits = make_x(*shape, dtype, seed=23)
    w = w_bits if op == "rmsnorm" else None
    y_bits = run_native(native, op, dtype, x_bits, w, cfg)
    y2, stats = run_native_stats(native, op, dtype, x_bits, w, cfg)
    assert np.array_equal(y2, y_bits)
    x32 = oracle.from_bits(x_bits, dtype)
    x64 = x32.astype(np.float64)
    if op == "rmsnorm":
        # the row statistic against float64, then every output bit from the kernel's own statistic by
        # the reference's rounding sequence (a comparison with the oracle's rounded outputs would
        # also see the rare element whose intermediate rounding flips with the last bit of r)
        _, ref32 = oracle.rmsnorm(x_bits, w_bits, 1e-6, dtype, want_f32=True)
        err = np.abs(oracle.from_bits(y_bits, dtype) - ref32)
        # three 16-bit ulps here instead of two: over millions of elements of long rows the intermediate
        # rounding flips where x * r lies one binade above the output (2 |w| output ulps) and the final
        # rounding adds up to one more; the exact check below is the binding one
        assert np.all(err <= 1e-3 * np.abs(ref32) + 3.0 * ulp(ref32, dtype))
        r_exact = 1.0 / np.sqrt((x64 * x64).mean(axis=1) + 1e-6)
        r = stats[:, 0]
        assert np.all(np.abs(r - r_exact) <= 5e-6 * r_exact)
        normed = oracle.from_bits(oracle.to_bits(x32 * r[:, None].astype(np.float32), dtype), dtype)
        assert np.array_equal(y_bits, oracle.to_bits(normed * oracle.from_bits(w_bits, dtype)[None, :], dtype))
    else:
        # against the oracle's fp32 value, and exactly from the kernel's own statistics (the oracle's
        # rounded outputs sum 128 Ki terms sequentially in fp32, which is less accurate than the kernel)
        _, ref32 = oracle.softmax(x_bits, dtype, want_f32=True)
        err = np.abs(oracle.from_bits(y_bits, dtype) - ref32)
        assert np.all(err <= rowwise_allowed(ref32, dtype) + 1e-4 * np.abs(ref32))
        assert_softmax_follows_stats(x_bits, y_bits, stats, dtype)


def test_cluster_mode_equals_register_mode_bits(native):
    """Where a row fits both modes the outputs are identical up to the summation order of the row
    statistic (softmax: the same maximum, sums within rounding; in practice the same bits in > 99 %)."""
    x_bits, w_bits = make_x(128, 8192, "float16", seed=29)
    for op, w in (("softmax", None), ("rmsnorm", w_bits)):
        reg = run_native(native, op, "float16", x_bits, w, dict(tpr=256, mode="reg"))
        clu = run_native(native, op, "float16", x_bits, w, dict(tpr=256, mode="cluster", unroll=4))
        assert np.mean(reg == clu) > 0.99
        a, b = oracle.from_bits(reg, "float16"), oracle.from_bits(clu, "float16")
        assert np.all(np.abs(a - b) <= ulp(a, "float16") * 1.0001)


def test_cluster_config_rules(native):
    L = native.lib()

    def rc(M, N, *fields):
        return L.deca_rowwise_check_config(0, 0, M, N, ctypes.byref(native.RowCfg(*fields)))

    assert rc(1024, 128256, 512, 1, 8, native.ROW_CLUSTER, 8, 1) == 0
    assert rc(1024, 128256, 512, 1, 8, native.ROW_CLUSTER, 3, 1) == -4   # clusters of 2, 4 or 8
    assert rc(1024, 128256, 512, 2, 8, native.ROW_CLUSTER, 8, 1) == -4   # one row per cluster
    assert rc(1024, 128256, 128, 1, 8, native.ROW_CLUSTER, 2, 1) == -4   # the slice does not fit the registers
    assert rc(1024, 128256, 48, 1, 8, native.ROW_CLUSTER, 8, 1) == -4
    from deca_b200.kernels.rowwise_b200 import RowConfig, check_config

    check_config(RowConfig(512, 1, 8, "cluster", 8, True), "softmax", 1024, 128256, "float16")
    with pytest.raises(AssertionError):
        check_config(RowConfig(128, 1, 8, "cluster", 2), "softmax", 1024, 128256, "float16")
    assert str(RowConfig(512, 1, 8, "cluster", 8, True)) == "tpr=512,rpb=1,vec=8,mode=cluster,unroll=8,hint=1"
