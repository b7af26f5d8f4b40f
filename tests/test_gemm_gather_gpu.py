"""GPU parity of the M-sharded GEMM with the all-gather fused into its epilogue
(deca_gemm16_gather), through the C ABI.

The ranks are emulated on one GPU: every rank's copy of the gathered output is a tensor of this
process, and the ranks' kernels run one after the other, each storing its shard into all
copies.  That exercises the multi-destination store path without a second GPU; the path over
NVLink differs only in where the destination addresses point.  Bar: every copy is bit-identical
to the unsharded kernel's output (same k order per element) and within the GEMM tolerance of the
oracle."""

import ctypes

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


def make_ab(M, N, K, dtype, seed=4):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.rand(M, K, generator=g) * 2 - 1
    b = torch.rand(K, N, generator=g) * 2 - 1
    return oracle.to_bits(a.numpy(), dtype), oracle.to_bits(b.numpy(), dtype)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_every_copy_holds_every_shard(native, world, dtype):
    from deca_b200.kernels.gemm_b200 import GemmConfig
    from deca_b200.sharding import GatheredOutput, gemm_gather, shard_gemm

    m_shard, N, K = 200, 328, 264  # partial tiles in every dimension
    M = world * m_shard
    a_bits, b_bits = make_ab(M, N, K, dtype)
    a, b = bits_to_torch(a_bits, dtype), bits_to_torch(b_bits, dtype)
    # canary rows around every copy
    bufs = [torch.full((M + 2, N), 7.0, dtype=a.dtype, device="cuda") for _ in range(world)]
    copies = [buf[1 : M + 1] for buf in bufs]
    cfg = GemmConfig(BM=128, BN=128, stages=3, raster=2, acc_bufs=2, epi_smem=True)
    for rank in range(world):
        a_shard, _, (m0, m1) = shard_gemm(a, b, rank, world)
        assert (m0, m1) == (rank * m_shard, (rank + 1) * m_shard)
        gemm_gather(a_shard.contiguous(), b, GatheredOutput.from_tensors(copies, rank), cfg)
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)

    full = torch.empty(M, N, dtype=a.dtype, device="cuda")
    ccfg = native.GemmCfg(128, 128, 64, 3, 2, 1, 1, 2)
    st = native.lib().deca_gemm16(native.DTYPE_CODE[dtype], a.data_ptr(), b.data_ptr(), full.data_ptr(), M, N, K,
                                  ctypes.byref(ccfg), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st == 0
    want = torch_to_bits(full)
    for buf, copy in zip(bufs, copies):
        assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
        assert np.array_equal(torch_to_bits(copy), want)
    _, c32 = oracle.gemm16(a_bits, b_bits, dtype, want_f32=True)
    err = np.abs(oracle.from_bits(want, dtype) - c32)
    assert np.all(err <= 1e-2 + 1e-2 * np.abs(c32)), f"max err {err.max()}"


def test_large_tile_config_and_default(native):
    from deca_b200.kernels.gemm_b200 import GemmConfig
    from deca_b200.sharding import GatheredOutput, gemm_gather

    world, m_shard, N, K = 2, 512, 512, 256
    a_bits, b_bits = make_ab(world * m_shard, N, K, "float16")
    a, b = bits_to_torch(a_bits, "float16"), bits_to_torch(b_bits, "float16")
    ref = (a.float() @ b.float())
    for cfg in (GemmConfig(BM=256, BN=256, stages=3, raster=1, acc_bufs=1, epi_smem=True), None):
        copies = [torch.zeros(world * m_shard, N, dtype=a.dtype, device="cuda") for _ in range(world)]
        for rank in range(world):
            gemm_gather(a[rank * m_shard : (rank + 1) * m_shard], b, GatheredOutput.from_tensors(copies, rank), cfg)
        torch.cuda.synchronize()
        assert native.last_device_status() == (0, 0, 0)
        assert torch.equal(copies[0], copies[1])
        assert (copies[0].float() - ref).abs().max().item() <= 1e-2 + 1e-2 * ref.abs().max().item()


def test_argument_errors(native):
    L = native.lib()
    a = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    b = torch.zeros(64, 128, dtype=torch.float16, device="cuda")
    c = torch.zeros(256, 128, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(ptrs, n_ranks, rank, cfg=None):
        arr = (ctypes.c_void_p * max(len(ptrs), 1))(*ptrs)
        return L.deca_gemm16_gather(native.F16, a.data_ptr(), b.data_ptr(), arr, n_ranks, rank, 128, 128, 64,
                                    ctypes.byref(cfg) if cfg is not None else None, st)

    two = [c.data_ptr(), c.data_ptr()]
    assert call(two, 2, 0) == 0
    assert call(two, 2, 2) == -2  # rank outside the world: DECA_ERR_SHAPE
    assert call(two * 5, 9, 0) == -2  # more than 8 ranks
    assert call([c.data_ptr(), None], 2, 0) == -1  # DECA_ERR_NULL
    assert L.deca_gemm16_gather(native.F16, a.data_ptr(), b.data_ptr(), None, 1, 0, 128, 128, 64, None, st) == -1
    direct = native.GemmCfg(128, 128, 64, 2, 1, 0, 1, 2)  # direct-store epilogue cannot gather
    assert call(two, 2, 0, direct) == -4  # DECA_ERR_CONFIG
    assert call([c.data_ptr()], 1, 0, direct) == 0  # ... but a single rank has no peers
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)
