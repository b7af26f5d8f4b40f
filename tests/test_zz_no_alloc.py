"""deca_gemm16_sk_static: the stream-K GEMM on scratch memory built into the library, through
the C ABI.  It must give the bits of deca_gemm16_ws (same split, same arithmetic) on two calls in
a row (the second call finds the ready flags of the first still in the scratch array, which is
never cleared, and must not take them for its own), leave the device's free memory untouched,
and refuse problems beyond its fixed buffer.
The file is collected last so that it also runs after every other test has used the library."""

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


def make_ab(M, N, K, dtype, seed=6):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.rand(M, K, generator=g) * 2 - 1
    b = torch.rand(K, N, generator=g) * 2 - 1
    return oracle.to_bits(a.numpy(), dtype), oracle.to_bits(b.numpy(), dtype)


@pytest.mark.parametrize("dtype,shape,tile", [
    ("float16", (2048, 2048, 1024), (128, 256, 4, 8, 2)),
    ("bfloat16", (1280, 1280, 1024), (128, 128, 4, 4, 2)),
    ("float16", (1000, 1096, 520), (128, 128, 3, 2, 2)),
    # fewer tiles than SMs and a deep K: every tile is cut into several shares, so a head adds the
    # partial tiles of several tails (the first through the shared-memory staging path)
    ("float16", (512, 512, 2048), (128, 128, 3, 1, 2)),
    ("bfloat16", (256, 384, 4096), (128, 128, 4, 1, 2)),
])
def test_matches_caller_workspace_entry_point(native, dtype, shape, tile):
    L = native.lib()
    M, N, K = shape
    BM, BN, stages, raster, acc = tile
    a_bits, b_bits = make_ab(M, N, K, dtype)
    a, b = bits_to_torch(a_bits, dtype), bits_to_torch(b_bits, dtype)
    ccfg = native.GemmCfg(BM, BN, 64, stages, raster, 1, 1, acc, 1)
    code = native.DTYPE_CODE[dtype]
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    nbytes = ctypes.c_size_t(0)
    assert L.deca_gemm16_workspace_bytes(code, M, N, K, ctypes.byref(ccfg), ctypes.byref(nbytes)) == 0
    assert nbytes.value > 0, "the shape was meant to be split"
    ws = torch.zeros(nbytes.value, dtype=torch.uint8, device="cuda")
    want = torch.empty(M, N, dtype=a.dtype, device="cuda")
    assert L.deca_gemm16_ws(code, a.data_ptr(), b.data_ptr(), want.data_ptr(), M, N, K, ctypes.byref(ccfg), ws.data_ptr(),
                            nbytes.value, st) == 0
    torch.cuda.synchronize()
    want_bits = torch_to_bits(want)

    bufs = [torch.full((M + 2, N), 7.0, dtype=a.dtype, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    free_before = None
    for i, buf in enumerate(bufs):  # two calls in a row on one stream
        c = buf[1 : M + 1]
        rc = L.deca_gemm16_sk_static(code, a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, ctypes.byref(ccfg), st)
        assert rc == 0, native.status_string(rc)
        if i == 0:
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]  # after the set-up call
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "a call changed the device's free memory"
    assert native.last_device_status() == (0, 0, 0)
    for buf in bufs:
        assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"
        assert np.array_equal(torch_to_bits(buf[1 : M + 1]), want_bits)
    _, c32 = oracle.gemm16(a_bits, b_bits, dtype, want_f32=True)
    err = np.abs(oracle.from_bits(want_bits, dtype) - c32)
    assert np.all(err <= 1e-2 + 1e-2 * np.abs(c32)), f"max err {err.max()}"


def test_limits_are_refused(native):
    L = native.lib()
    g = torch.Generator(device="cpu").manual_seed(9)
    a = (torch.rand(512, 2048, generator=g) * 2 - 1).half().cuda()
    b = (torch.rand(2048, 512, generator=g) * 2 - 1).half().cuda()
    c = torch.full((512, 512), 7.0, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (native.F16, a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 512, 2048)
    big = native.GemmCfg(256, 256, 64, 3, 1, 1, 1, 1, 1)  # a 256 x 256 fp32 tile per CTA does not fit
    rc = L.deca_gemm16_sk_static(*args, ctypes.byref(big), st)
    assert rc == -6 and "scratch" in native.status_string(rc)
    whole = native.GemmCfg(128, 128, 64, 3, 1, 1, 1, 2, 0)  # not a stream-K config
    assert L.deca_gemm16_sk_static(*args, ctypes.byref(whole), st) == -4
    assert L.deca_gemm16_sk_static(*args, None, st) == -1
    torch.cuda.synchronize()
    assert torch.all(c == 7.0), "a refused call wrote to C"
    ok = native.GemmCfg(128, 128, 64, 3, 1, 1, 1, 2, 1)
    assert L.deca_gemm16_sk_static(*args, ctypes.byref(ok), st) == 0
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    assert torch.all((c.float() - ref).abs() <= 1e-2 + 1e-2 * ref.abs())
    assert native.last_device_status() == (0, 0, 0)
