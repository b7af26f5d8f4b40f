"""GPU parity at the shapes of the multi-GPU configuration: the GEMM 65536 x 8192 x 8192 split
along M (the whole problem on one GPU, and the 8192-row shard one of eight GPUs gets) and the
causal attention B32 H32 S8192 D128 split along B*H (the 128-head shard of one of eight GPUs).

GEMM: sampled rows against the CPU oracle's fp32-accumulated result (1e-2 + 1e-2 |c|), every
element against the reference's own acceptance test (fp32 torch matmul of the fp16 inputs,
operators/GEMMTC.py:92-103, tolerance :51-63).  Attention: sampled heads against the oracle
(max-abs 2e-3), every element against torch SDPA at the reference's 2e-2 (RuntimeMod.py:156-180),
and bit equality of the persistent schedule with the one-item-per-CTA kernel at 32 Q-tile pairs
per head."""

import ctypes

import numpy as np
import pytest

import oracle
from util import torch_to_bits

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def native():
    from deca_b200 import native as n

    n.lib()
    return n


def gemm_inputs(M, N, K, seed=4):
    """A, B ~ U[-1, 1] drawn on the device (a CPU draw of 65536 x 8192 takes too long); the oracle
    gets the very bits the kernel saw."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = (torch.rand(M, K, generator=g, device="cuda") * 2 - 1).half()
    b = (torch.rand(K, N, generator=g, device="cuda") * 2 - 1).half()
    return a, b


@pytest.mark.parametrize("M", [8192, 65536], ids=["shard_of_8", "whole"])
def test_gemm_config5_shapes(native, M):
    from deca_b200.operators import GEMMTC

    N = K = 8192
    a, b = gemm_inputs(M, N, K)
    op = GEMMTC(M, N, K)
    buf = torch.full((M + 2, N), 7.0, dtype=torch.float16, device="cuda")
    c = buf[1 : M + 1]
    op(a, b, out=c)
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)
    assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0), "canary rows overwritten"

    # every element: the reference's acceptance test and the stated bound, in row chunks
    atol, rtol = op.tolerance
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        b32 = b.float()
        for r0 in range(0, M, 8192):
            ref = a[r0 : r0 + 8192].float() @ b32
            err = (c[r0 : r0 + 8192].float() - ref).abs()
            assert torch.all(err <= atol + rtol * ref.abs()), f"rows {r0}..: reference bound"
            assert torch.all(err <= 1e-2 + 1e-2 * ref.abs())
            del ref, err
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev

    # 16 sampled rows (first, last, tile edges, random) against the CPU oracle
    rows = sorted({0, M - 1, 127, 128, 255, 256, M // 2} | set(
        torch.randint(0, M, (9,), generator=torch.Generator().manual_seed(0)).tolist()))
    idx = torch.tensor(rows, device="cuda")
    a_rows = torch_to_bits(a[idx])
    _, c32 = oracle.gemm16(a_rows, torch_to_bits(b), "float16", want_f32=True)
    got = c[idx].float().cpu().numpy()
    err = np.abs(got - c32)
    assert np.all(err <= 1e-2 + 1e-2 * np.abs(c32)), f"max err {err.max()}"

    # determinism, and exact linearity: (2A) B == 2 (A B) wherever the result is a normal fp16
    # number (scaling by two is exact in fp16 and fp32; subnormal results round on a fixed grid)
    c2 = op(a, b)
    assert torch.equal(c2, c)
    del c2
    a.mul_(2)
    twice = op(a, b)
    for r0 in range(0, M, 8192):
        want = c[r0 : r0 + 8192].float()
        normal = want.abs() >= 2.0**-13
        assert torch.equal(twice[r0 : r0 + 8192].float()[normal], (want * 2)[normal])


def test_attention_config5_shard(native):
    """B1 H128 S8192 D128 causal: what one of eight GPUs computes."""
    from deca_b200.kernels.flash_attn_b200 import FAConfig
    from deca_b200.operators import FlashAttention

    B, H, S, D = 1, 128, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(4)
    q, k, v = (torch.randn(B, H, S, D, generator=g, device="cuda").half() for _ in range(3))
    op = FlashAttention(B, H, S, S, D, causal=True)
    cfg = op.default_config()
    assert cfg.persistent, "the default for this shape is the persistent schedule"
    o = op(q, k, v)
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)

    # the host-chosen head sections and the longest-first order change nothing in the arithmetic
    plain = op(q, k, v, cfg=FAConfig(Bc=128, stages=cfg.stages, q_tiles=2, p_tmem=True))
    assert torch.equal(plain, o), "persistent schedule differs from one item per CTA"
    del plain
    assert torch.equal(op(q, k, v), o)

    # every element against SDPA, head chunks keep the temporaries small
    worst = 0.0
    for h0 in range(0, H, 16):
        sl = (slice(None), slice(h0, h0 + 16))
        ref = FlashAttention(B, 16, S, S, D, causal=True).reference((q[sl], k[sl], v[sl]))
        worst = max(worst, (o[sl].float() - ref.float()).abs().max().item())
        del ref
    assert worst <= 2e-2, f"max abs err vs SDPA {worst}"
    assert worst <= 4e-3  # two fp16 results, each within 2e-3 of exact

    # two heads against the oracle (first and one from the last section)
    for h in (0, 101):
        sl = (slice(0, 1), slice(h, h + 1))
        _, o32 = oracle.attention(torch_to_bits(q[sl]), torch_to_bits(k[sl]), torch_to_bits(v[sl]), causal=True,
                                  want_f32=True)
        err = np.abs(o[sl].float().cpu().numpy() - o32).max()
        assert err <= 2e-3, f"head {h}: max abs err {err}"


def test_bounded_wait_gives_up_and_reports(native):
    """A wait that nothing completes runs into its limit, reports through the device status word
    and the kernel returns: the path every pipelined kernel takes when one of its waits runs out.
    Nothing faults or hangs: the wait is 2 ms long and then over; the context stays usable."""
    L = native.lib()
    assert native.last_device_status() == (0, 0, 0)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.deca_selftest_bounded_wait(2000, st) == 0
    words = native.device_status_words(16)
    code, where, block = native.last_device_status(clear=True)
    assert (code, where, block) == (100001, 0x7E57, 0)
    assert "bounded wait" in native.status_string(code)
    waited_first, waited_second = words[4], words[5]
    assert 2000 <= waited_first < 50000, f"the limited wait took {waited_first} us"
    # the second waiter had a 1 s limit and left through the abort flag right after the first
    assert waited_second < 100000, f"the abort flag was not seen: waited {waited_second} us"
    assert native.last_device_status() == (0, 0, 0)
    # the next real launches are clean
    from deca_b200.operators import GEMMTC

    a = torch.ones(256, 128, dtype=torch.float16, device="cuda")
    b = torch.ones(128, 256, dtype=torch.float16, device="cuda")
    c = GEMMTC(256, 256, 128)(a, b)
    torch.cuda.synchronize()
    assert torch.all(c == 128.0)
    assert native.last_device_status() == (0, 0, 0)
    assert L.deca_selftest_bounded_wait(0, st) == -2 and L.deca_selftest_bounded_wait(200000, st) == -2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_one_process_two_devices(native):
    """The per-kernel attributes (dynamic shared-memory limit, status word, device info) are kept
    per device: the same process launches every family on cuda:0 and then on cuda:1."""
    from deca_b200.operators import GEMMTC, FlashAttention, Softmax

    results = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            g = torch.Generator(device="cpu").manual_seed(5)
            a = (torch.rand(512, 256, generator=g) * 2 - 1).half().cuda()
            b = (torch.rand(256, 512, generator=g) * 2 - 1).half().cuda()
            q, k, v = (torch.randn(1, 2, 512, 128, generator=g).half().cuda() for _ in range(3))
            x = torch.randn(64, 4096, generator=g).half().cuda()
            out = (GEMMTC(512, 512, 256)(a, b), FlashAttention(1, 2, 512, 512, 128, causal=True)(q, k, v),
                   Softmax(64, 4096, "fp16")(x))
            torch.cuda.synchronize()
            assert native.last_device_status() == (0, 0, 0)
            results.append([t.cpu() for t in out])
    for t0, t1 in zip(*results):
        assert torch.equal(t0, t1)
