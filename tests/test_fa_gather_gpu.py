"""GPU parity of the head-sharded FlashAttention with the all-gather of O fused into its
epilogue (deca_fa_fwd_f16_gather), through the C ABI.  The ranks are emulated on one GPU as in
test_gemm_gather_gpu.py: every rank's copy of the gathered output is a tensor of this process and
the ranks' kernels run one after the other.  Bar: every copy is bit-identical to the unsharded
kernel's output (heads are independent), which itself is within 2e-3 of the oracle."""

import ctypes

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def native():
    from deca_b200 import native as n

    n.lib()
    return n


@pytest.mark.parametrize("world", [1, 2, 3])
@pytest.mark.parametrize("D,causal,cfg", [
    (128, False, dict(Bc=128, stages=4, q_tiles=2, p_tmem=True)),
    (128, True, dict(Bc=128, stages=4, q_tiles=2, p_tmem=True)),
    (64, True, dict(Bc=64, stages=2, q_tiles=1, p_tmem=True)),
    (64, False, dict(Bc=128, stages=2, q_tiles=1, p_tmem=False)),
])
def test_every_copy_holds_every_head(native, world, D, causal, cfg):
    from deca_b200.kernels.flash_attn_b200 import FAConfig
    from deca_b200.operators import FlashAttention
    from deca_b200.sharding import GatheredOutput, attention_gather, shard_attention

    B, H, S = 1, 2 * world, 512
    g = torch.Generator(device="cpu").manual_seed(3)
    q, k, v = (torch.randn(B, H, S, D, generator=g).half().cuda() for _ in range(3))
    fcfg = FAConfig(**cfg)
    bufs = [torch.full((B * H * S + 2, D), 7.0, dtype=torch.float16, device="cuda") for _ in range(world)]
    copies = [buf[1 : B * H * S + 1] for buf in bufs]
    for rank in range(world):
        qs, ks, vs, (h0, h1) = shard_attention(q, k, v, rank, world)
        assert (h0, h1) == (2 * rank, 2 * rank + 2)
        attention_gather(qs.contiguous(), ks.contiguous(), vs.contiguous(), GatheredOutput.from_tensors(copies, rank),
                         causal=causal, cfg=fcfg)
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)
    want = FlashAttention(B, H, S, S, D, causal=causal)(q, k, v, cfg=fcfg)
    torch.cuda.synchronize()
    for buf, copy in zip(bufs, copies):
        assert torch.all(buf[0] == 7.0) and torch.all(buf[-1] == 7.0), "canary rows overwritten"
        assert torch.equal(copy.view(B, H, S, D), want)
    # one head against the oracle
    bits = [t[:1, :1].cpu().numpy().view(np.uint16) for t in (q, k, v)]
    ref = oracle.attention(*bits, D ** -0.5, causal)
    got = want[:1, :1].float().cpu().numpy()
    assert np.abs(got - oracle.from_bits(ref, "float16")).max() <= 2e-3


def test_argument_errors(native):
    L = native.lib()
    q = torch.zeros(1, 1, 256, 64, dtype=torch.float16, device="cuda")
    o = torch.zeros(2 * 256, 64, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    cfg = native.FaCfg(128, 64, 2, 1, 0)

    def call(ptrs, n_ranks, rank):
        arr = (ctypes.c_void_p * max(len(ptrs), 1))(*ptrs)
        return L.deca_fa_fwd_f16_gather(q.data_ptr(), q.data_ptr(), q.data_ptr(), arr, n_ranks, rank, 1, 1, 256, 256, 64,
                                        ctypes.c_float(0.125), 0, ctypes.byref(cfg), st)

    two = [o.data_ptr(), o.data_ptr()]
    assert call(two, 2, 1) == 0
    assert call(two, 2, 2) == -2
    assert call(two * 5, 9, 0) == -2
    assert call([o.data_ptr(), None], 2, 0) == -1
    torch.cuda.synchronize()
    assert native.last_device_status() == (0, 0, 0)
