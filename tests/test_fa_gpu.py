"""GPU parity of the FlashAttention forward kernel against the CPU oracle, through the C ABI.

Tolerance: max-abs 2e-3 against the oracle's fp32 softmax(scale QK^T + mask) V (the stated
bound for fp16); the reference's own acceptance test (max-abs 2e-2 against torch SDPA,
RuntimeMod.py:156-180) is checked at the benchmark shape."""

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


def make_qkv(B, H, S_q, S_kv, D, seed=3):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, H, S_q, D, generator=g)
    k = torch.randn(B, H, S_kv, D, generator=g)
    v = torch.randn(B, H, S_kv, D, generator=g)
    return tuple(oracle.to_bits(t.numpy(), "float16") for t in (q, k, v))


def run_native(native, q_bits, k_bits, v_bits, causal, scale=None, cfg=None):
    B, H, S_q, D = q_bits.shape
    S_kv = k_bits.shape[2]
    q, k, v = (bits_to_torch(t, "float16") for t in (q_bits, k_bits, v_bits))
    o = torch.full_like(q, 7.0)
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    ccfg = None
    if cfg is not None:
        ccfg = ctypes.byref(native.FaCfg(128, cfg.get("Bc", 128), cfg.get("stages", 2), cfg.get("q_tiles", 1), cfg.get("p_tmem", 0),
                                         cfg.get("persistent", 0)))
    st = native.lib().deca_fa_fwd_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, S_q, S_kv, D,
                                      ctypes.c_float(scale), int(causal), ccfg,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st == 0, native.status_string(st)
    assert native.last_device_status() == (0, 0, 0)
    return torch_to_bits(o)


def check(q, k, v, o_bits, causal, scale=None):
    _, o32 = oracle.attention(q, k, v, scale=scale, causal=causal, want_f32=True)
    got = oracle.from_bits(o_bits, "float16")
    err = np.abs(got - o32).max()
    assert err <= 2e-3, f"max abs err {err}"


SHAPES = [(1, 2, 128, 128, 64), (1, 1, 256, 256, 128), (2, 3, 512, 512, 128), (1, 2, 384, 384, 64),
          (1, 1, 1024, 1024, 128), (3, 1, 128, 128, 128)]


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_default_config_matches_oracle(native, shape, causal):
    q, k, v = make_qkv(*shape)
    check(q, k, v, run_native(native, q, k, v, causal), causal)


def test_cross_attention_lengths(native):
    """S_q != S_kv (non-causal), and a non-default softmax scale."""
    q, k, v = make_qkv(1, 2, 128, 640, 128, seed=11)
    check(q, k, v, run_native(native, q, k, v, False), False)
    q, k, v = make_qkv(1, 1, 512, 128, 64, seed=12)
    check(q, k, v, run_native(native, q, k, v, False, scale=0.3), False, scale=0.3)


@pytest.mark.parametrize("cfg", [dict(Bc=64, stages=1), dict(Bc=64, stages=3), dict(Bc=128, stages=1), dict(Bc=64, stages=4),
                                 dict(Bc=128, stages=3, q_tiles=2), dict(Bc=128, stages=2, q_tiles=2),
                                 dict(Bc=128, stages=6, q_tiles=2), dict(Bc=128, stages=4, q_tiles=2, p_tmem=1),
                                 dict(Bc=128, stages=2, q_tiles=2, p_tmem=1), dict(Bc=128, stages=5, q_tiles=2, p_tmem=1),
                                 dict(Bc=128, stages=3, p_tmem=1), dict(Bc=64, stages=2, p_tmem=1), dict(Bc=128, stages=1, p_tmem=1),
                                 dict(Bc=64, stages=4, q_tiles=2, p_tmem=1), dict(Bc=64, stages=8, q_tiles=2, p_tmem=1),
                                 dict(Bc=64, stages=5, q_tiles=2, p_tmem=1),
                                 dict(Bc=128, stages=4, q_tiles=2, p_tmem=1, persistent=1),
                                 dict(Bc=128, stages=2, q_tiles=2, p_tmem=1, persistent=1),
                                 dict(Bc=128, stages=3, q_tiles=2, p_tmem=1, persistent=1)],
                         ids=lambda c: ",".join(f"{k}={v}" for k, v in c.items()))
def test_configs_match_oracle(native, cfg):
    for D in (64, 128):
        S = 768 if cfg.get("q_tiles", 1) == 2 else 640
        if native.lib().deca_fa_fwd_f16_check_config(1, 2, S, S, D, 1, ctypes.byref(
                native.FaCfg(128, cfg["Bc"], cfg["stages"], cfg.get("q_tiles", 1), cfg.get("p_tmem", 0),
                             cfg.get("persistent", 0)))) != 0:
            continue
        q, k, v = make_qkv(1, 2, S, S, D, seed=5)
        for causal in (False, True):
            check(q, k, v, run_native(native, q, k, v, causal, cfg=cfg), causal)


def test_large_scores_and_rescale(native):
    """Scores with a large spread force the running-max rescale path on late KV tiles."""
    g = torch.Generator(device="cpu").manual_seed(21)
    B, H, S, D = 1, 1, 512, 64
    q = torch.randn(B, H, S, D, generator=g)
    k = torch.randn(B, H, S, D, generator=g)
    k[:, :, 300:] *= 6.0  # later keys dominate: max jumps by far more than 2^8
    v = torch.randn(B, H, S, D, generator=g)
    qb, kb, vb = (oracle.to_bits(t.numpy(), "float16") for t in (q, k, v))
    for causal in (False, True):
        check(qb, kb, vb, run_native(native, qb, kb, vb, causal, scale=1.0), causal, scale=1.0)


@pytest.mark.parametrize("tag", ["d64", "d128"])
def test_golden_vectors(native, golden, tag):
    """Q, K, V and the outputs of the reference's own torch code (SDPA, flash backend on CPU)."""
    q, k, v = (golden[f"attn_{tag}_{n}"] for n in "qkv")
    for causal in (False, True):
        ref = oracle.from_bits(golden[f"attn_{tag}_o_{'causal' if causal else 'full'}"], "float16")
        got = oracle.from_bits(run_native(native, q, k, v, causal), "float16")
        assert np.abs(got - ref).max() <= 2e-3


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_full_size(native, D, causal):
    """B=4 H=16 S=4096: every element against torch SDPA (the reference's acceptance test, 2e-2),
    one head against the oracle (2e-3), determinism, and invariance to a permutation of the keys
    (non-causal)."""
    from deca_b200.operators import FlashAttention

    B, H, S = 4, 16, 4096
    g = torch.Generator(device="cpu").manual_seed(3)
    q, k, v = (torch.randn(B, H, S, D, generator=g).half().cuda() for _ in range(3))
    op = FlashAttention(B, H, S, S, D, causal=causal)
    o = op(q, k, v)
    torch.cuda.synchronize()
    ref = op.reference((q, k, v))
    assert (o.float() - ref.float()).abs().max().item() <= 2e-2
    assert (o.float() - ref.float()).abs().max().item() <= 4e-3  # two fp16 results, each within 2e-3 of exact
    assert torch.equal(op(q, k, v), o)
    b, h = 2, 5
    sl = (slice(b, b + 1), slice(h, h + 1))
    check(torch_to_bits(q[sl]), torch_to_bits(k[sl]), torch_to_bits(v[sl]), torch_to_bits(o[sl]), causal)
    if not causal:
        perm = torch.randperm(S, generator=torch.Generator().manual_seed(1)).cuda()
        o2 = op(q, k[:, :, perm].contiguous(), v[:, :, perm].contiguous())
        assert (o2.float() - o.float()).abs().max().item() <= 2e-3


def test_argument_errors(native):
    L = native.lib()
    t = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device="cuda")
    st = ctypes.c_void_p(0)
    f = ctypes.c_float(0.125)
    p = t.data_ptr()
    assert L.deca_fa_fwd_f16(None, p, p, p, 1, 1, 128, 128, 64, f, 0, None, st) == -1
    assert L.deca_fa_fwd_f16(p, p, p, p, 1, 1, 128, 128, 96, f, 0, None, st) == -5
    assert L.deca_fa_fwd_f16(p, p, p, p, 1, 1, 128, 256, 64, f, 1, None, st) == -2  # causal needs S_q == S_kv
    assert L.deca_fa_fwd_f16(p, p, p, p, 1, 1, 100, 128, 64, f, 0, None, st) == -4  # S_q % 128
    bad = native.FaCfg(128, 128, 4, 1, 0)  # 4 stages of 64 KB do not fit at D = 128
    assert L.deca_fa_fwd_f16(p, p, p, p, 1, 1, 128, 128, 128, f, 0, ctypes.byref(bad), st) == -4
    torch.cuda.synchronize()


@pytest.mark.parametrize("shape", [(1, 150, 256, 64), (2, 3, 1024, 128), (5, 31, 512, 128), (1, 2, 2560, 64)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_persistent_kernel_matches_one_item_per_cta(native, shape, causal):
    """The persistent schedule does the arithmetic of the two-tile kernel item by item: identical
    bits, whatever the number of items per CTA (fewer items than SMs, several items per CTA, an odd
    number of Q-tile pairs per head); one head is also checked against the oracle."""
    B, H, S, D = shape
    q, k, v = make_qkv(B, H, S, S, D, seed=9)
    cfg = dict(Bc=128, stages=4 if D == 64 or S >= 512 else 2, q_tiles=2, p_tmem=1)
    plain = run_native(native, q, k, v, causal, cfg=cfg)
    pers = run_native(native, q, k, v, causal, cfg=dict(cfg, persistent=1))
    assert np.array_equal(plain, pers)
    check(q[:1, :1], k[:1, :1], v[:1, :1], pers[:1, :1], causal)


def test_persistent_config_rules(native):
    L = native.lib()

    def rc(*fields, S=1024, D=128):
        return L.deca_fa_fwd_f16_check_config(1, 2, S, S, D, 0, ctypes.byref(native.FaCfg(*fields)))

    assert rc(128, 128, 4, 2, 1, 1) == 0
    assert rc(128, 128, 4, 1, 1, 1) == -4  # two Q tiles only
    assert rc(128, 64, 4, 2, 1, 1) == -4   # 128-key tiles only
    assert rc(128, 128, 4, 2, 0, 1) == -4  # P in tensor memory only
    assert rc(128, 128, 5, 2, 1, 1) == -4  # five slots and the staging panels do not fit at D = 128
    assert rc(128, 128, 8, 2, 1, 1, D=64) == 0
    assert rc(128, 128, 4, 2, 1, 2) == -4
    assert rc(128, 128, 4, 2, 1, 1, S=384) == -4  # S_q % 256
