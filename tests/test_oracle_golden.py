"""Pins the CPU oracle against golden vectors produced by the reference's own Python code
(tests/golden/make_golden.py).  Tolerances are the ones stated for the hot path:
GEMM rtol 1e-2 / atol 1e-2 (far tighter here), attention max-abs 2e-3, row-wise 1e-3
relative (one ulp of the 16-bit output type where that is coarser)."""

import numpy as np
import pytest

import oracle


def ulp(ref32, dtype):
    """Spacing of the 16-bit output type at |ref32| (fp16 subnormals included)."""
    mant = 10 if dtype == "float16" else 7
    emin = -14 if dtype == "float16" else -126
    e = np.floor(np.log2(np.maximum(np.abs(ref32), 2.0**emin)))
    return 2.0 ** (e - mant)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("tag", ["hid", "ragged", "vocab"])
def test_softmax_matches_reference(golden, dtype, tag):
    x = golden[f"row_{tag}_{dtype}_x"]
    ref = oracle.from_bits(golden[f"row_{tag}_{dtype}_softmax"], dtype)
    y, y32 = oracle.softmax(x, dtype, want_f32=True)
    got = oracle.from_bits(y, dtype)
    # The two fp32 computations agree to ~1e-6 relative; the 16-bit results may differ by one ulp.
    assert np.all(np.abs(got - ref) <= ulp(ref, dtype) + 1e-12)
    assert np.all(np.abs(y32 - ref) <= 1e-3 * np.abs(ref) + 0.5 * ulp(ref, dtype))
    assert np.mean(got == ref) > 0.99
    np.testing.assert_allclose(y32.astype(np.float64).sum(-1), 1.0, rtol=1e-4)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("tag", ["hid", "ragged"])
def test_rmsnorm_matches_reference(golden, dtype, tag):
    x, w = golden[f"row_{tag}_{dtype}_x"], golden[f"row_{tag}_{dtype}_w"]
    ref = oracle.from_bits(golden[f"row_{tag}_{dtype}_rmsnorm"], dtype)
    # The golden vectors come from torch's CPU rms_norm, which rounds once (y = dt(x*r*w)).
    # The single-rounding form of the oracle reproduces them bit for bit ...
    single = oracle.from_bits(oracle.rmsnorm(x, w, 1e-6, dtype, round_normed=False), dtype)
    assert np.mean(single == ref) > 0.995
    assert np.all(np.abs(single - ref) <= ulp(ref, dtype))
    # ... and the kernel's form (x*r rounded to the I/O dtype before the weight multiply,
    # rowwise_tir.py:340-344) moves a result by at most one extra rounding step.
    got = oracle.from_bits(oracle.rmsnorm(x, w, 1e-6, dtype), dtype)
    assert np.all(np.abs(got - ref) <= 1.5 * ulp(ref, dtype))
    atol, rtol = (1e-2, 1e-2) if dtype == "float16" else (3e-2, 3e-2)  # operators/Rowwise.py:15-20
    assert np.all(np.abs(got - ref) <= atol + rtol * np.abs(ref))


def test_gemm16_matches_reference(golden):
    c, c32 = oracle.gemm16(golden["gemm_a"], golden["gemm_b"], "float16", want_f32=True)
    ref = golden["gemm_c32"]
    np.testing.assert_allclose(c32, ref, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(oracle.from_bits(c, "float16"), ref, rtol=1e-2, atol=1e-2)
    assert np.array_equal(c, c32.astype(np.float16).view(np.uint16))


def test_f32_gemm_matches_reference_tir(golden, golden_meta):
    c = oracle.gemm_f32_naive(golden["f32gemm_a"], golden["f32gemm_b"])
    np.testing.assert_allclose(c, golden["f32gemm_c"], rtol=1e-6, atol=1e-6)
    import torch

    g = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.rand(512, 512, generator=g) * 2 - 1).numpy()
    b = (torch.rand(512, 512, generator=g) * 2 - 1).numpy()
    c = oracle.gemm_f32_naive(a, b)
    np.testing.assert_allclose(c[::37, ::41], golden["f32gemm512_sample"], rtol=1e-5, atol=1e-5)
    assert abs(c.astype(np.float64).sum() - golden_meta["f32gemm512"]["sum"]) < 1e-2
    assert abs(np.abs(c).astype(np.float64).sum() / golden_meta["f32gemm512"]["abs_sum"] - 1) < 1e-6


@pytest.mark.parametrize("tag", ["d64", "d128"])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_matches_reference(golden, tag, causal):
    q, k, v = (golden[f"attn_{tag}_{n}"] for n in "qkv")
    ref = oracle.from_bits(golden[f"attn_{tag}_o_{'causal' if causal else 'full'}"], "float16")
    o, o32 = oracle.attention(q, k, v, causal=causal, want_f32=True)
    assert np.abs(o32 - ref).max() <= 2e-3
    assert np.abs(oracle.from_bits(o, "float16") - ref).max() <= 2e-3
    # the kernel-shaped recurrence (fp16 P, finite -1e30 mask, exp2 form) agrees with the plain form
    for bc in (32, 128):
        ob = oracle.from_bits(oracle.attention(q, k, v, causal=causal, blockwise_bc=bc), "float16")
        assert np.abs(ob - ref).max() <= 2e-3
        assert np.abs(ob - o32).max() <= 2e-3
