"""Attention benchmark helpers behind the names the reference's CLIs and RuntimeMod import from
src/kernels/attn_bench.py: the sweep grid (:17-27), the work formula (:30-32), the timers
(:35-70, :94-100; implemented in ``timing.py``), seeded inputs (:73-78) and the SDPA baseline
(:81-91)."""

from __future__ import annotations

import math

from .timing import bench_cuda, bench_interleaved  # noqa: F401  (part of this module's surface)

# The FlashAttention-2 paper grid: 16 Ki tokens per batch, model width 2048 split into heads of
# 64 or 128, sequence lengths 512 ... 16 Ki.
TOKENS_PER_BATCH = 16384
MODEL_WIDTH = 2048
HEAD_DIMS = (64, 128)
SEQ_LENS = tuple(1 << p for p in range(9, 15))


def standard_shapes():
    """[(B, H, S, D)] of the sweep, head dim outermost."""
    return [(TOKENS_PER_BATCH // S, MODEL_WIDTH // D, S, D) for D in HEAD_DIMS for S in SEQ_LENS]


def attn_flops(B: int, H: int, S_q: int, S_kv: int, D: int, causal: bool = False) -> float:
    """Two GEMMs of 2 * S_q * S_kv * D flops per head; a causal mask halves the count."""
    return 4.0 * B * H * S_q * S_kv * D * (0.5 if causal else 1.0)


def default_scale(D: int) -> float:
    return 1.0 / math.sqrt(D)


def make_qkv(B: int, H: int, S_q: int, S_kv: int, D: int, dtype=None, seed: int = 0):
    """Standard-normal Q, K, V on the GPU from one seeded CUDA generator (drawn in that order)."""
    import torch

    dtype = dtype or torch.float16
    gen = torch.Generator(device="cuda").manual_seed(seed)
    return tuple(torch.randn(B, H, S, D, device="cuda", dtype=dtype, generator=gen) for S in (S_q, S_kv, S_kv))


def sdpa_flash(q, k, v, causal: bool = False, scale: float | None = None):
    """torch's scaled_dot_product_attention restricted to its flash backend: the baseline and the
    correctness reference of the attention operator."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
        return F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)


def bench_sdpa_flash(B, H, S_q, S_kv, D, causal=False, dtype=None):
    """(seconds, TFLOPS) of the SDPA-flash baseline on fresh seeded inputs."""
    q, k, v = make_qkv(B, H, S_q, S_kv, D, dtype)
    seconds = bench_cuda(lambda: sdpa_flash(q, k, v, causal=causal))
    return seconds, attn_flops(B, H, S_q, S_kv, D, causal) / seconds / 1e12
