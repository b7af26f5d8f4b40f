"""Shapes, inputs and baselines of the 16-bit tensor-core GEMM C = A @ B (same surface as the
reference's src/kernels/gemm_bench.py).  A[M, K], B[K, N], C[M, N] are row-major; accumulation
is fp32."""

import torch

from .attn_bench import bench_cuda, bench_interleaved  # noqa: F401  (re-exported)

# Square GEMMs from 2K to 16K in steps of 2K.
SQUARE_SIZES = list(range(2048, 16384 + 1, 2048))


def standard_shapes():
    """Returns a list of (M, N, K)."""
    return [(n, n, n) for n in SQUARE_SIZES]


def gemm_flops(M: int, N: int, K: int) -> float:
    return 2.0 * M * N * K


def make_inputs(M: int, N: int, K: int, seed: int = 0, dtype=torch.float16):
    """Returns (a, b) with unit-variance 16-bit entries."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device="cuda", dtype=dtype, generator=g)
    b = torch.randn(K, N, device="cuda", dtype=dtype, generator=g)
    return a, b


def torch_ref(inputs):
    """torch (cuBLAS) baseline."""
    a, b = inputs
    return a @ b


def bench_torch(M: int, N: int, K: int):
    """Returns (seconds, TFLOPS) of torch.matmul."""
    inputs = make_inputs(M, N, K)
    t = bench_cuda(lambda: torch_ref(inputs))
    return t, gemm_flops(M, N, K) / t / 1e12
