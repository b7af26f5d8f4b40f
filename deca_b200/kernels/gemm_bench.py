"""GEMM benchmark helpers behind the names the reference's CLI imports from
src/kernels/gemm_bench.py: the square sweep (:14-19), the work formula (:22-23), seeded inputs
(:26-31) and the torch baseline (:34-44).  A[M, K], B[K, N], C[M, N] row-major, fp32 accumulation."""

from __future__ import annotations

from .timing import bench_cuda, bench_interleaved  # noqa: F401  (part of this module's surface)

SWEEP_FIRST, SWEEP_LAST, SWEEP_STEP = 2048, 16384, 2048


def standard_shapes():
    """[(n, n, n)] for n = 2048, 4096, ..., 16384."""
    return [(n, n, n) for n in range(SWEEP_FIRST, SWEEP_LAST + 1, SWEEP_STEP)]


def gemm_flops(M: int, N: int, K: int) -> float:
    return 2.0 * M * N * K


def make_inputs(M: int, N: int, K: int, seed: int = 0, dtype=None):
    """Standard-normal A then B on the GPU from one seeded CUDA generator."""
    import torch

    dtype = dtype or torch.float16
    gen = torch.Generator(device="cuda").manual_seed(seed)
    return tuple(torch.randn(*shape, device="cuda", dtype=dtype, generator=gen) for shape in ((M, K), (K, N)))


def torch_ref(inputs):
    """The cuBLAS baseline (torch.matmul on the 16-bit inputs)."""
    a, b = inputs
    return a @ b


def bench_torch(M: int, N: int, K: int):
    """(seconds, TFLOPS) of torch.matmul on fresh seeded inputs."""
    inputs = make_inputs(M, N, K)
    seconds = bench_cuda(lambda: torch_ref(inputs))
    return seconds, gemm_flops(M, N, K) / seconds / 1e12
