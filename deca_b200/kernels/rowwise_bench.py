"""Row-wise benchmark helpers behind the names the reference's CLI and operators import from
src/kernels/rowwise_bench.py: dtype names (:22-26), the sweep grids (:29-34), the byte count that
is the roofline numerator (:37-39), seeded inputs (:42-50) and the eager torch baselines (:53-66).
Softmax and RMSNorm are memory bound: throughput is reported as effective bytes (x read once,
y written once, plus the weight vector for RMSNorm) per second."""

from __future__ import annotations

from .timing import bench_cuda, bench_interleaved  # noqa: F401  (part of this module's surface)

ROWWISE_OPS = ("softmax", "rmsnorm")
RMSNORM_EPS = 1e-6

# Sweep: transformer hidden sizes against token counts, and (softmax only) vocabulary-sized rows.
HIDDEN_GRID = {"cols": (1024, 2048, 4096, 8192), "rows": (4096, 16384, 65536)}
VOCAB_GRID = {"cols": (32000, 128256), "rows": (1024, 4096, 8192)}

_CANONICAL = {"fp16": "float16", "float16": "float16", "bf16": "bfloat16", "bfloat16": "bfloat16"}


def canonical_dtype(dtype: str) -> str:
    """'fp16' / 'bf16' (the CLI spelling) or the torch names -> the torch name."""
    return _CANONICAL[dtype]


def _torch_dtype(dtype: str):
    import torch

    return getattr(torch, canonical_dtype(dtype))


def standard_shapes(op: str):
    """[(M, N)] of the sweep for ``op``: columns outermost, hidden sizes before vocabulary sizes."""
    grids = [HIDDEN_GRID] + ([VOCAB_GRID] if op == "softmax" else [])
    return [(rows, cols) for grid in grids for cols in grid["cols"] for rows in grid["rows"]]


def rowwise_bytes(op: str, M: int, N: int, type_size: int = 2) -> int:
    """Algorithmic traffic of one launch: M * N elements in, M * N out, N weights for RMSNorm."""
    elements = 2 * M * N + (N if op == "rmsnorm" else 0)
    return elements * type_size


def make_inputs(op: str, M: int, N: int, dtype: str, seed: int = 0):
    """(x,) for softmax, (x, w) for RMSNorm, on the GPU from one seeded CUDA generator:
    x ~ N(0, 1) drawn in the I/O type, w = 1 + 0.1 N(0, 1) drawn in fp32 and then rounded."""
    import torch

    tdt = _torch_dtype(dtype)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, N, device="cuda", dtype=tdt, generator=gen)
    if op == "softmax":
        return (x,)
    w = torch.randn(N, device="cuda", generator=gen).mul_(0.1).add_(1.0).to(tdt)
    return (x, w)


def torch_ref(op: str, inputs, eps: float = RMSNORM_EPS):
    """Eager torch on the same tensors: the baseline and the correctness reference."""
    import torch
    import torch.nn.functional as F

    if op == "softmax":
        return torch.softmax(inputs[0], dim=-1)
    x, w = inputs
    return F.rms_norm(x, (x.shape[-1],), w, eps=eps)


def bench_torch(op: str, M: int, N: int, dtype: str):
    """(seconds, GB/s) of the eager torch operator on fresh seeded inputs."""
    inputs = make_inputs(op, M, N, dtype)
    seconds = bench_cuda(lambda: torch_ref(op, inputs))
    return seconds, rowwise_bytes(op, M, N) / seconds / 1e9
