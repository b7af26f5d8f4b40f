"""GEMM benchmark helpers behind the names the reference's CLI imports from
src/kernels/gemm_bench.py: the square sweep (:14-19), the work formula (:22-23), seeded inputs
(:26-31), the torch baseline (:34-44) and the fp16-accumulating cuBLAS baseline (:47-85).
A[M, K], B[K, N], C[M, N] row-major."""

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


class CublasHgemm:
    """Baseline for the fp16-accumulate mode: ``cublasHgemm`` (fp16 in, fp16 accumulate, fp16 out)
    on torch tensors, called through ctypes on torch's current stream, since torch itself only
    offers fp32-accumulating half GEMMs.  ``CublasHgemm()(a, b, c)`` computes c = a @ b for
    row-major tensors (cuBLAS is column-major: it is asked for c^T = b^T a^T)."""

    def __init__(self):
        import ctypes
        import glob
        import os

        import nvidia.cublas as pkg

        libs = sorted(glob.glob(os.path.join(os.path.dirname(pkg.__file__), "lib", "libcublas.so*")))
        if not libs:
            raise RuntimeError("the cuBLAS library that ships with torch was not found")
        self._c = ctypes
        self._lib = ctypes.CDLL(libs[-1])
        self._handle = ctypes.c_void_p()
        self._must(self._lib.cublasCreate_v2(ctypes.byref(self._handle)), "cublasCreate")
        one, zero = 0x3C00, 0x0000  # fp16 bit patterns of alpha = 1 and beta = 0 (host pointers)
        self._alpha, self._beta = ctypes.c_uint16(one), ctypes.c_uint16(zero)

    @staticmethod
    def _must(status: int, what: str):
        if status != 0:
            raise RuntimeError(f"{what} failed with cuBLAS status {status}")

    def __call__(self, a, b, c):
        import torch

        ct = self._c
        (M, K), N = a.shape, b.shape[1]
        self._must(self._lib.cublasSetStream_v2(self._handle, ct.c_void_p(torch.cuda.current_stream().cuda_stream)),
                   "cublasSetStream")
        no_trans = 0
        self._must(self._lib.cublasHgemm(self._handle, no_trans, no_trans, N, M, K, ct.byref(self._alpha),
                                         ct.c_void_p(b.data_ptr()), N, ct.c_void_p(a.data_ptr()), K,
                                         ct.byref(self._beta), ct.c_void_p(c.data_ptr()), N), "cublasHgemm")
        return c

    def __del__(self):
        try:
            self._lib.cublasDestroy_v2(self._handle)
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass
