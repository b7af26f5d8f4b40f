"""CPU oracle for the DeCA operator hot path (numpy in, numpy out).

TEST INFRASTRUCTURE ONLY.  This package is the checker for the CUDA kernels and the
timed CPU baseline of ``bench.py``; the product package never imports it.  The
arithmetic lives in ``oracle.c`` (each function cites the reference lines it
restates); this module builds that file with gcc and wraps it with ctypes.

Parity pin: ``tests/test_oracle_golden.py`` checks these functions against golden
vectors produced by the reference's own Python code (``tests/golden/make_golden.py``).

16-bit tensors travel as numpy ``uint16`` bit patterns (numpy has no bfloat16);
``to_bits`` / ``from_bits`` convert from and to fp32.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_DIR, "oracle.c")
_LIB = os.path.join(_DIR, "liboracle.so")
_lib = None

DT_F16, DT_BF16 = 0, 1
DTYPE_CODE = {"float16": DT_F16, "fp16": DT_F16, "bfloat16": DT_BF16, "bf16": DT_BF16}


def build(force: bool = False) -> str:
    """Compiles oracle.c into liboracle.so next to it (no-op when up to date)."""
    if (
        not force
        and os.path.exists(_LIB)
        and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC)
    ):
        return _LIB
    cmd = ["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", _SRC, "-o", _LIB, "-lm"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int | None = None) -> int:
    """Uses ``n`` OpenMP threads (default: every core the process may run on); returns the count."""
    if n is None:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


def to_bits(x32: np.ndarray, dtype: str) -> np.ndarray:
    """fp32 array -> uint16 bit patterns of float16 / bfloat16 (round to nearest even)."""
    x32 = np.ascontiguousarray(x32, dtype=np.float32)
    if DTYPE_CODE[dtype] == DT_F16:
        return x32.astype(np.float16).view(np.uint16)
    u = x32.view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def from_bits(bits: np.ndarray, dtype: str) -> np.ndarray:
    """uint16 bit patterns of float16 / bfloat16 -> fp32 array."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if DTYPE_CODE[dtype] == DT_F16:
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def softmax(x_bits: np.ndarray, dtype: str = "float16", want_f32: bool = False):
    """Row-wise softmax of X[M, N]; returns y bits (and the unrounded fp32 values)."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    M, N = x_bits.shape
    y = np.empty_like(x_bits)
    y32 = np.empty((M, N), np.float32) if want_f32 else None
    lib().oracle_softmax(_p(x_bits), _p(y), _p(y32), _i64(M), _i64(N), DTYPE_CODE[dtype])
    return (y, y32) if want_f32 else y


def rmsnorm(x_bits, w_bits, eps: float = 1e-6, dtype: str = "float16", want_f32: bool = False,
            round_normed: bool = True):
    """RMSNorm of X[M, N] with weight W[N]; returns y bits (and the unrounded fp32 values).

    ``round_normed`` (the kernel's behaviour) rounds x*r to the I/O dtype before the weight
    multiply; False gives the single-rounding form of torch's CPU rms_norm."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    M, N = x_bits.shape
    assert w_bits.shape == (N,)
    y = np.empty_like(x_bits)
    y32 = np.empty((M, N), np.float32) if want_f32 else None
    lib().oracle_rmsnorm(
        _p(x_bits), _p(w_bits), _p(y), _p(y32), _i64(M), _i64(N), ctypes.c_float(eps), DTYPE_CODE[dtype],
        ctypes.c_int(int(round_normed)),
    )
    return (y, y32) if want_f32 else y


def gemm16(a_bits, b_bits, dtype: str = "float16", want_f32: bool = False):
    """C = A @ B on 16-bit inputs with fp32 accumulation; returns c bits (and fp32 C)."""
    a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    M, K = a_bits.shape
    K2, N = b_bits.shape
    assert K == K2
    c = np.empty((M, N), np.uint16)
    c32 = np.empty((M, N), np.float32) if want_f32 else None
    lib().oracle_gemm16(_p(a_bits), _p(b_bits), _p(c), _p(c32), _i64(M), _i64(N), _i64(K), DTYPE_CODE[dtype])
    return (c, c32) if want_f32 else c


def gemm_f32_naive(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """The reference's unscheduled fp32 GEMM (single thread, k innermost)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32_naive(_p(a), _p(b), _p(c), _i64(M), _i64(N), _i64(K))
    return c


def attention(q_bits, k_bits, v_bits, scale=None, causal=False, want_f32=False, blockwise_bc=0):
    """fp16 attention forward on [B, H, S, D] bit arrays.

    ``blockwise_bc == 0``: plain fp32 softmax(scale QK^T + mask) V (the ground truth).
    ``blockwise_bc > 0``: the kernel's online-softmax recurrence over KV tiles of that size.
    """
    q_bits = np.ascontiguousarray(q_bits, dtype=np.uint16)
    k_bits = np.ascontiguousarray(k_bits, dtype=np.uint16)
    v_bits = np.ascontiguousarray(v_bits, dtype=np.uint16)
    B, H, Sq, D = q_bits.shape
    Skv = k_bits.shape[2]
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    assert not causal or Sq == Skv
    o = np.empty_like(q_bits)
    o32 = np.empty(q_bits.shape, np.float32) if want_f32 else None
    args = [_p(q_bits), _p(k_bits), _p(v_bits), _p(o), _p(o32), _i64(B * H), _i64(Sq), _i64(Skv), _i64(D),
            ctypes.c_float(scale), ctypes.c_int(int(causal))]
    if blockwise_bc:
        assert Skv % blockwise_bc == 0
        lib().oracle_attention_blockwise(*args, _i64(blockwise_bc))
    else:
        lib().oracle_attention(*args)
    return (o, o32) if want_f32 else o
