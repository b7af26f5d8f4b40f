"""ctypes binding of libdeca_b200.so, the C ABI declared in include/deca_b200.h.

There is no fallback: if the library is missing, loading raises, and every operator call
goes through it.  Build it with ``python -m deca_b200.build``.
"""

from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

_lib = None

F16, BF16 = 0, 1
SOFTMAX, RMSNORM = 0, 1
ROW_REG, ROW_TWOPASS, ROW_TMA, ROW_CLUSTER = 0, 1, 2, 3
DTYPE_CODE = {"float16": F16, "bfloat16": BF16}
ROW_OP_CODE = {"softmax": SOFTMAX, "rmsnorm": RMSNORM}
ROW_MODE_CODE = {"reg": ROW_REG, "twopass": ROW_TWOPASS, "tma": ROW_TMA, "cluster": ROW_CLUSTER}
ROW_MODE_NAME = {v: k for k, v in ROW_MODE_CODE.items()}


class DecaError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: status {status} ({status_string(status)})")


class RowCfg(ctypes.Structure):
    _fields_ = [
        ("threads_per_row", ctypes.c_int),
        ("rows_per_block", ctypes.c_int),
        ("vec", ctypes.c_int),
        ("mode", ctypes.c_int),
        ("unroll", ctypes.c_int),
        ("hint", ctypes.c_int),
    ]


class GemmCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("BM", "BN", "BK", "stages", "raster", "epi_smem", "cta_group", "acc_bufs",
                                            "stream_k", "acc_f16", "raster_n")]


class FaCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("Br", "Bc", "stages", "q_tiles", "p_tmem", "persistent")]


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA kernels are not built and there is no fallback. "
                "Run `python -m deca_b200.build`."
            )
        L = ctypes.CDLL(LIB_PATH)
        L.deca_version.restype = ctypes.c_char_p
        L.deca_status_string.restype = ctypes.c_char_p
        L.deca_status_string.argtypes = [ctypes.c_int]
        vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.deca_rowwise.argtypes = [ci, ci, vp, vp, vp, i64, i64, cf, ctypes.POINTER(RowCfg), vp]
        L.deca_rowwise_stats.argtypes = [ci, ci, vp, vp, vp, vp, i64, i64, cf, ctypes.POINTER(RowCfg), vp]
        L.deca_rowwise_check_config.argtypes = [ci, ci, i64, i64, ctypes.POINTER(RowCfg)]
        L.deca_rowwise_default_config.argtypes = [ci, ci, i64, i64, ctypes.POINTER(RowCfg)]
        L.deca_gemm16_check_config.argtypes = [ci, i64, i64, i64, ctypes.POINTER(GemmCfg)]
        L.deca_gemm16.argtypes = [ci, vp, vp, vp, i64, i64, i64, ctypes.POINTER(GemmCfg), vp]
        L.deca_gemm16_default_config.argtypes = [i64, i64, i64, ci, ci, ctypes.POINTER(GemmCfg)]
        L.deca_gemm16_workspace_bytes.argtypes = [ci, i64, i64, i64, ctypes.POINTER(GemmCfg), ctypes.POINTER(ctypes.c_size_t)]
        L.deca_gemm16_ws.argtypes = [ci, vp, vp, vp, i64, i64, i64, ctypes.POINTER(GemmCfg), vp, ctypes.c_size_t, vp]
        L.deca_gemm16_sk_static.argtypes = [ci, vp, vp, vp, i64, i64, i64, ctypes.POINTER(GemmCfg), vp]
        L.deca_gemm16_gather.argtypes = [ci, vp, vp, ctypes.POINTER(vp), ci, ci, i64, i64, i64, ctypes.POINTER(GemmCfg), vp]
        L.deca_fa_fwd_f16_check_config.argtypes = [ci, ci, ci, ci, ci, ci, ctypes.POINTER(FaCfg)]
        L.deca_fa_fwd_f16.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, ctypes.POINTER(FaCfg), vp]
        L.deca_fa_fwd_f16_gather.argtypes = [vp, vp, vp, ctypes.POINTER(vp), ci, ci, ci, ci, ci, ci, ci, cf, ci,
                                             ctypes.POINTER(FaCfg), vp]
        ip = ctypes.POINTER(ci)
        L.deca_last_device_status.argtypes = [ip, ip, ip, ci]
        L.deca_device_status_words.argtypes = [ctypes.POINTER(ctypes.c_uint), ci]
        L.deca_selftest_bounded_wait.argtypes = [ctypes.c_uint, vp]
        _lib = L
    return _lib


def version() -> str:
    return lib().deca_version().decode()


def status_string(status: int) -> str:
    return lib().deca_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        raise DecaError(status, what)


def last_device_status(clear: bool = True):
    """(code, where, block) of the first bounded wait that ran out since the last clear;
    code 0 means none.  Synchronises the device."""
    c, w, b = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    check(lib().deca_last_device_status(ctypes.byref(c), ctypes.byref(w), ctypes.byref(b), int(clear)),
          "deca_last_device_status")
    return c.value, w.value, b.value


def device_status_words(n: int = 16):
    """The raw status record (see deca_device_status_words); for diagnosing a timeout."""
    buf = (ctypes.c_uint * 16)()
    check(lib().deca_device_status_words(buf, n), "deca_device_status_words")
    return [int(x) for x in buf[:n]]
