"""Row-wise (softmax / RMSNorm) kernel configs for B200 and their binding to the native library.

Mirrors the module-level surface of the reference's src/kernels/rowwise_tir.py: ``RowConfig``
(:42-61), ``num_chunks`` (:64-65), ``est_regs_per_thread`` (:68-85), ``check_config``
(:88-96), ``make_rowwise`` (:99), ``build_rowwise`` (:394-399), ``build_rowwise_to_file``
(:402-410).  The kernels themselves are csrc/rowwise.cu.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass

from .module import KernelModule, KernelSpec, _check_tensor, current_stream_ptr

LOG2E = 1.4426950408889634
NEG_INF = -1e30
OPS = ("softmax", "rmsnorm")
DTYPES = ("float16", "bfloat16")
MODES = ("reg", "twopass", "tma", "cluster")
MAX_CLUSTER_CHUNKS = 8  # chunk counts the cluster-mode kernels are instantiated for
MAX_REGS_PER_SM = 65536
MAX_REG_CHUNKS = 32  # chunk counts the register-mode kernels are instantiated for
MAX_TMA_CHUNKS = 16
TMA_MAX_THREADS = 512
TMA_OUT_SLOTS = 2
MAX_DYN_SMEM = 232448
KEEP_EXP_ELEMS = 128  # softmax keeps the exponentials in fp32 registers up to this many elements


@dataclass(frozen=True)
class RowConfig:
    threads_per_row: int = 128
    rows_per_block: int = 1
    vec: int = 8  # elements per vector access (8 -> 16 B for 16-bit dtypes)
    mode: str = "reg"
    # twopass: chunks loaded back to back per iteration; tma: rows in flight per row group;
    # cluster: CTAs of the thread-block cluster that shares a row (2, 4 or 8)
    unroll: int = 1
    hint: bool = False  # no-allocate loads and streaming stores

    @property
    def threads(self) -> int:
        return self.threads_per_row * self.rows_per_block

    def as_dict(self):
        return asdict(self)

    def __str__(self):
        s = f"tpr={self.threads_per_row},rpb={self.rows_per_block},vec={self.vec},mode={self.mode}"
        s += f",unroll={self.unroll}" if self.mode in ("twopass", "tma", "cluster") else ""
        return s + (",hint=1" if self.hint else "")


def cluster_slice(cfg: RowConfig, N: int) -> int:
    """Elements of a row one CTA of the cluster takes: an equal share rounded up to whole vectors."""
    return -(-(-(-N // cfg.unroll)) // cfg.vec) * cfg.vec


def num_chunks(cfg: RowConfig, N: int) -> int:
    if cfg.mode == "cluster":
        N = cluster_slice(cfg, N)
    return -(-N // (cfg.threads_per_row * cfg.vec))


def est_regs_per_thread(cfg: RowConfig, N: int, op: str) -> int:
    """32-bit registers per thread of csrc/rowwise.cu (fitted to ptxas -v for sm_100a).

    Register mode caches the row packed (vec/2 registers per chunk).  Softmax additionally
    keeps the exponentials in fp32 up to KEEP_EXP_ELEMS elements (one register each, the packed
    copy dies as they are produced); RMSNorm keeps only the packed row plus one weight chunk.
    """
    if cfg.mode in ("reg", "tma", "cluster"):
        elems = num_chunks(cfg, N) * cfg.vec
        if op == "softmax":
            regs = (elems if elems <= KEEP_EXP_ELEMS else elems // 2 + cfg.vec) + 24
        else:
            regs = elems // 2 + cfg.vec + 24
    else:
        elems = cfg.unroll * cfg.vec
        regs = elems + elems // 2 + 28
    return regs


def tma_smem_bytes(cfg: RowConfig, op: str, N: int) -> int:
    """Dynamic shared memory of the bulk-copy mode: barriers + the weight row (RMSNorm) + per
    row group an input ring of ``unroll`` rows and an output ring of two."""
    pitch = -(-N * 2 // 128) * 128
    return 2048 + (pitch if op == "rmsnorm" else 0) + cfg.rows_per_block * (cfg.unroll + TMA_OUT_SLOTS) * pitch


def check_config(cfg: RowConfig, op: str, M: int, N: int, dtype: str) -> None:
    assert op in OPS and dtype in DTYPES and cfg.mode in MODES
    if cfg.mode == "tma":
        # persistent CTAs; `rows_per_block` independent row groups, `unroll` rows in flight each
        tpr = cfg.threads_per_row
        assert cfg.vec == 8 and N % 8 == 0
        assert 32 <= tpr <= TMA_MAX_THREADS and tpr & (tpr - 1) == 0
        assert 1 <= cfg.rows_per_block <= 15 and cfg.threads <= TMA_MAX_THREADS
        assert 1 <= cfg.unroll <= 8 and cfg.rows_per_block * cfg.unroll <= 64
        assert num_chunks(cfg, N) <= MAX_TMA_CHUNKS
        assert tma_smem_bytes(cfg, op, N) <= MAX_DYN_SMEM
        return
    assert cfg.vec in (2, 4, 8) and N % cfg.vec == 0
    if cfg.mode == "cluster":
        # one row per cluster of `unroll` CTAs; each CTA caches its slice of the row in registers
        assert cfg.unroll in (2, 4, 8) and cfg.rows_per_block == 1
        assert cfg.threads_per_row % 32 == 0 and 32 <= cfg.threads_per_row <= 1024
        assert num_chunks(cfg, N) <= MAX_CLUSTER_CHUNKS
        regs = est_regs_per_thread(cfg, N, op) + 4
        assert regs <= 255 and regs * cfg.threads <= MAX_REGS_PER_SM
        return
    assert cfg.threads_per_row % 32 == 0 and cfg.threads_per_row >= 32 and cfg.threads <= 1024
    assert cfg.rows_per_block >= 1 and M % cfg.rows_per_block == 0
    assert cfg.unroll in (1, 2, 4)
    if cfg.mode == "reg":
        assert num_chunks(cfg, N) <= MAX_REG_CHUNKS
    regs = est_regs_per_thread(cfg, N, op)
    assert regs <= 255 and regs * cfg.threads <= MAX_REGS_PER_SM


def make_rowwise(op: str, M: int, N: int, dtype: str, cfg: RowConfig, eps: float = 1e-6) -> KernelSpec:
    """Softmax: y = softmax(x, -1).  RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w."""
    check_config(cfg, op, M, N, dtype)
    return KernelSpec("rowwise", (M, N), dtype, cfg.as_dict(), {"op": op, "eps": float(eps)})


def build_rowwise(mod: KernelSpec, target=None, dump_dir=None) -> KernelModule:
    return KernelModule(mod)


def build_rowwise_to_file(op: str, shape, dtype: str, cfg: RowConfig, eps: float, arch: str, path: str) -> str:
    """Writes the kernel spec to ``path`` (safe in a worker process without a CUDA context)."""
    M, N = shape
    return make_rowwise(op, M, N, dtype, cfg, eps).export_library(path)


def native_cfg(cfg: RowConfig):
    from .. import native

    return native.RowCfg(
        cfg.threads_per_row, cfg.rows_per_block, cfg.vec, native.ROW_MODE_CODE[cfg.mode], cfg.unroll,
        int(cfg.hint),
    )


def bind(spec: KernelSpec):
    """Returns main(x[, w], y) launching deca_rowwise on torch's current stream."""
    import ctypes

    import torch

    from .. import native

    L = native.lib()
    M, N = spec.shape
    op = spec.params["op"]
    cfg = RowConfig(**spec.config)
    ccfg = native_cfg(cfg)
    op_code, dt_code = native.ROW_OP_CODE[op], native.DTYPE_CODE[spec.dtype]
    native.check(L.deca_rowwise_check_config(op_code, dt_code, M, N, ctypes.byref(ccfg)), f"{op} config {cfg}")
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[spec.dtype]
    eps = ctypes.c_float(spec.params.get("eps", 1e-6))
    cfg_ref = ctypes.byref(ccfg)
    fn = L.deca_rowwise
    what = f"deca_rowwise({op})"

    if op == "softmax":
        def main(x, y):
            _check_tensor(x, (M, N), tdt, "x")
            _check_tensor(y, (M, N), tdt, "y")
            native.check(fn(op_code, dt_code, x.data_ptr(), None, y.data_ptr(), M, N, eps, cfg_ref,
                            current_stream_ptr()), what)
    else:
        def main(x, w, y):
            _check_tensor(x, (M, N), tdt, "x")
            _check_tensor(w, (N,), tdt, "w")
            _check_tensor(y, (M, N), tdt, "y")
            native.check(fn(op_code, dt_code, x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, eps, cfg_ref,
                            current_stream_ptr()), what)

    main._keepalive = ccfg
    return main
