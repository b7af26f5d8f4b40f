"""16-bit tensor-core GEMM configs for B200 and their binding to the native library.

Mirrors the module-level surface of the reference's src/kernels/gemm_tir.py -- ``GemmConfig``
(:42-76), ``smem_bytes`` (:79-89), ``check_config`` (:101-120), ``make_gemm_tc`` (:123),
``build_gemm_tc`` (:392-398), ``build_gemm_tc_to_file`` (:401-407) -- with the tile space
of the tcgen05 kernel in csrc/gemm_f16.cu instead of the mma.sync one: there are no warp
tiles (one thread issues the MMAs, the accumulator lives in tensor memory), the CTA tile is
the MMA tile (BM = 128 rows per CTA, BN <= 256 columns), ``cta_group = 2`` pairs two CTAs on
a 256-row tile, ``stages`` counts TMA pipeline slots and ``acc_bufs`` tensor-memory
accumulators (2 lets the epilogue of one tile overlap the main loop of the next).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass

from .module import KernelModule, KernelSpec, _check_tensor, current_stream_ptr

MAX_DYN_SMEM = 232448  # 227 KB opt-in per CTA
TMEM_COLUMNS = 512
SMEM_RESERVED = 2048  # barriers, tensor-memory base slot, alignment slack
GEMM_DTYPES = ("float16", "bfloat16")


@dataclass(frozen=True)
class GemmConfig:
    BM: int = 128  # tile rows per CTA: 128 (one MMA per k step) or 256 (two MMAs share the B tile)
    BN: int = 256  # tile columns (the tcgen05 N)
    BK: int = 64  # K depth of one pipeline stage (one 128-byte swizzle row of fp16)
    stages: int = 4  # TMA -> MMA shared-memory ring depth
    raster: int = 8  # tile rows per rasterization group (1: plain row-major order)
    epi_smem: bool = True  # stage C through shared memory and write it with TMA stores
    cta_group: int = 1  # 2: two CTAs of a cluster share one 256-row MMA tile
    acc_bufs: int = 2  # tensor-memory accumulator buffers
    stream_k: bool = False  # cut the k blocks of the last tiles into one equal share per SM
    raster_n: bool = False  # raster groups are tile columns walked down M (keeps a band of B in L2; for M > N)
    acc_f16: bool = False  # fp16 accumulators (tcgen05 D type f16) instead of fp32: fp16 inputs, one-CTA tiles only

    @property
    def threads(self) -> int:
        return 192  # TMA warp + MMA warp + 4 epilogue warps

    def as_dict(self):
        return asdict(self)

    def __str__(self):
        return (
            f"{self.BM}x{self.BN}x{self.BK},cta={self.cta_group},stages={self.stages},"
            f"raster={self.raster},epi_smem={int(self.epi_smem)},acc={self.acc_bufs}"
            + (",sk=1" if self.stream_k else "")
            + (",raster_n=1" if self.raster_n else "")
            + (",acc_f16=1" if self.acc_f16 else "")
        )


def pipeline_smem_bytes(cfg: GemmConfig) -> int:
    # per CTA: its A rows and (BN / cta_group) of the B columns per stage
    return cfg.stages * (cfg.BM * cfg.BK + cfg.BK * cfg.BN // cfg.cta_group) * 2


def epilogue_smem_bytes(cfg: GemmConfig) -> int:
    # per epilogue warp two 32 x 64 staging panels (double buffered TMA stores)
    return 4 * 2 * 32 * 64 * 2 if cfg.epi_smem else 0


def smem_bytes(cfg: GemmConfig) -> int:
    return pipeline_smem_bytes(cfg) + epilogue_smem_bytes(cfg) + SMEM_RESERVED


def tmem_columns(cfg: GemmConfig) -> int:
    cols = cfg.acc_bufs * (cfg.BM // 128) * cfg.BN
    p = 32
    while p < cols:
        p *= 2
    return p


def check_config(cfg: GemmConfig, M: int, N: int, K: int, max_smem: int = MAX_DYN_SMEM) -> None:
    assert cfg.BM in (128, 256) and cfg.BK == 64
    assert cfg.BN in (64, 128, 256) and not (cfg.BM == 256 and cfg.BN == 64)
    assert cfg.cta_group in (1, 2) and cfg.acc_bufs in (1, 2)
    if cfg.cta_group == 2:
        # CTA pairs: a (2 BM) x BN tile, each CTA holds BM rows and fetches half of the B columns
        assert cfg.BN in (128, 256) and cfg.epi_smem and not cfg.stream_k
    if cfg.raster_n:
        assert cfg.cta_group == 1
    if cfg.acc_f16:  # fp16 accumulators: one-CTA kernel, whole tiles (split tiles exchange fp32 partial sums)
        assert cfg.cta_group == 1 and not cfg.stream_k
    assert 2 <= cfg.stages <= 8
    assert cfg.raster >= 1
    assert tmem_columns(cfg) <= TMEM_COLUMNS
    assert smem_bytes(cfg) <= max_smem
    assert M >= 1 and N >= 8 and K >= 8
    # TMA needs 16-byte row pitches; partial tiles are zero-filled / clipped by TMA
    assert N % 8 == 0 and K % 8 == 0


def default_config(M: int, N: int, K: int, acc_f16: bool = False, sms: int = 148) -> GemmConfig:
    """The config the native library uses when none is given (``deca_gemm16_default_config``, a
    host-only call): 256 x 256 tiles once they give every SM one (one B tile feeds two MMAs, which
    halves the L2 -> shared-memory traffic per flop), else the best-scoring narrower tile."""
    import ctypes

    from .. import native

    c = native.GemmCfg()
    native.check(native.lib().deca_gemm16_default_config(M, N, K, sms, int(acc_f16), ctypes.byref(c)),
                 "deca_gemm16_default_config")
    return GemmConfig(BM=c.BM, BN=c.BN, BK=c.BK, stages=c.stages, raster=c.raster, epi_smem=bool(c.epi_smem),
                      cta_group=c.cta_group, acc_bufs=c.acc_bufs, stream_k=bool(c.stream_k), raster_n=bool(c.raster_n),
                      acc_f16=bool(c.acc_f16))


def make_gemm_tc(M: int, N: int, K: int, cfg: GemmConfig, dtype: str = "float16") -> KernelSpec:
    check_config(cfg, M, N, K)
    assert dtype in GEMM_DTYPES
    assert not cfg.acc_f16 or dtype == "float16", "fp16 accumulation needs fp16 inputs"
    return KernelSpec("gemm", (M, N, K), dtype, cfg.as_dict())


def build_gemm_tc(mod: KernelSpec, target=None, dump_dir=None) -> KernelModule:
    return KernelModule(mod)


def build_gemm_tc_to_file(shape, cfg: GemmConfig, arch: str, path: str, dtype: str = "float16") -> str:
    """Writes the kernel spec to ``path`` (safe in a worker process without a CUDA context)."""
    M, N, K = shape
    return make_gemm_tc(M, N, K, cfg, dtype).export_library(path)


def native_cfg(cfg: GemmConfig):
    from .. import native

    return native.GemmCfg(cfg.BM, cfg.BN, cfg.BK, cfg.stages, cfg.raster, int(cfg.epi_smem), cfg.cta_group,
                          cfg.acc_bufs, int(cfg.stream_k), int(cfg.acc_f16), int(cfg.raster_n))


def stream_k_plan(cfg: GemmConfig, M: int, N: int, K: int, sms: int = 148):
    """(grid, whole tiles, split units) of the stream-K mode for this shape, or None where the
    native library would not split (mirror of plan_stream_k in csrc/gemm_f16.cu)."""
    tiles = -(-M // cfg.BM) * -(-N // cfg.BN)
    num_kb = -(-K // cfg.BK)
    waves = -(-tiles // sms)
    if sms < 2 or tiles / (waves * sms) >= 0.95:
        return None
    if tiles >= sms:
        dp_tiles = (tiles // sms - 1) * sms
        grid = sms
    else:
        dp_tiles = 0
        grid = min(sms, tiles * num_kb // 8)
        if grid <= tiles:
            return None
    return grid, dp_tiles, (tiles - dp_tiles) * num_kb


def bind(spec: KernelSpec):
    """Returns main(a, b, c) launching deca_gemm16 on torch's current stream."""
    import ctypes

    import torch

    from .. import native

    L = native.lib()
    M, N, K = spec.shape
    cfg = GemmConfig(**spec.config)
    ccfg = native_cfg(cfg)
    dt_code = native.DTYPE_CODE[spec.dtype]
    native.check(L.deca_gemm16_check_config(dt_code, M, N, K, ctypes.byref(ccfg)), f"gemm config {cfg}")
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[spec.dtype]
    cfg_ref = ctypes.byref(ccfg)
    fn = L.deca_gemm16
    ws_bytes = ctypes.c_size_t(0)
    if cfg.stream_k:
        native.check(L.deca_gemm16_workspace_bytes(dt_code, M, N, K, cfg_ref, ctypes.byref(ws_bytes)),
                     "deca_gemm16_workspace_bytes")
    if ws_bytes.value == 0:

        def main(a, b, c):
            _check_tensor(a, (M, K), tdt, "a")
            _check_tensor(b, (K, N), tdt, "b")
            _check_tensor(c, (M, N), tdt, "c")
            native.check(fn(dt_code, a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, cfg_ref,
                            current_stream_ptr()), "deca_gemm16")

        if cfg.stream_k:  # nothing to split for this shape: the plain entry point, whole tiles
            ccfg.stream_k = 0
    else:
        # scratch memory of the stream-K mode: zero once, owned by this module, one launch at a time
        state = {}

        def main(a, b, c):
            _check_tensor(a, (M, K), tdt, "a")
            _check_tensor(b, (K, N), tdt, "b")
            _check_tensor(c, (M, N), tdt, "c")
            ws = state.get(a.device)
            if ws is None:
                ws = state[a.device] = torch.zeros(ws_bytes.value, dtype=torch.uint8, device=a.device)
            native.check(L.deca_gemm16_ws(dt_code, a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, cfg_ref,
                                          ws.data_ptr(), ws_bytes.value, current_stream_ptr()), "deca_gemm16_ws")

    main._keepalive = ccfg
    return main
