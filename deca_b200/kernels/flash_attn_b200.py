"""FlashAttention forward configs for B200 and their binding to the native library.

Mirrors the module-level surface of the reference's src/kernels/flash_attn_tir.py --
``FAConfig`` (:31-51), ``smem_bytes`` (:54-56), ``check_config`` (:70-80),
``make_flash_attn_fwd`` (:83), ``build_flash_attn`` (:494-501), ``build_flash_attn_to_file``
(:484-491) -- with the tile space of the tcgen05 kernel in csrc/fa_fwd_f16.cu: a Q tile is
128 rows (the tensor-memory lanes), S = Q K^T and O accumulate in tensor memory, K/V tiles
of ``Bc`` keys stream through a TMA ring of ``stages`` slots, and ``q_tiles = 2`` lets one
CTA alternate between two Q tiles so the softmax of one overlaps the MMAs of the other.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass

from .module import KernelModule, KernelSpec, _check_tensor, current_stream_ptr

LOG2E = 1.4426950408889634
NEG_INF = -1e30
MAX_DYN_SMEM = 232448
TMEM_COLUMNS = 512


@dataclass(frozen=True)
class FAConfig:
    Br: int = 128  # Q rows per tile (tensor-memory lanes)
    Bc: int = 128  # KV rows per pipeline step
    stages: int = 2  # K/V shared-memory ring depth (q_tiles = 2: slots of the ring K and V share)
    q_tiles: int = 1  # Q tiles a CTA works on alternately (1 or 2)
    p_tmem: bool = False  # keep P in tensor memory (MMA A operand) instead of shared memory
    persistent: bool = False  # one CTA per SM walks the (head, Q-tile pair) items (q_tiles = 2, Bc = 128, p_tmem)

    @property
    def threads(self) -> int:
        # TMA warp + MMA warp + one softmax warpgroup per Q tile (+ correction inside it)
        return 64 + 128 * self.q_tiles

    def as_dict(self):
        return asdict(self)

    def __str__(self):
        return (f"Br={self.Br},Bc={self.Bc},stages={self.stages},q_tiles={self.q_tiles}"
                + (",p_tmem=1" if self.p_tmem else "") + (",persistent=1" if self.persistent else ""))


def smem_bytes(cfg: FAConfig, D: int) -> int:
    q = cfg.q_tiles * cfg.Br * D * 2
    if cfg.persistent:
        return q + cfg.stages * cfg.Bc * D * 2 + 8 * 4096 + 2048  # ring + O staging panels
    if cfg.q_tiles == 2:
        kv = cfg.stages * cfg.Bc * D * 2  # one ring shared by K and V tiles
        p = 0 if cfg.p_tmem else 2 * cfg.Br * cfg.Bc * 2  # one P tile per Q tile
    else:
        kv = 2 * cfg.stages * cfg.Bc * D * 2  # a K ring and a V ring
        p = 0 if cfg.p_tmem else 2 * cfg.Br * cfg.Bc * 2  # double-buffered P
    return q + kv + p + 2048


def tmem_columns(cfg: FAConfig, D: int) -> int:
    # q_tiles = 1: two score buffers + O; q_tiles = 2: per Q tile one 128-key or two 64-key score
    # buffers and one O
    cols = (2 * cfg.Bc if cfg.q_tiles == 1 else 256) + cfg.q_tiles * D
    p = 32
    while p < cols:
        p *= 2
    return p


def check_config(cfg: FAConfig, S_q: int, S_kv: int, D: int) -> None:
    assert D in (64, 128), "head dim 64 or 128"
    assert cfg.Br == 128
    assert cfg.Bc in (64, 128)
    assert cfg.q_tiles in (1, 2)
    if cfg.persistent:
        assert cfg.q_tiles == 2 and cfg.Bc == 128 and cfg.p_tmem
    if cfg.q_tiles == 2:
        # 64-key tiles: P must live in tensor memory and K_{j+2}, V_j, V_{j+1} are in flight together
        assert cfg.Bc == 128 or cfg.p_tmem
        assert (4 if cfg.Bc == 64 else 2) <= cfg.stages <= 8
    else:
        assert 1 <= cfg.stages <= 4
    assert S_q % (cfg.Br * cfg.q_tiles) == 0 and S_kv % cfg.Bc == 0
    assert smem_bytes(cfg, D) <= MAX_DYN_SMEM
    assert tmem_columns(cfg, D) <= TMEM_COLUMNS


def make_flash_attn_fwd(B: int, H: int, S_q: int, S_kv: int, D: int, cfg: FAConfig,
                        softmax_scale: float | None = None, causal: bool = False) -> KernelSpec:
    """``causal`` applies the top-left aligned mask (key j visible to query i iff j <= i)."""
    check_config(cfg, S_q, S_kv, D)
    assert not causal or S_q == S_kv, "causal attention requires S_q == S_kv"
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    return KernelSpec("flash_attn", (B, H, S_q, S_kv, D), "float16", cfg.as_dict(),
                      {"softmax_scale": float(scale), "causal": bool(causal)})


def build_flash_attn(mod: KernelSpec, target=None, dump_dir=None) -> KernelModule:
    return KernelModule(mod)


def build_flash_attn_to_file(shape, cfg: FAConfig, softmax_scale, arch: str, path: str, causal: bool = False) -> str:
    """Writes the kernel spec to ``path`` (safe in a worker process without a CUDA context)."""
    B, H, S_q, S_kv, D = shape
    return make_flash_attn_fwd(B, H, S_q, S_kv, D, cfg, softmax_scale, causal).export_library(path)


def native_cfg(cfg: FAConfig):
    from .. import native

    return native.FaCfg(cfg.Br, cfg.Bc, cfg.stages, cfg.q_tiles, int(cfg.p_tmem), int(cfg.persistent))


def bind(spec: KernelSpec):
    """Returns main(q, k, v, o) launching deca_fa_fwd_f16 on torch's current stream."""
    import ctypes

    import torch

    from .. import native

    L = native.lib()
    B, H, S_q, S_kv, D = spec.shape
    cfg = FAConfig(**spec.config)
    ccfg = native_cfg(cfg)
    scale = ctypes.c_float(spec.params["softmax_scale"])
    causal = int(spec.params["causal"])
    native.check(L.deca_fa_fwd_f16_check_config(B, H, S_q, S_kv, D, causal, ctypes.byref(ccfg)), f"fa config {cfg}")
    cfg_ref = ctypes.byref(ccfg)
    fn = L.deca_fa_fwd_f16

    def main(q, k, v, o):
        _check_tensor(q, (B, H, S_q, D), torch.float16, "q")
        _check_tensor(k, (B, H, S_kv, D), torch.float16, "k")
        _check_tensor(v, (B, H, S_kv, D), torch.float16, "v")
        _check_tensor(o, (B, H, S_q, D), torch.float16, "o")
        native.check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, S_q, S_kv, D, scale, causal,
                        cfg_ref, current_stream_ptr()), "deca_fa_fwd_f16")

    main._keepalive = ccfg
    return main
