"""FlashAttention (forward) operator: same record as the reference's
src/operators/FlashAttention.py:17-62; an ``FAConfig`` fully determines the kernel."""

import math

from ..kernels.flash_attn_b200 import FAConfig, check_config, make_flash_attn_fwd
from .Op import Operator


class FlashAttention(Operator):
    def __init__(self, B: int, H: int, S_q: int, S_kv: int, D: int, dtype: str = "float16",
                 softmax_scale: float | None = None, causal: bool = False, name: str = "FlashAttention"):
        """B, H: batch and heads; S_q, S_kv: query / key-value lengths; D: head dim; only
        float16 (fp32 accumulation); softmax_scale defaults to 1/sqrt(D); causal = top-left
        aligned mask (requires S_q == S_kv)."""
        assert dtype == "float16", "FlashAttention only supports float16 inputs"
        self.B, self.H, self.S_q, self.S_kv, self.D = B, H, S_q, S_kv, D
        self.dtype = dtype
        self.softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
        assert not causal or S_q == S_kv, "causal attention requires S_q == S_kv"
        self.causal = causal
        self.num_flops = 4 * B * H * S_q * S_kv * D // (2 if causal else 1)
        self._default_mod = None
        super().__init__(name=name)

    @property
    def shape(self):
        return (self.B, self.H, self.S_q, self.S_kv, self.D)

    def is_valid(self, cfg: FAConfig) -> bool:
        try:
            check_config(cfg, self.S_q, self.S_kv, self.D)
            return True
        except AssertionError:
            return False

    def build_mod(self, cfg: FAConfig):
        return make_flash_attn_fwd(self.B, self.H, self.S_q, self.S_kv, self.D, cfg, self.softmax_scale, self.causal)

    def compile(self, mod):
        from ..kernels.flash_attn_b200 import build_flash_attn

        return build_flash_attn(mod)

    def default_config(self) -> FAConfig:
        # measured on B200 over the FlashAttention-2 grid: two Q tiles per CTA with 128-key tiles and
        # P in tensor memory win at both head dims (S = 4096: 1.09 PFLOPS at D = 128, 0.58 at D = 64);
        # shapes that schedule cannot tile fall back to one Q tile (D = 64: 64-key tiles, P in
        # tensor memory, 0.54 PFLOPS)
        # ... in their persistent form (one CTA per SM walking the Q-tile pairs: +4 % at S = 4096,
        # +30 % at S = 512, where a CTA's start and end cost as much as its four KV steps)
        if self.S_q % 256 == 0 and self.S_kv % 128 == 0:
            stages = 4 if self.S_kv >= 512 else 2
            if self.D == 64 and self.S_kv >= 1024:
                stages = 7 if self.causal else 5  # 16 KB slots: a deeper ring measured 1-3 % faster
            return FAConfig(Bc=128, stages=stages, q_tiles=2, p_tmem=True, persistent=True)
        if self.D == 64 and self.S_kv % 64 == 0:
            return FAConfig(Bc=64, stages=2, p_tmem=True)
        if self.S_kv % 128 == 0:
            return FAConfig(Bc=128, stages=2)
        return FAConfig(Bc=64, stages=2)

    def __call__(self, q, k, v, out=None, cfg: FAConfig | None = None):
        """Runs the kernel: returns O = softmax(scale Q K^T [+ causal mask]) V."""
        import torch

        if cfg is None:
            if self._default_mod is None:
                self._default_mod = self.compile(self.build_mod(self.default_config()))
            mod = self._default_mod
        else:
            mod = self.compile(self.build_mod(cfg))
        if out is None:
            out = torch.empty_like(q)
        mod["main"](q, k, v, out)
        return out

    def make_inputs(self):
        from ..kernels.attn_bench import make_qkv

        return make_qkv(self.B, self.H, self.S_q, self.S_kv, self.D)

    def reference(self, inputs):
        from ..kernels.attn_bench import sdpa_flash

        q, k, v = inputs
        return sdpa_flash(q, k, v, causal=self.causal, scale=self.softmax_scale)

    def kernel_args(self, inputs, out):
        """Tensors in the kernel's argument order: q, k, v, o."""
        return (*inputs, out)

    def describe(self) -> str:
        return (f"{self.name}(B={self.B}, H={self.H}, S_q={self.S_q}, S_kv={self.S_kv}, D={self.D}, {self.dtype}"
                f"{', causal' if self.causal else ''})")
