"""16-bit tensor-core GEMM operator (C = A @ B, fp32 accumulation, 16-bit output).

Same record as the reference's src/operators/GEMMTC.py:19-111.  ``acc="fp16"`` selects fp16
accumulators (``GemmConfig.acc_f16``: the accumulator type of tcgen05.mma set to f16, every
16-deep partial sum rounded to fp16, the reference's looser tolerance for that mode);
``acc_splits`` is accepted and recorded (it enters the tolerance and ``describe()`` as in the
reference) but the tensor-memory accumulator is a single one.  ``dtype`` may also be
"bfloat16" (fp32 accumulation only).
"""

import math

from ..kernels.gemm_b200 import GemmConfig, check_config, make_gemm_tc
from .Op import Operator


class GEMMTC(Operator):
    # RuntimeMod reports compute-bound kernels in TFLOPS.
    metric = "TFLOPS"

    def __init__(self, M: int, N: int, K: int, dtype: str = "float16", acc: str = "fp32", acc_splits: int = 1,
                 name: str = "GEMMTC"):
        assert dtype in ("float16", "bfloat16"), "GEMMTC only supports float16 / bfloat16 inputs"
        assert acc in ("fp32", "fp16")
        assert acc == "fp32" or dtype == "float16", "fp16 accumulation needs float16 inputs"
        self.M, self.N, self.K = M, N, K
        self.dtype = dtype
        self.acc = acc
        self.acc_splits = acc_splits if acc == "fp16" else 1
        self.num_flops = 2 * M * N * K
        self._default_mod = None
        super().__init__(name=name)

    @property
    def shape(self):
        return (self.M, self.N, self.K)

    @property
    def tolerance(self):
        """(atol, rtol) vs the fp32 reference: 16-bit output rounding is ~5e-4 (fp16) or ~4e-3
        (bf16) relative, the accumulation error grows like sqrt(K)."""
        if self.acc == "fp16":  # the reference's bound for its fp16 accumulators (GEMMTC.py:61-62)
            return (2e-3 * self.K / math.sqrt(self.acc_splits), 1e-2)
        if self.dtype == "bfloat16":
            return (1e-2 * math.sqrt(self.K / 1024), 1.6e-2)
        return (1e-2 * math.sqrt(self.K / 1024), 2e-3)

    def is_valid(self, cfg: GemmConfig) -> bool:
        if cfg.acc_f16 != (self.acc == "fp16"):  # as the reference does (GEMMTC.py:65-67)
            return False
        try:
            check_config(cfg, self.M, self.N, self.K)
            return True
        except AssertionError:
            return False

    def build_mod(self, cfg: GemmConfig):
        return make_gemm_tc(self.M, self.N, self.K, cfg, self.dtype)

    def compile(self, mod):
        from ..kernels.gemm_b200 import build_gemm_tc

        return build_gemm_tc(mod)

    def default_config(self) -> GemmConfig:
        from ..kernels.gemm_b200 import default_config

        return default_config(self.M, self.N, self.K, acc_f16=self.acc == "fp16")

    def __call__(self, a, b, out=None, cfg: GemmConfig | None = None):
        """Runs the kernel: returns C = A @ B."""
        if cfg is None:
            if self._default_mod is None:
                self._default_mod = self.compile(self.build_mod(self.default_config()))
            mod = self._default_mod
        else:
            mod = self.compile(self.build_mod(cfg))
        if out is None:
            out = self.make_output((a, b))
        mod["main"](a, b, out)
        return out

    def make_inputs(self):
        import torch

        from ..kernels.gemm_bench import make_inputs

        return make_inputs(self.M, self.N, self.K, dtype=getattr(torch, self.dtype))

    def make_output(self, inputs):
        import torch

        return torch.empty(self.M, self.N, device="cuda", dtype=getattr(torch, self.dtype))

    def reference(self, inputs):
        """fp32 GEMM of the 16-bit inputs (torch's own 16-bit GEMM may use reduced-precision
        reductions, so it is not used as the reference)."""
        import torch

        a, b = inputs
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            return a.float() @ b.float()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = tf32

    def kernel_args(self, inputs, out):
        """Tensors in the kernel's argument order: a, b, c."""
        return (*inputs, out)

    def describe(self) -> str:
        acc = f", acc=fp16x{self.acc_splits}" if self.acc == "fp16" else ""  # the reference's form (GEMMTC.py:109-111)
        return f"{self.name}(M={self.M}, N={self.N}, K={self.K}, {self.dtype}{acc})"
