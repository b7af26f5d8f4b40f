"""Row-wise memory-bound operators over an [M, N] input (reduction over N): the base record and
its two operators.

Same records as the reference's src/operators/Rowwise.py:23-73, Softmax.py:8-18 and
RMSNorm.py:9-22: a ``RowConfig`` fully determines the kernel; the operator provides the inputs,
the torch reference and the tolerance RuntimeMod verifies against.  Calling the operator runs the
kernel.  ``Softmax(M, N, dtype)``: y = softmax(x, -1).  ``RMSNorm(M, N, dtype, eps)``:
y = x * rsqrt(mean(x^2) + eps) * w.  dtype "float16" / "bfloat16" (or "fp16" / "bf16"), fp32 math.
"""

from ..kernels.rowwise_b200 import RowConfig, check_config, make_rowwise
from .Op import Operator

# (atol, rtol) of the comparison with torch: |y - ref| <= atol + rtol * |ref|
TOLERANCE = {
    ("softmax", "float16"): (1e-5, 1e-2),
    ("softmax", "bfloat16"): (1e-5, 3e-2),
    ("rmsnorm", "float16"): (1e-2, 1e-2),
    ("rmsnorm", "bfloat16"): (3e-2, 3e-2),
}


class RowwiseOperator(Operator):
    op_kind: str = ""

    def __init__(self, M: int, N: int, dtype: str = "float16", eps: float = 1e-6, name: str = ""):
        from ..kernels.rowwise_bench import canonical_dtype, rowwise_bytes

        self.M, self.N = M, N
        self.dtype = canonical_dtype(dtype)
        self.eps = eps
        self.num_bytes = rowwise_bytes(self.op_kind, M, N)
        self._default_mod = None
        super().__init__(name=name or type(self).__name__)

    @property
    def shape(self):
        return (self.M, self.N)

    @property
    def tolerance(self):
        return TOLERANCE[(self.op_kind, self.dtype)]

    def is_valid(self, cfg: RowConfig) -> bool:
        try:
            check_config(cfg, self.op_kind, self.M, self.N, self.dtype)
            return True
        except AssertionError:
            return False

    def build_mod(self, cfg: RowConfig):
        return make_rowwise(self.op_kind, self.M, self.N, self.dtype, cfg, self.eps)

    def compile(self, mod):
        from ..kernels.rowwise_b200 import build_rowwise

        return build_rowwise(mod)

    def default_config(self) -> RowConfig:
        """The config the native library picks for this shape when none is given."""
        import ctypes

        from .. import native

        c = native.RowCfg()
        native.check(
            native.lib().deca_rowwise_default_config(
                native.ROW_OP_CODE[self.op_kind], native.DTYPE_CODE[self.dtype], self.M, self.N, ctypes.byref(c)
            ),
            "deca_rowwise_default_config",
        )
        return RowConfig(c.threads_per_row, c.rows_per_block, c.vec, native.ROW_MODE_NAME[c.mode], c.unroll,
                         bool(c.hint))

    def __call__(self, *inputs, out=None, cfg: RowConfig | None = None):
        """Runs the kernel on ``inputs`` (x[, w]); returns y."""
        import torch

        if cfg is None:
            if self._default_mod is None:
                self._default_mod = self.compile(self.build_mod(self.default_config()))
            mod = self._default_mod
        else:
            mod = self.compile(self.build_mod(cfg))
        if out is None:
            out = torch.empty_like(inputs[0])
        mod["main"](*self.kernel_args(inputs, out))
        return out

    def make_inputs(self):
        from ..kernels.rowwise_bench import make_inputs

        return make_inputs(self.op_kind, self.M, self.N, self.dtype)

    def reference(self, inputs):
        from ..kernels.rowwise_bench import torch_ref

        return torch_ref(self.op_kind, inputs, self.eps)

    def kernel_args(self, inputs, out):
        """Tensors in the kernel's argument order: x[, w], y."""
        return (*inputs, out)

    def describe(self) -> str:
        return f"{self.name}(M={self.M}, N={self.N}, {self.dtype})"


class Softmax(RowwiseOperator):
    op_kind = "softmax"

    def __init__(self, M: int, N: int, dtype: str = "float16", name: str = "Softmax"):
        super().__init__(M, N, dtype, name=name)


class RMSNorm(RowwiseOperator):
    op_kind = "rmsnorm"

    def __init__(self, M: int, N: int, dtype: str = "float16", eps: float = 1e-6, name: str = "RMSNorm"):
        super().__init__(M, N, dtype, eps, name=name)
