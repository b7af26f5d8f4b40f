"""One kernel config, loaded, checked against torch and timed: the harness the tuning CLIs drive.

The surface is the reference's ``RuntimeMod`` (src/RuntimeMod.py:14-238): constructor
``(operator, arch, use_tc, compute_pattern)``; ``build`` / ``load_kernel`` / ``load_flash_attn``
produce ``runtime_mod`` whose ``["main"]`` takes the tensors in ``operator.kernel_args`` order;
``time_evaluator`` fills ``execution_time`` (seconds), ``throughput`` (TFLOPS, or GB/s for the
memory-bound operators), ``max_error`` and ``record`` (the line the CLIs print, :185-190 and
:235-238).  A kernel whose result is out of tolerance raises ``RuntimeError``, which the CLIs
report as "is not a valid config" (test_gemm_tc.py:126-132).  The reference's legacy
TVM-schedule paths (``build_with_tc`` / ``build_without_tc``) have no counterpart here.
"""

from __future__ import annotations

from .arch.Arch import Arch
from .kernels.module import load_module
from .operators.FlashAttention import FlashAttention
from .operators.Op import Operator

# Rows of the reference output converted to fp32 at a time while checking (bounds the temporaries
# for vocabulary-sized rows): about 16 Mi elements.
CHECK_CHUNK_ELEMENTS = 1 << 24


def worst_excess(out, ref, atol: float, rtol: float):
    """(max |out - ref|, max |out - ref| / (atol + rtol |ref|)) over row chunks, as Python floats."""
    rows = max(1, CHECK_CHUNK_ELEMENTS // ref.shape[-1])
    max_err = ratio = 0.0
    for r0 in range(0, ref.shape[0], rows):
        want = ref[r0 : r0 + rows].float()
        err = (out[r0 : r0 + rows].float() - want).abs_()
        max_err = max(max_err, err.max().item())
        ratio = max(ratio, err.div_(want.abs_().mul_(rtol).add_(atol)).max().item())
    return max_err, ratio


class RuntimeMod:
    def __init__(self, operator: Operator, arch: Arch, use_tc: bool, compute_pattern):
        """``compute_pattern`` is the operator's config object (GemmConfig / FAConfig / RowConfig);
        ``use_tc`` is accepted for call-site compatibility (every kernel here is config-driven)."""
        self.operator = operator
        self.arch = arch
        self.use_tc = use_tc
        self.compute_pattern = compute_pattern
        self.ir_mod = None
        self.runtime_mod = None
        self.execution_time: float = 0.0
        self.throughput: float = 0.0
        self.max_error: float = float("nan")
        self.record: str = ""

    # ------------------------------------------------------------------ producing the module
    @property
    def is_flash_attn(self) -> bool:
        return isinstance(self.operator, FlashAttention)

    @property
    def is_kernel_op(self) -> bool:
        return hasattr(self.operator, "build_mod")

    def build(self):
        """In-process: config -> kernel spec -> bound module."""
        if not self.is_kernel_op:
            raise NotImplementedError("only config-driven operators (build_mod) are supported")
        self.ir_mod = self.operator.build_mod(self.compute_pattern)
        self.runtime_mod = self.operator.compile(self.ir_mod)

    build_flash_attn = build

    def load_kernel(self, path: str):
        """Binds a kernel file written by one of the ``build_*_to_file`` functions."""
        self.ir_mod = self.operator.build_mod(self.compute_pattern)
        self.runtime_mod = load_module(path)

    load_flash_attn = load_kernel

    def get_mod(self):
        return self.ir_mod

    def show(self):
        self.get_mod().show()

    # ------------------------------------------------------------------ verify + time
    def time_evaluator(self):
        return self.time_flash_attn() if self.is_flash_attn else self.time_kernel_op()

    def _run_checked(self, args, out, reference, atol, rtol, verify):
        """Launches once and compares with ``reference()``; then times the launch."""
        import torch

        from .kernels.timing import bench_cuda

        launch = self.runtime_mod["main"]
        if verify:
            launch(*args)
            torch.cuda.synchronize()
            ref = reference()
            self.max_error, ratio = worst_excess(out.reshape(-1, out.shape[-1]), ref.reshape(-1, ref.shape[-1]), atol, rtol)
            del ref
            if not ratio <= 1.0:
                return ratio
        self.execution_time = bench_cuda(lambda: launch(*args))
        return 0.0

    def time_flash_attn(self, verify: bool = True, atol: float = 2e-2):
        """Attention: max-abs error against SDPA-flash on the same seeded tensors must be <= atol."""
        import torch

        op = self.operator
        q, k, v = op.make_inputs()
        o = torch.empty_like(q)
        bad = self._run_checked(op.kernel_args((q, k, v), o), o, lambda: op.reference((q, k, v)), atol, 0.0, verify)
        if bad:
            raise RuntimeError(f"{self.compute_pattern}: max error {self.max_error} exceeds {atol}")
        B, H, S_q, S_kv, D = op.shape
        self.throughput = op.num_flops / self.execution_time / 1e12
        self.record = (
            f"{op.name}(B={B}, H={H}, S_q={S_q}, S_kv={S_kv}, D={D}, {op.dtype}"
            f"{', causal' if op.causal else ''}) "
            f"\n\t{self.compute_pattern} \n\tcost time: {self.execution_time * 1000:.4f} ms, "
            f"throughput: {self.throughput:.2f} TFLOPS, max err: {self.max_error:.2e}"
        )

    def time_kernel_op(self, verify: bool = True):
        """GEMM and row-wise operators: |out - ref| <= atol + rtol |ref| element-wise against the
        operator's torch reference, with the operator's own (atol, rtol)."""
        import torch

        op = self.operator
        inputs = op.make_inputs()
        out = op.make_output(inputs) if hasattr(op, "make_output") else torch.empty_like(inputs[0])
        atol, rtol = op.tolerance
        bad = self._run_checked(op.kernel_args(inputs, out), out, lambda: op.reference(inputs), atol, rtol, verify)
        if bad:
            raise RuntimeError(
                f"{self.compute_pattern}: max error {self.max_error:.3e} exceeds "
                f"atol={atol} + rtol={rtol} * |ref| (x{bad:.2f})"
            )
        if getattr(op, "metric", "GB/s") == "TFLOPS":
            self.throughput, unit = op.num_flops / self.execution_time / 1e12, "TFLOPS"
        else:
            self.throughput, unit = op.num_bytes / self.execution_time / 1e9, "GB/s"
        self.record = (
            f"{op.describe()} \n\t{self.compute_pattern} \n\tcost time: {self.execution_time * 1000:.4f} ms, "
            f"throughput: {self.throughput:.1f} {unit}, max err: {self.max_error:.2e}"
        )
