"""Build-or-load one kernel config, verify it against the operator's torch reference and
time it -- the harness the tuning CLIs drive (same surface and record strings as the
reference's src/RuntimeMod.py:14-238, minus its TVM-schedule legacy paths)."""

from .arch.Arch import Arch
from .kernels.module import load_module
from .operators.FlashAttention import FlashAttention
from .operators.Op import Operator


class RuntimeMod:
    def __init__(self, operator: Operator, arch: Arch, use_tc: bool, compute_pattern):
        """operator: kernel to be tuned; arch: the GPU model; compute_pattern: the operator's
        config object (GemmConfig / FAConfig / RowConfig).  ``use_tc`` is kept for call-site
        compatibility; every operator here generates its kernel from a config."""
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

    @property
    def is_flash_attn(self) -> bool:
        return isinstance(self.operator, FlashAttention)

    @property
    def is_kernel_op(self) -> bool:
        """Operators that generate their kernel from a config (``build_mod``)."""
        return hasattr(self.operator, "build_mod")

    def build(self):
        """Builds the runtime module in-process."""
        if not self.is_kernel_op:
            raise NotImplementedError("only config-driven operators (build_mod) are supported")
        self.ir_mod = self.operator.build_mod(self.compute_pattern)
        self.runtime_mod = self.operator.compile(self.ir_mod)

    def build_flash_attn(self):
        self.build()

    def load_flash_attn(self, path: str):
        """Loads a FlashAttention kernel exported by ``build_flash_attn_to_file``."""
        self.load_kernel(path)

    def load_kernel(self, path: str):
        """Loads a kernel of a ``build_mod`` operator exported to a file."""
        self.ir_mod = self.operator.build_mod(self.compute_pattern)
        self.runtime_mod = load_module(path)

    def show(self):
        self.get_mod().show()

    def get_mod(self):
        return self.ir_mod

    def time_evaluator(self):
        """Verifies and times the runtime module; fills execution_time, throughput, max_error, record."""
        if self.is_flash_attn:
            return self.time_flash_attn()
        return self.time_kernel_op()

    def time_flash_attn(self, verify: bool = True, atol: float = 2e-2):
        """Times (and verifies against torch SDPA) the FlashAttention kernel on tensors shared
        with the baseline, with the same CUDA-event harness."""
        import torch

        from .kernels.attn_bench import bench_cuda, make_qkv, sdpa_flash

        op = self.operator
        B, H, S_q, S_kv, D = op.shape
        q, k, v = make_qkv(B, H, S_q, S_kv, D)
        o = torch.empty_like(q)
        args = (q, k, v, o)
        func = self.runtime_mod["main"]

        if verify:
            func(*args)
            torch.cuda.synchronize()
            ref = sdpa_flash(q, k, v, causal=op.causal, scale=op.softmax_scale)
            self.max_error = (o.float() - ref.float()).abs().max().item()
            if not self.max_error <= atol:
                raise RuntimeError(f"{self.compute_pattern}: max error {self.max_error} exceeds {atol}")

        t = bench_cuda(lambda: func(*args))
        self.execution_time = t
        self.throughput = op.num_flops / t / 1e12
        self.record = (
            f"{op.name}(B={B}, H={H}, S_q={S_q}, S_kv={S_kv}, D={D}, {op.dtype}"
            f"{', causal' if op.causal else ''}) "
            f"\n\t{self.compute_pattern} \n\tcost time: {t * 1000:.4f} ms, "
            f"throughput: {self.throughput:.2f} TFLOPS, max err: {self.max_error:.2e}"
        )

    def time_kernel_op(self, verify: bool = True):
        """Times (and verifies against the operator's torch reference) a ``build_mod`` operator.
        Throughput is GB/s for memory-bound operators, TFLOPS when ``metric == "TFLOPS"``."""
        import torch

        from .kernels.attn_bench import bench_cuda

        op = self.operator
        inputs = op.make_inputs()
        out = op.make_output(inputs) if hasattr(op, "make_output") else torch.empty_like(inputs[0])
        args = op.kernel_args(inputs, out)
        func = self.runtime_mod["main"]

        if verify:
            func(*args)
            torch.cuda.synchronize()
            ref = op.reference(inputs)
            atol, rtol = op.tolerance
            self.max_error, excess = 0.0, 0.0
            # Row chunks keep the fp32 temporaries small for vocab-sized inputs.
            step = max(1, (1 << 24) // ref.shape[-1])
            for r0 in range(0, ref.shape[0], step):
                r = ref[r0 : r0 + step].float()
                diff = (out[r0 : r0 + step].float() - r).abs()
                self.max_error = max(self.max_error, diff.max().item())
                excess = max(excess, (diff / (atol + rtol * r.abs())).max().item())
            del ref
            if not excess <= 1.0:
                raise RuntimeError(
                    f"{self.compute_pattern}: max error {self.max_error:.3e} exceeds "
                    f"atol={atol} + rtol={rtol} * |ref| (x{excess:.2f})"
                )

        t = bench_cuda(lambda: func(*args))
        self.execution_time = t
        if getattr(op, "metric", "GB/s") == "TFLOPS":
            self.throughput = op.num_flops / t / 1e12
            unit = "TFLOPS"
        else:
            self.throughput = op.num_bytes / t / 1e9
            unit = "GB/s"
        self.record = (
            f"{op.describe()} \n\t{self.compute_pattern} \n\tcost time: {t * 1000:.4f} ms, "
            f"throughput: {self.throughput:.1f} {unit}, max err: {self.max_error:.2e}"
        )
