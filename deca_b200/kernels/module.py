"""Kernel specs and runtime modules.

In the reference a config becomes a TIR module (``build_mod``), TVM + nvcc turn it into a
shared library (``build_*_to_file``) and ``tvm.runtime.load_module(path)["main"]`` is the
function that is called with DLPack tensors (src/RuntimeMod.py:104-109, :204-208).

Here the kernels are precompiled into one native library that takes shape and config at
run time, so the per-config artefact is a small JSON *spec* (family, shape, dtype, config,
scalars).  ``KernelSpec`` plays the role of the IR module, ``KernelModule`` that of the
loaded runtime module: ``module["main"](*tensors)`` launches the kernel on torch's current
stream with the tensors in the reference's argument order.  Writing a spec needs neither
CUDA nor the native library, so ``build_*_to_file`` keeps working inside spawned compile
workers; binding to the native library happens at load time and raises if it is missing.
"""

from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field

SPEC_MAGIC = "deca_b200.kernel_spec.v1"


@dataclass(frozen=True)
class KernelSpec:
    family: str  # "rowwise" | "gemm" | "flash_attn"
    shape: tuple
    dtype: str
    config: dict
    params: dict = field(default_factory=dict)  # op kind, eps, softmax_scale, causal, ...

    def to_json(self) -> str:
        return json.dumps(
            {"magic": SPEC_MAGIC, "family": self.family, "shape": list(self.shape), "dtype": self.dtype,
             "config": self.config, "params": self.params},
            sort_keys=True,
        )

    @staticmethod
    def from_json(text: str) -> "KernelSpec":
        d = json.loads(text)
        if d.get("magic") != SPEC_MAGIC:
            raise ValueError("not a deca_b200 kernel spec")
        return KernelSpec(d["family"], tuple(d["shape"]), d["dtype"], d["config"], d.get("params", {}))

    def show(self, **_):
        print(self.to_json())

    def export_library(self, path: str) -> str:
        with open(path, "w") as f:
            f.write(self.to_json())
        return path


def _check_tensor(t, shape, torch_dtype, name):
    # one cheap test on the launch path; the messages below only when it fails
    if t.shape == shape and t.dtype == torch_dtype and t.is_cuda and t.is_contiguous():
        return
    if not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    if t.dtype != torch_dtype:
        raise ValueError(f"{name}: expected {torch_dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous tensor")


class KernelModule:
    """A spec bound to the native library; ``module["main"]`` is the launch function."""

    entry_name = "main"

    def __init__(self, spec: KernelSpec):
        from . import flash_attn_b200, gemm_b200, rowwise_b200

        self.spec = spec
        binder = {
            "rowwise": rowwise_b200.bind,
            "gemm": gemm_b200.bind,
            "flash_attn": flash_attn_b200.bind,
        }[spec.family]
        self._main = binder(spec)

    def __getitem__(self, name):
        if name != "main":
            raise KeyError(name)
        return self._main

    def __call__(self, *tensors):
        return self._main(*tensors)

    def export_library(self, path: str) -> str:
        return self.spec.export_library(path)


def load_module(path: str) -> KernelModule:
    """Counterpart of ``tvm.runtime.load_module``: reads a spec file and binds it."""
    with open(path) as f:
        return KernelModule(KernelSpec.from_json(f.read()))


def current_stream_ptr():
    """torch's current stream on the current device as a raw handle (no Stream object is built)."""
    global _raw_stream
    if _raw_stream is None:
        import torch

        _raw_stream = (torch._C._cuda_getCurrentRawStream, torch.cuda.current_device)
    return _raw_stream[0](_raw_stream[1]())


_raw_stream = None
