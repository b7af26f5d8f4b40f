"""Loader for the reference's own GPU kernels prebuilt under oracle/_ref/ (test infrastructure).

``oracle/build_ref_kernels.py`` writes the shared libraries and ``manifest.json`` where the
reference checkout exists; here they are only loaded, through the TVM runtime bundled with the
``tilelang`` wheel, and called with torch tensors shared by DLPack, exactly as the reference's
harness calls them (src/RuntimeMod.py:104-109, :169-172, :204-208).  Used by the GPU tests as a
second oracle and by ``bench.py`` as the like-for-like baseline; never by the product package.
"""

from __future__ import annotations

import json
import os

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_tvm = None


def unavailable_reason() -> str | None:
    """None when the prebuilt kernels can be used here, else why not (one line)."""
    if not os.path.exists(os.path.join(REF_DIR, "manifest.json")):
        return "oracle/_ref/manifest.json is missing (run oracle/build_ref_kernels.py where the reference checkout is)"
    try:
        _runtime()
    except Exception as e:  # noqa: BLE001
        return f"TVM runtime not importable: {type(e).__name__}: {str(e)[-120:]}"
    return None


def _runtime():
    global _tvm
    if _tvm is None:
        import tilelang  # noqa: F401  (puts its bundled tvm on the path)
        import tvm

        _tvm = tvm
    return _tvm


def manifest() -> dict:
    with open(os.path.join(REF_DIR, "manifest.json")) as f:
        return json.load(f)


def entries(family: str, shape=None, **params):
    """Manifest entries of a family, optionally for one shape and parameter values (op, dtype, causal)."""
    out = []
    for e in manifest()["kernels"]:
        if e["family"] != family or (shape is not None and tuple(e["shape"]) != tuple(shape)):
            continue
        if all(e.get(k) == v for k, v in params.items()):
            out.append(e)
    return out


def bind(entry: dict, *tensors):
    """A zero-argument launcher of the kernel on the given torch CUDA tensors (kernel argument
    order).  The TVM runtime launches on the legacy default stream, as in the reference."""
    tvm = _runtime()
    mod = tvm.runtime.load_module(os.path.join(REF_DIR, entry["file"]))
    func = mod["main"]
    args = [tvm.runtime.from_dlpack(t) for t in tensors]

    def launch():
        func(*args)

    launch._keepalive = (mod, args, tensors)
    return launch
