"""Builds the REFERENCE's own GPU kernels into oracle/_ref/ (test infrastructure, second oracle).

    python oracle/build_ref_kernels.py /path/to/Deca [--jobs 8] [--force]

The reference generates one CUDA kernel per (shape, config) with its TIR generators
(src/kernels/gemm_tir.py:392-407 ``build_gemm_tc_to_file``, flash_attn_tir.py:484-491
``build_flash_attn_to_file``, rowwise_tir.py:402-410 ``build_rowwise_to_file``) and TVM + nvcc.
Apache TVM at the commit the reference pins is not installed; the TVM fork bundled with the
``tilelang`` wheel lowers the same generators (one alias, ``tvm.ffi.register_func``, is applied
here, outside the reference tree).  The kernels are plain ``mma.sync`` / ``ldmatrix`` /
``cp.async`` code, compiled for sm_100a; nothing of the reference is copied into this
repository: the outputs are shared libraries under oracle/_ref/ (git-ignored) plus
``manifest.json`` describing them.  Needs the reference checkout, so it runs where that exists;
the GPU machine only loads the prebuilt files (``oracle/ref_kernels.py``).

What is built: for each benchmark shape a handful of the reference's configs (its defaults and
the choices its cost model ranks first for an H100), so that the comparison on the GPU can take
the reference's best.
"""

from __future__ import annotations

import hashlib
import json
import multiprocessing as mp
import os
import sys
from concurrent.futures import ProcessPoolExecutor

OUT_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
ARCH = "sm_100a"

GEMM_SHAPES = [(1024, 1024, 1024), (4096, 4096, 4096), (8192, 8192, 8192)]
GEMM_CONFIGS = [
    dict(),  # the reference's default: 128x256x32, warp 64x64, 3 stages
    dict(BM=256, BN=128, BK=64, warp_m=64, warp_n=64, stages=3),
    dict(BM=128, BN=256, BK=64, warp_m=64, warp_n=64, stages=3),
    dict(BM=128, BN=128, BK=32, warp_m=64, warp_n=64, stages=4),
    dict(BM=128, BN=128, BK=64, warp_m=64, warp_n=32, stages=3),
]
FA_SHAPES = [((1, 2, 512, 512, 128), False), ((1, 2, 512, 512, 128), True), ((1, 2, 512, 512, 64), True),
             ((4, 16, 4096, 4096, 128), False), ((4, 16, 4096, 4096, 128), True),
             ((4, 16, 4096, 4096, 64), False), ((4, 16, 4096, 4096, 64), True)]
FA_CONFIGS = [
    dict(),  # default: Br=128, Bc=64, 4 warps, 1 stage
    dict(Br=128, Bc=32, num_warps=4, stages=1, q_in_smem=True),
    dict(Br=128, Bc=64, num_warps=8, stages=2),
    dict(Br=64, Bc=64, num_warps=4, stages=2),
    dict(Br=128, Bc=128, num_warps=8, stages=1),
]
ROW_SHAPES = [("softmax", (16384, 4096), "float16"), ("softmax", (16384, 4096), "bfloat16"),
              ("rmsnorm", (16384, 4096), "float16"), ("rmsnorm", (16384, 4096), "bfloat16"),
              ("softmax", (64, 4096), "float16"), ("rmsnorm", (64, 4096), "bfloat16")]
ROW_CONFIGS = [dict(), dict(threads_per_row=64), dict(threads_per_row=256), dict(threads_per_row=128, hint=True)]
RMS_EPS = 1e-6


def _import_reference(ref_root: str):
    import tilelang  # noqa: F401  (makes its bundled tvm importable)
    import tvm

    if not hasattr(tvm.ffi, "register_func"):
        tvm.ffi.register_func = tvm.ffi.register_global_func
    for p in (os.path.join(ref_root, "src"), ref_root):
        if p not in sys.path:
            sys.path.insert(0, p)


def _build_one(job):
    """Runs in a spawned worker (as the reference's CLIs do): returns the manifest entry or an error."""
    ref_root, family, name, path, spec = job
    try:
        _import_reference(ref_root)
        if family == "gemm":
            from kernels.gemm_tir import GemmConfig, build_gemm_tc_to_file, check_config

            cfg = GemmConfig(**spec["config"])
            check_config(cfg, *spec["shape"])
            build_gemm_tc_to_file(tuple(spec["shape"]), cfg, ARCH, path)
        elif family == "flash_attn":
            from kernels.flash_attn_tir import FAConfig, build_flash_attn_to_file, check_config

            cfg = FAConfig(**spec["config"])
            B, H, S_q, S_kv, D = spec["shape"]
            check_config(cfg, S_q, S_kv, D)
            build_flash_attn_to_file(tuple(spec["shape"]), cfg, spec["softmax_scale"], ARCH, path, causal=spec["causal"])
        else:
            from kernels.rowwise_tir import RowConfig, build_rowwise_to_file, check_config

            cfg = RowConfig(**spec["config"])
            check_config(cfg, spec["op"], *spec["shape"], spec["dtype"])
            build_rowwise_to_file(spec["op"], tuple(spec["shape"]), spec["dtype"], cfg, spec["eps"], ARCH, path)
        entry = dict(spec, family=family, name=name, file=os.path.basename(path), config_str=str(cfg))
        return entry, None
    except Exception as e:  # noqa: BLE001  (invalid config for the shape, lowering error)
        return None, f"{name}: {type(e).__name__}: {str(e)[-200:]}"


def jobs_for(ref_root: str):
    jobs = []

    def add(family, spec):
        tag = hashlib.sha1(json.dumps(spec, sort_keys=True).encode()).hexdigest()[:10]
        name = f"{family}_{tag}"
        jobs.append((ref_root, family, name, os.path.join(OUT_DIR, name + ".so"), spec))

    for shape in GEMM_SHAPES:
        for cfg in GEMM_CONFIGS:
            add("gemm", {"shape": list(shape), "dtype": "float16", "config": cfg})
    for shape, causal in FA_SHAPES:
        for cfg in FA_CONFIGS:
            add("flash_attn", {"shape": list(shape), "dtype": "float16", "config": cfg, "causal": causal,
                               "softmax_scale": shape[4] ** -0.5})
    for op, shape, dtype in ROW_SHAPES:
        for cfg in ROW_CONFIGS:
            add("rowwise", {"op": op, "shape": list(shape), "dtype": dtype, "config": cfg, "eps": RMS_EPS})
    return jobs


def build(ref_root: str, jobs: int = 8, force: bool = False) -> str:
    """Builds what is missing; returns the manifest path."""
    os.makedirs(OUT_DIR, exist_ok=True)
    manifest_path = os.path.join(OUT_DIR, "manifest.json")
    have = {}
    if os.path.exists(manifest_path) and not force:
        with open(manifest_path) as f:
            have = {e["name"]: e for e in json.load(f)["kernels"]}
    todo, entries, errors = [], [], []
    for job in jobs_for(ref_root):
        name, path = job[2], job[3]
        if name in have and os.path.exists(path):
            entries.append(have[name])
        else:
            todo.append(job)
    if todo:
        with ProcessPoolExecutor(max_workers=max(1, jobs), mp_context=mp.get_context("spawn")) as pool:
            for entry, err in pool.map(_build_one, todo):
                (entries if entry else errors).append(entry or err)
    with open(manifest_path, "w") as f:
        json.dump({"arch": ARCH, "generator": "reference TIR generators lowered by the TVM bundled with tilelang",
                   "kernels": sorted(entries, key=lambda e: e["name"]), "skipped": sorted(errors)}, f, indent=1)
    return manifest_path


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    n_jobs = int(sys.argv[sys.argv.index("--jobs") + 1]) if "--jobs" in sys.argv else 8
    path = build(sys.argv[1], n_jobs, "--force" in sys.argv)
    with open(path) as f:
        m = json.load(f)
    print(f"{len(m['kernels'])} kernels in {OUT_DIR}; skipped {len(m['skipped'])}")
    for s in m["skipped"]:
        print("  skipped", s)
