"""Generates the golden fixtures in this directory from the REFERENCE's own Python code.

Run once where the reference checkout is available (it is not on the GPU machine):

    python tests/golden/make_golden.py /path/to/Deca

The reference needs Apache TVM only to import; the TVM bundled with the ``tilelang``
wheel is enough for that and for building the reference's naive TIR GEMM for the ``c``
target.  Everything else is the reference's torch code run on the CPU:

* ``kernels.rowwise_bench.torch_ref``       softmax / RMSNorm, fp16 and bf16
* ``operators.GEMMTC.GEMMTC.reference``     fp32 GEMM of fp16 inputs (+ tolerance, flops, describe)
* ``kernels.attn_bench.sdpa_flash``         attention forward, causal and not
* ``operators.GEMM.create_gemm_ir_module``  the unscheduled fp32 GEMM, compiled TIR -> C -> gcc
* shape grids and work formulas of the three ``*_bench`` modules

Inputs are drawn with CPU generators (the seeds and distributions of the benchmark
configurations), stored with the outputs, so the fixtures are self-contained.
"""

import json
import os
import sys

import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(ref_root: str):
    import tilelang  # noqa: F401  (makes its bundled tvm importable)
    import tvm

    if not hasattr(tvm.ffi, "register_func"):
        tvm.ffi.register_func = tvm.ffi.register_global_func
    sys.path[:0] = [os.path.join(ref_root, "src"), ref_root]
    from kernels import attn_bench, gemm_bench, rowwise_bench
    from operators.FlashAttention import FlashAttention
    from operators.GEMM import create_gemm_ir_module
    from operators.GEMMTC import GEMMTC
    from operators.RMSNorm import RMSNorm
    from operators.Softmax import Softmax

    out = os.path.dirname(os.path.abspath(__file__))
    arrays, meta = {}, {}

    # ---- row-wise: X = 3 * N(0,1), W = N(1, 0.1), seed 1 ----
    for dt_name, tdt in (("float16", torch.float16), ("bfloat16", torch.bfloat16)):
        for tag, (M, N) in (("hid", (2, 4096)), ("ragged", (3, 1000)), ("vocab", (1, 32000))):
            g = torch.Generator(device="cpu").manual_seed(1)
            x = (3.0 * torch.randn(M, N, generator=g)).to(tdt)
            w = (1.0 + 0.1 * torch.randn(N, generator=g)).to(tdt)
            arrays[f"row_{tag}_{dt_name}_x"] = bits(x)
            arrays[f"row_{tag}_{dt_name}_softmax"] = bits(rowwise_bench.torch_ref("softmax", (x,)))
            if tag == "vocab":  # the reference sweeps vocabulary-sized rows for softmax only
                continue
            arrays[f"row_{tag}_{dt_name}_w"] = bits(w)
            arrays[f"row_{tag}_{dt_name}_rmsnorm"] = bits(rowwise_bench.torch_ref("rmsnorm", (x, w), 1e-6))

    # ---- fp16 GEMM: A, B ~ U[-1, 1], seed 2; reference = fp32 matmul of the fp16 inputs ----
    g = torch.Generator(device="cpu").manual_seed(2)
    M, N, K = 64, 80, 96
    a = (torch.rand(M, K, generator=g) * 2 - 1).half()
    b = (torch.rand(K, N, generator=g) * 2 - 1).half()
    op = GEMMTC(M, N, K)
    arrays["gemm_a"], arrays["gemm_b"] = bits(a), bits(b)
    arrays["gemm_c32"] = op.reference((a, b)).numpy()
    meta["gemmtc"] = []
    for shape in ((64, 80, 96), (4096, 4096, 4096), (16384, 16384, 16384), (65536, 8192, 8192)):
        o = GEMMTC(*shape)
        meta["gemmtc"].append(
            {"shape": shape, "tolerance": list(o.tolerance), "num_flops": o.num_flops, "describe": o.describe()}
        )

    # ---- attention: Q, K, V ~ N(0,1), seed 3; reference = SDPA restricted to the flash backend ----
    meta["attention"] = []
    for tag, (B, H, S, D) in (("d64", (1, 2, 128, 64)), ("d128", (1, 1, 256, 128))):
        g = torch.Generator(device="cpu").manual_seed(3)
        q, k, v = (torch.randn(B, H, S, D, generator=g).half() for _ in range(3))
        arrays[f"attn_{tag}_q"], arrays[f"attn_{tag}_k"], arrays[f"attn_{tag}_v"] = bits(q), bits(k), bits(v)
        for causal in (False, True):
            fa = FlashAttention(B, H, S, S, D, causal=causal)
            ref = attn_bench.sdpa_flash(q, k, v, causal=causal, scale=fa.softmax_scale)
            arrays[f"attn_{tag}_o_{'causal' if causal else 'full'}"] = bits(ref)
    for shape, causal in (((4, 16, 4096, 4096, 128), False), ((4, 16, 4096, 4096, 64), True),
                          ((32, 32, 8192, 8192, 128), True)):
        fa = FlashAttention(*shape, causal=causal)
        meta["attention"].append(
            {"shape": shape, "causal": causal, "num_flops": fa.num_flops, "softmax_scale": fa.softmax_scale}
        )

    # ---- the unscheduled fp32 TIR GEMM, built for the C target and run here ----
    def tir_gemm(M, N, K, a, b):
        mod = create_gemm_ir_module(M, N, K, "float32")
        lib = tvm.compile(mod, target="c")
        c = np.zeros((M, N), np.float32)
        ta, tb, tc = (tvm.runtime.tensor(x) for x in (a, b, c))
        lib["main"](ta, tb, tc)
        return tc.numpy()

    g = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.rand(48, 32, generator=g) * 2 - 1).numpy()
    b = (torch.rand(32, 40, generator=g) * 2 - 1).numpy()
    arrays["f32gemm_a"], arrays["f32gemm_b"] = a, b
    arrays["f32gemm_c"] = tir_gemm(48, 40, 32, a, b)
    g = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.rand(512, 512, generator=g) * 2 - 1).numpy()
    b = (torch.rand(512, 512, generator=g) * 2 - 1).numpy()
    c = tir_gemm(512, 512, 512, a, b)
    # 512^3 is the benchmark's CPU configuration; keep a strided sample and a checksum.
    arrays["f32gemm512_sample"] = c[::37, ::41].copy()
    meta["f32gemm512"] = {"sum": float(c.astype(np.float64).sum()), "abs_sum": float(np.abs(c).astype(np.float64).sum())}

    # ---- operator records, grids, work formulas ----
    meta["rowwise"] = []
    for cls, kind in ((Softmax, "softmax"), (RMSNorm, "rmsnorm")):
        for dt in ("fp16", "bf16"):
            o = cls(16384, 4096, dt)
            meta["rowwise"].append(
                {"op": kind, "dtype_in": dt, "dtype": o.dtype, "num_bytes": o.num_bytes,
                 "tolerance": list(o.tolerance), "describe": o.describe()}
            )
    meta["grids"] = {
        "gemm": gemm_bench.standard_shapes(),
        "attention": attn_bench.standard_shapes(),
        "softmax": rowwise_bench.standard_shapes("softmax"),
        "rmsnorm": rowwise_bench.standard_shapes("rmsnorm"),
    }
    meta["attn_flops_causal_4_16_4096_128"] = attn_bench.attn_flops(4, 16, 4096, 4096, 128, True)

    np.savez_compressed(os.path.join(out, "golden.npz"), **arrays)
    with open(os.path.join(out, "golden_meta.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays;", os.path.getsize(os.path.join(out, "golden.npz")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/Deca")
    main(sys.argv[1])
