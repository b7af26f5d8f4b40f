"""Runs one kernel case a few times (for profilers and quick checks).

    python -m deca_b200.run_case --op softmax --dtype fp16 --shape 16384 4096 --iters 5
    python -m deca_b200.run_case --op gemm --shape 4096 4096 4096
    python -m deca_b200.run_case --op attention --shape 4 16 4096 128 [--causal]

Prints the median CUDA-event time and the throughput in the operator's unit.
"""

import argparse

import torch

from .operators import GEMMTC, FlashAttention, RMSNorm, Softmax


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["softmax", "rmsnorm", "gemm", "attention"], required=True)
    ap.add_argument("--dtype", default="fp16")
    ap.add_argument("--shape", nargs="+", type=int, required=True)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--config", default="", help="key=value,... overrides of the default config")
    args = ap.parse_args()

    dt = {"fp16": "float16", "bf16": "bfloat16"}.get(args.dtype, args.dtype)
    if args.op in ("softmax", "rmsnorm"):
        M, N = args.shape
        op = Softmax(M, N, dt) if args.op == "softmax" else RMSNorm(M, N, dt)
    elif args.op == "gemm":
        op = GEMMTC(*args.shape, dtype=dt)
    else:
        B, H, S, D = args.shape
        op = FlashAttention(B, H, S, S, D, causal=args.causal)
    cfg = op.default_config()
    if args.config:
        kv = {}
        for item in args.config.split(","):
            k, v = item.split("=")
            cur = getattr(cfg, k)
            kv[k] = type(cur)(int(v)) if not isinstance(cur, str) else v
        cfg = type(cfg)(**{**cfg.as_dict(), **kv})
    mod = op.compile(op.build_mod(cfg))
    inputs = op.make_inputs()
    out = op.make_output(inputs) if hasattr(op, "make_output") else torch.empty_like(inputs[0])
    fn = mod["main"]
    a = op.kernel_args(inputs, out)
    times = []
    for _ in range(args.iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn(*a)
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e) / 1e3)
    t = sorted(times)[len(times) // 2]
    if getattr(op, "metric", "GB/s") == "TFLOPS" or hasattr(op, "num_flops"):
        print(f"{op.describe()} {cfg}: {t * 1e3:.4f} ms, {op.num_flops / t / 1e12:.1f} TFLOPS")
    else:
        print(f"{op.describe()} {cfg}: {t * 1e3:.4f} ms, {op.num_bytes / t / 1e9:.1f} GB/s")


if __name__ == "__main__":
    main()
