"""Auto-tune the row-wise softmax / RMSNorm kernels on B200 and compare them with eager torch.

    python -m deca_b200.cli.test_rowwise --op softmax --shape 16384 4096
    python -m deca_b200.cli.test_rowwise --op rmsnorm --dtype bf16 --sweep

Flags, progress lines and the final record follow the reference's test_rowwise.py
(:26-42 flags, :133-141 record).
"""

import argparse
import csv
import os


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--op", choices=["softmax", "rmsnorm"], default="softmax")
    p.add_argument("--dtype", choices=["fp16", "bf16"], default="fp16")
    p.add_argument("--shape", nargs=2, type=int, default=[16384, 4096], metavar=("M", "N"))
    p.add_argument("--sweep", action="store_true", default=False, help="tune the standard row-wise benchmark grid")
    p.add_argument("--eps", type=float, default=1e-6, help="RMSNorm epsilon")
    p.add_argument("--top_n", type=int, default=24, help="number of ranked configs to build and measure (0 = all)")
    p.add_argument("--jobs", type=int, default=min(16, os.cpu_count() or 1), help="parallel build workers")
    p.add_argument("--finalists", type=int, default=3, help="best configs re-timed against torch in the final round")
    p.add_argument("--rounds", type=int, default=5, help="interleaved timing rounds of the final comparison")
    return p.parse_args(argv)


def tune(args, shape, arch, arch_str, log):
    import torch

    from ..cost_model.CostModel import rank_rowwise_configs
    from ..kernels.module import load_module
    from ..kernels.rowwise_b200 import build_rowwise_to_file
    from ..operators import RMSNorm, Softmax
    from ..Solver import solve_rowwise
    from . import _tune

    M, N = shape
    timer = _tune.Timer()
    op = Softmax(M, N, args.dtype) if args.op == "softmax" else RMSNorm(M, N, args.dtype, args.eps)

    configs = solve_rowwise(arch, args.op, M, N)
    ranked = rank_rowwise_configs(configs, arch, args.op, M, N, top_n=args.top_n or None)
    print(f"Find {len(configs)} {op.name} configs, measuring {len(ranked)}", flush=True)

    paths = _tune.build_all(build_rowwise_to_file,
                            lambda cfg, path: (args.op, shape, op.dtype, cfg, op.eps, arch_str, path), ranked,
                            args.jobs, "rw_tune_")
    compile_time = timer.elapsed()

    res = _tune.measure_configs(op, arch, False, ranked, paths)
    total = timer.elapsed()
    if not res:
        raise RuntimeError(f"no valid {op.name} config for {shape}")
    res.sort(key=lambda x: x[0], reverse=True)
    err_of = {cfg: err for _, cfg, _, err in res}

    inputs = op.make_inputs()
    out = torch.empty_like(inputs[0])
    fns = {"torch": lambda: op.reference(inputs)}
    for _, cfg, _, _ in res[: args.finalists]:
        func = load_module(paths[cfg])["main"]
        fns[cfg] = lambda func=func: func(*op.kernel_args(inputs, out))
    torch_t, best_cfg, best_t = _tune.final_round(fns, args.rounds)
    best_gbps = op.num_bytes / best_t / 1e9
    torch_gbps = op.num_bytes / torch_t / 1e9
    peak = 100 * best_gbps / arch.dram_bw

    msg = (
        f"{_tune.stamp()} [{arch.name}]\n"
        f" DeCA {op.describe()}, config: {best_cfg} "
        f"(cost-model rank {ranked.index(best_cfg) + 1}/{len(ranked)})\n"
        f" throughput: {best_gbps:.1f} GB/s ({peak:.0f}% of DRAM peak), "
        f"runtime: {best_t * 1e3:.4f} ms, max err: {err_of[best_cfg]:.2e}\n"
        f" torch: {torch_gbps:.1f} GB/s, runtime: {torch_t * 1e3:.4f} ms, ratio: {torch_t / best_t:.3f}\n"
        f" compile time: {compile_time:.1f} s, total tuning time: {total:.1f} s\n"
    )
    _tune.emit(msg, log)
    return best_cfg, best_gbps, torch_gbps


def main(argv=None):
    from ..kernels.rowwise_bench import standard_shapes
    from ..utils.helper import GPUDetector
    from . import _tune

    args = parse_args(argv)
    arch = GPUDetector.create_gpu_instance()
    arch_str = "sm_100a"

    shapes = standard_shapes(args.op) if args.sweep else [tuple(args.shape)]
    summary = []
    with open(_tune.log_path(), "a") as log:
        for shape in shapes:
            try:
                cfg, gbps, torch_gbps = tune(args, shape, arch, arch_str, log)
            except RuntimeError as e:
                # e.g. out of memory on a shared GPU; keep sweeping the other shapes
                if not args.sweep:
                    raise
                print(f"skipping {shape}: {e}", flush=True)
                continue
            summary.append((shape, cfg, gbps, torch_gbps))

    if len(summary) > 1:
        print(f"\nSummary of {args.op} ({args.dtype}) on {arch.name}:")
        print(f"{'M':>6} {'N':>7} | {'DeCA':>7} {'torch':>7} {'%peak':>5} {'ratio':>6} | config")
        for (M, N), cfg, gbps, torch_gbps in summary:
            print(f"{M:>6} {N:>7} | {gbps:>7.0f} {torch_gbps:>7.0f} "
                  f"{100 * gbps / arch.dram_bw:>5.0f} {gbps / torch_gbps:>6.3f} | {cfg}")
    if args.sweep:
        # the sweep's table as a file, next to the log (the GEMM CLI's CSV, for this operator)
        csv_path = os.path.join(os.path.dirname(_tune.log_path()), f"{args.op}_{args.dtype}_sweep.csv")
        with open(csv_path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["M", "N", "DeCA_GBps", "torch_GBps", "ratio", "config"])
            for (M, N), cfg, gbps, torch_gbps in summary:
                w.writerow([M, N, f"{gbps:.2f}", f"{torch_gbps:.2f}",
                            f"{gbps / torch_gbps if torch_gbps else float('nan'):.4f}", str(cfg)])
        print(f"wrote {len(summary)} shapes to {csv_path}", flush=True)


if __name__ == "__main__":
    main()
