"""Auto-tune the 16-bit tensor-core GEMM on B200 and compare it with torch (cuBLAS).

    python -m deca_b200.cli.test_gemm_tc --shape 4096 4096 4096
    python -m deca_b200.cli.test_gemm_tc --sweep

Flags, progress lines, the final record and the sweep CSV follow the reference's
test_gemm_tc.py (:27-67 flags, :159-167 record, :174-190 CSV); ``--dtype`` and ``--gpus`` are
additions.  Only light imports at module level: build workers re-import this module.
"""

import argparse
import csv
import os


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--shape", nargs=3, type=int, default=[4096, 4096, 4096], metavar=("M", "N", "K"))
    p.add_argument("--sweep", action="store_true", default=False, help="tune the square sizes 2K..16K in steps of 2K")
    p.add_argument("--dtype", choices=["fp16", "bf16"], default="fp16")
    p.add_argument("--top_n", type=int, default=24, help="number of ranked configs to build and measure (0 = all)")
    p.add_argument("--jobs", type=int, default=min(16, os.cpu_count() or 1), help="parallel build workers")
    p.add_argument("--finalists", type=int, default=3, help="best configs re-timed against torch in the final round")
    p.add_argument("--rounds", type=int, default=5, help="interleaved timing rounds of the final comparison")
    return p.parse_args(argv)


def tune(args, shape, arch, arch_str, log):
    from ..cost_model.CostModel import rank_gemm_configs
    from ..kernels.gemm_b200 import build_gemm_tc_to_file
    from ..kernels.gemm_bench import torch_ref
    from ..kernels.module import load_module
    from ..operators import GEMMTC
    from ..Solver import solve_gemm_tc
    from . import _tune

    M, N, K = shape
    timer = _tune.Timer()
    dtype = {"fp16": "float16", "bf16": "bfloat16"}[args.dtype]
    op = GEMMTC(M, N, K, dtype)

    configs = solve_gemm_tc(arch, M, N, K)
    ranked = rank_gemm_configs(configs, arch, M, N, K, top_n=args.top_n or None)
    print(f"Find {len(configs)} {op.name} configs, measuring {len(ranked)}", flush=True)

    paths = _tune.build_all(build_gemm_tc_to_file, lambda cfg, path: (shape, cfg, arch_str, path, dtype), ranked,
                            args.jobs, "gemm_tune_")
    compile_time = timer.elapsed()

    res = _tune.measure_configs(op, arch, True, ranked, paths)
    total = timer.elapsed()
    if not res:
        raise RuntimeError(f"no valid {op.name} config for {shape}")
    res.sort(key=lambda x: x[0], reverse=True)
    err_of = {cfg: err for _, cfg, _, err in res}

    inputs = op.make_inputs()
    out = op.make_output(inputs)
    fns = {"torch": lambda: torch_ref(inputs)}
    for _, cfg, _, _ in res[: args.finalists]:
        func = load_module(paths[cfg])["main"]
        fns[cfg] = lambda func=func: func(*op.kernel_args(inputs, out))
    torch_t, best_cfg, best_t = _tune.final_round(fns, args.rounds)
    best_tflops = op.num_flops / best_t / 1e12
    torch_tflops = op.num_flops / torch_t / 1e12
    peak = 100 * best_tflops * 1e3 / arch.peak_mma_sync_flops

    msg = (
        f"{_tune.stamp()} [{arch.name}]\n"
        f" DeCA {op.describe()}, config: {best_cfg} "
        f"(cost-model rank {ranked.index(best_cfg) + 1}/{len(ranked)})\n"
        f" throughput: {best_tflops:.1f} TFLOPS ({peak:.0f}% of fp32-acc TC peak), "
        f"runtime: {best_t * 1e3:.4f} ms, max err: {err_of[best_cfg]:.2e}\n"
        f" torch: {torch_tflops:.1f} TFLOPS, runtime: {torch_t * 1e3:.4f} ms, ratio: {torch_t / best_t:.3f}\n"
        f" compile time: {compile_time:.1f} s, total tuning time: {total:.1f} s\n"
    )
    _tune.emit(msg, log)
    return best_cfg, best_tflops, torch_tflops


def write_sweep_csv(summary, path):
    """Writes DeCA and torch TFLOPS for the 2K-16K sweep."""
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["M", "N", "K", "DeCA_TFLOPS", "torch_TFLOPS", "ratio"])
        for (M, N, K), _, tflops, torch_tflops in summary:
            ratio = tflops / torch_tflops if torch_tflops else float("nan")
            w.writerow([M, N, K, f"{tflops:.4f}", f"{torch_tflops:.4f}", f"{ratio:.4f}"])


def main(argv=None):
    from ..kernels.gemm_bench import standard_shapes
    from ..utils.helper import GPUDetector
    from . import _tune

    args = parse_args(argv)
    arch = GPUDetector.create_gpu_instance()
    arch_str = "sm_100a"

    shapes = standard_shapes() if args.sweep else [tuple(args.shape)]
    summary = []
    with open(_tune.log_path(), "a") as log:
        for shape in shapes:
            try:
                cfg, tflops, torch_tflops = tune(args, shape, arch, arch_str, log)
            except RuntimeError as e:
                # e.g. out of memory on a shared GPU; keep sweeping the other shapes
                if not args.sweep:
                    raise
                print(f"skipping {shape}: {e}", flush=True)
                continue
            summary.append((shape, cfg, tflops, torch_tflops))

    if len(summary) > 1:
        print(f"\nSummary of FP16 Tensor Core GEMM on {arch.name}:")
        print(f"{'M':>6} {'N':>6} {'K':>6} | {'DeCA':>6} {'torch':>6} {'ratio':>6} | config")
        for (M, N, K), cfg, tflops, torch_tflops in summary:
            print(f"{M:>6} {N:>6} {K:>6} | {tflops:>6.1f} {torch_tflops:>6.1f} {tflops / torch_tflops:>6.3f} | {cfg}")
    if args.sweep:
        csv_path = os.path.join(os.path.dirname(_tune.log_path()), "gemm_tc_2K_to_16K.csv")
        write_sweep_csv(summary, csv_path)
        print(f"wrote {len(summary)} shapes to {csv_path}", flush=True)


if __name__ == "__main__":
    main()
