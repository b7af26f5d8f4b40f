"""Auto-tune the FlashAttention forward kernel on B200 and compare it with torch SDPA (flash).

    python -m deca_b200.cli.test_flash_attn --shape 4 16 4096 128 [--causal]
    python -m deca_b200.cli.test_flash_attn --sweep

Flags, progress lines and the final record follow the reference's test_flash_attn.py
(:26-42 flags, :143-151 record).
"""

import argparse
import csv
import os


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--shape", nargs="*", type=int, default=[4, 16, 4096, 128],
                   help="B H S D (S_q = S_kv) or B H S_q S_kv D")
    p.add_argument("--sweep", action="store_true", default=False, help="tune the FlashAttention-2 benchmark grid")
    p.add_argument("--causal", action="store_true", default=False, help="top-left aligned causal mask (S_q == S_kv)")
    p.add_argument("--top_n", type=int, default=16, help="number of ranked configs to build and measure (0 = all)")
    p.add_argument("--jobs", type=int, default=min(16, os.cpu_count() or 1), help="parallel build workers")
    p.add_argument("--finalists", type=int, default=3, help="best configs re-timed against SDPA in the final round")
    p.add_argument("--rounds", type=int, default=5, help="interleaved timing rounds of the final comparison")
    return p.parse_args(argv)


def parse_shape(s):
    if len(s) == 4:
        B, H, S, D = s
        return (B, H, S, S, D)
    assert len(s) == 5, "--shape expects B H S D or B H S_q S_kv D"
    return tuple(s)


def tune(args, shape, arch, arch_str, log):
    import torch

    from ..cost_model.CostModel import rank_fa_configs
    from ..kernels.attn_bench import make_qkv, sdpa_flash
    from ..kernels.flash_attn_b200 import build_flash_attn_to_file
    from ..kernels.module import load_module
    from ..operators import FlashAttention
    from ..Solver import solve_flash_attn
    from . import _tune

    B, H, S_q, S_kv, D = shape
    timer = _tune.Timer()
    op = FlashAttention(B, H, S_q, S_kv, D, causal=args.causal)

    configs = solve_flash_attn(arch, B, H, S_q, S_kv, D)
    ranked = rank_fa_configs(configs, arch, shape, args.causal, top_n=args.top_n or None)
    print(f"Find {len(configs)} FlashAttention configs, measuring {len(ranked)}", flush=True)

    paths = _tune.build_all(build_flash_attn_to_file,
                            lambda cfg, path: (shape, cfg, op.softmax_scale, arch_str, path, args.causal), ranked,
                            args.jobs, "fa_tune_")
    compile_time = timer.elapsed()

    res = _tune.measure_configs(op, arch, True, ranked, paths, loader="load_flash_attn")
    total = timer.elapsed()
    if not res:
        raise RuntimeError(f"no valid FlashAttention config for {shape}")
    res.sort(key=lambda x: x[0], reverse=True)
    err_of = {cfg: err for _, cfg, _, err in res}

    q, k, v = make_qkv(B, H, S_q, S_kv, D)
    o = torch.empty_like(q)
    fns = {"torch": lambda: sdpa_flash(q, k, v, causal=args.causal, scale=op.softmax_scale)}
    for _, cfg, _, _ in res[: args.finalists]:
        func = load_module(paths[cfg])["main"]
        fns[cfg] = lambda func=func: func(q, k, v, o)
    sdpa_t, best_cfg, best_t = _tune.final_round(fns, args.rounds)
    best_tflops = op.num_flops / best_t / 1e12
    sdpa_tflops = op.num_flops / sdpa_t / 1e12

    msg = (
        f"{_tune.stamp()} [{arch.name}]\n"
        f" DeCA FlashAttention: B = {B}, H = {H}, S_q = {S_q}, S_kv = {S_kv}, D = {D}, "
        f"causal = {args.causal}, "
        f"config: {best_cfg} (cost-model rank {ranked.index(best_cfg) + 1}/{len(ranked)})\n"
        f" throughput: {best_tflops:.2f} TFLOPS, runtime: {best_t * 1e3:.4f} ms, max err: {err_of[best_cfg]:.2e}\n"
        f" SDPA-flash: {sdpa_tflops:.2f} TFLOPS, runtime: {sdpa_t * 1e3:.4f} ms, "
        f"ratio: {best_tflops / sdpa_tflops:.3f}\n"
        f" compile time: {compile_time:.1f} s, total tuning time: {total:.1f} s\n"
    )
    _tune.emit(msg, log)
    return best_cfg, best_tflops, sdpa_tflops


def main(argv=None):
    from ..kernels.attn_bench import standard_shapes
    from ..utils.helper import GPUDetector
    from . import _tune

    args = parse_args(argv)
    arch = GPUDetector.create_gpu_instance()
    arch_str = "sm_100a"

    shapes = [(B, H, S, S, D) for B, H, S, D in standard_shapes()] if args.sweep else [parse_shape(args.shape)]
    summary = []
    with open(_tune.log_path(), "a") as log:
        for shape in shapes:
            cfg, tflops, sdpa = tune(args, shape, arch, arch_str, log)
            summary.append((shape, cfg, tflops, sdpa))

    if len(summary) > 1:
        print(f"\nSummary on {arch.name}:")
        print(f"{'B':>3} {'H':>3} {'S':>6} {'D':>4} | {'DeCA':>8} {'SDPA':>8} {'ratio':>6} | config")
        for (B, H, S_q, _, D), cfg, tflops, sdpa in summary:
            print(f"{B:>3} {H:>3} {S_q:>6} {D:>4} | {tflops:>8.2f} {sdpa:>8.2f} {tflops / sdpa:>6.3f} | {cfg}")
    if args.sweep:
        # the sweep's table as a file, next to the log (the GEMM CLI's CSV, for this operator)
        name = "flash_attn_causal_sweep.csv" if args.causal else "flash_attn_sweep.csv"
        csv_path = os.path.join(os.path.dirname(_tune.log_path()), name)
        with open(csv_path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["B", "H", "S_q", "S_kv", "D", "causal", "DeCA_TFLOPS", "SDPA_TFLOPS", "ratio", "config"])
            for (B, H, S_q, S_kv, D), cfg, tflops, sdpa in summary:
                w.writerow([B, H, S_q, S_kv, D, int(args.causal), f"{tflops:.4f}", f"{sdpa:.4f}",
                            f"{tflops / sdpa if sdpa else float('nan'):.4f}", str(cfg)])
        print(f"wrote {len(summary)} shapes to {csv_path}", flush=True)


if __name__ == "__main__":
    main()
