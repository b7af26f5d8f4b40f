"""The tune-verify-benchmark loop shared by the three CLIs.

Same flow as ``tune()`` in the reference's test_gemm_tc.py:101-171, test_flash_attn.py:85-155
and test_rowwise.py:76-145: enumerate configs (Solver), rank them (cost model), build the
top ones in spawned worker processes that need no CUDA context, load / verify / time each
with RuntimeMod, re-time the finalists alternately with the torch baseline, print the record
and append it to ``deca_performance.log``.
"""

from __future__ import annotations

import multiprocessing as mp
import os
import tempfile
import time
from concurrent.futures import ProcessPoolExecutor, as_completed
from concurrent.futures.process import BrokenProcessPool
from datetime import datetime

LOG_NAME = "deca_performance.log"


def log_path() -> str:
    """The log sits in the working directory unless DECA_LOG_DIR names another one."""
    return os.path.join(os.environ.get("DECA_LOG_DIR", os.getcwd()), LOG_NAME)


def build_all(build_fn, build_args_of, configs, jobs: int, prefix: str):
    """Builds configs in parallel; returns {cfg: path of the exported kernel file}.

    ``build_fn`` is a picklable top-level ``build_*_to_file``; ``build_args_of(cfg, path)``
    gives its positional arguments.  A worker that dies breaks the whole pool: the affected
    configs are then rebuilt serially in this process."""
    tmpdir = tempfile.mkdtemp(prefix=prefix)
    path_of = {cfg: os.path.join(tmpdir, f"cfg{i}.so") for i, cfg in enumerate(configs)}
    paths, crashed = {}, []
    with ProcessPoolExecutor(max_workers=max(1, jobs), mp_context=mp.get_context("spawn")) as pool:
        futures = {pool.submit(build_fn, *build_args_of(cfg, path_of[cfg])): cfg for cfg in configs}
        for fut in as_completed(futures):
            cfg = futures[fut]
            try:
                paths[cfg] = fut.result()
            except BrokenProcessPool:
                crashed.append(cfg)
            except Exception as e:  # noqa: BLE001
                print(f"{cfg} failed to build: {str(e)[-200:]}", flush=True)
    for cfg in crashed:
        try:
            paths[cfg] = build_fn(*build_args_of(cfg, path_of[cfg]))
        except Exception as e:  # noqa: BLE001
            print(f"{cfg} failed to build: {str(e)[-200:]}", flush=True)
    return paths


def measure_configs(op, arch, use_tc, ranked, paths, loader: str = "load_kernel"):
    """Loads, verifies and times every built config; returns [(throughput, cfg, seconds, max_err)]."""
    import torch

    from ..RuntimeMod import RuntimeMod

    res = []
    for cfg in ranked:
        if cfg not in paths:
            continue
        rt = RuntimeMod(op, arch, use_tc, cfg)
        try:
            getattr(rt, loader)(paths[cfg])
            rt.time_evaluator()
            print(rt.record, flush=True)
            res.append((rt.throughput, cfg, rt.execution_time, rt.max_error))
        except Exception as e:  # noqa: BLE001
            print(f"{cfg} is not a valid config: {str(e)[-200:]}", flush=True)
        torch.cuda.empty_cache()
    return res


def final_round(fns: dict, rounds: int):
    """Times the finalists and the baseline (key "torch") alternately; returns
    (baseline seconds, best config, its seconds)."""
    from ..kernels.attn_bench import bench_interleaved

    times = bench_interleaved(fns, rounds=rounds)
    base_t = times.pop("torch")
    best_cfg, best_t = min(times.items(), key=lambda x: x[1])
    return base_t, best_cfg, best_t


def emit(msg: str, log) -> None:
    print("✅✅✅ " + msg, flush=True)
    log.write(msg + "\n")
    log.flush()


def stamp() -> str:
    return datetime.now().strftime("%Y-%m-%d %H:%M:%S")


class Timer:
    def __init__(self):
        self.start = time.time()

    def elapsed(self) -> float:
        return time.time() - self.start
