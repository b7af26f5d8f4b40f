"""CUDA-event timers used by the harness, the CLIs and the benchmark.

The reference times one call per pair of CUDA events and takes the median, after a warm-up that
lasts a set wall time rather than a set number of calls (src/kernels/attn_bench.py:35-70), and
compares candidates by timing them alternately (:94-100).  The timers here keep that contract
(``bench_cuda``: seconds per call, median of per-call event pairs; ``bench_interleaved``: median of
the per-round medians) with one difference in mechanics: the event pairs of a whole measurement
window are queued back to back and read after a single synchronisation, so the device never idles
between two timed calls waiting for the host.
"""

from __future__ import annotations

import statistics
import time
from typing import Callable, Dict, Hashable

MAX_TIMED_CALLS = 20000  # keeps the event pool bounded for microsecond-sized kernels


def _burst(fn: Callable[[], None], calls: int) -> list:
    """Runs ``fn`` ``calls`` times back to back, each between its own pair of events; returns the
    per-call device times in seconds (one synchronisation at the end)."""
    import torch

    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(calls)]
    for begin, end in pairs:
        begin.record()
        fn()
        end.record()
    torch.cuda.synchronize()
    return [begin.elapsed_time(end) * 1e-3 for begin, end in pairs]


def bench_cuda(fn: Callable[[], None], warmup_s: float = 0.3, measure_s: float = 0.3, min_iters: int = 20) -> float:
    """Median device time of one call of ``fn`` in seconds.

    Warm-up runs for ``warmup_s`` of wall time (clocks and caches settle by time, not by call
    count); the measurement then covers at least ``min_iters`` calls and about ``measure_s`` of
    device time."""
    import torch

    fn()
    torch.cuda.synchronize()
    batch, stop_at = 1, time.perf_counter() + warmup_s
    while time.perf_counter() < stop_at:
        for _ in range(batch):
            fn()
        torch.cuda.synchronize()
        batch = min(2 * batch, 32)
    estimate = max(statistics.median(_burst(fn, 3)), 1e-6)
    calls = min(MAX_TIMED_CALLS, max(min_iters, int(measure_s / estimate)))
    return statistics.median(_burst(fn, calls))


def bench_interleaved(fns: Dict[Hashable, Callable[[], None]], rounds: int = 3) -> Dict[Hashable, float]:
    """Times the callables in turn, ``rounds`` times over, so that slow drifts (clocks, other
    tenants of the machine) hit every candidate alike; returns name -> median seconds."""
    per_name = {name: [] for name in fns}
    for _ in range(rounds):
        for name, fn in fns.items():
            per_name[name].append(bench_cuda(fn))
    return {name: statistics.median(ts) for name, ts in per_name.items()}


def sustained(fn: Callable[[], None], seconds: float, calls_per_burst: int) -> float:
    """Average device time of one call of ``fn`` (seconds) over back-to-back bursts that together
    last at least ``seconds``: the figure a power-capped part settles at, as opposed to the burst
    figure ``bench_cuda`` gives for short kernels."""
    import torch

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms, calls = 0.0, 0
    while total_ms < seconds * 1e3:
        begin.record()
        for _ in range(calls_per_burst):
            fn()
        end.record()
        end.synchronize()
        total_ms += begin.elapsed_time(end)
        calls += calls_per_burst
    return total_ms * 1e-3 / calls
