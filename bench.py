"""Benchmark of the hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload rowwise|gemm|attention|gemm_sharded|attention_sharded|gemm_gather|attention_gather]

Default workload ``rowwise``: X[16384, 4096] ~ 3*N(0,1) (seed 1), W ~ N(1, 0.1), eps 1e-6.
One step = softmax and RMSNorm, each in fp16 and in bf16 (4 kernel launches,
1 073 758 208 algorithmic bytes: read x [+ w], write y).  The two dtypes use different
buffers and alternate, so 384 MB of other traffic passes between two reads of one input
(L2 is 126 MB): no flush is needed.

``value`` is whole-job throughput with inputs resident in HBM; ``e2e`` is the same work
through the operator API with pinned host inputs and outputs (copies inside the timed
region); ``roofline`` is the dominant kernel against the measured HBM / tensor peak;
``cpu_baseline`` is the CPU oracle (a port of the reference's arithmetic) timed on the
host cores on a bounded sample.  ``--impl reference`` times only that CPU arm.

Multi-GPU (torchrun, one rank per GPU): every rank runs the same per-GPU workload on its
own shard (weak scaling: row-wise shards rows, GEMM shards M, attention shards B*H); there
is no data-path collective; time is the max over ranks.  ``gemm_sharded`` and
``attention_sharded`` split one fixed problem instead (strong scaling); ``gemm_gather`` and
``attention_gather`` are those two with the epilogue also storing the output into every rank's
copy (the all-gather fused into the kernel), the unfused form (kernel, then NCCL all-gather)
timed beside it in ``comparison``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/ (None until a capture exists for that kernel).
NCU_TRAFFIC_BYTES = {
    # profiles/rowwise_softmax_f16_16384x4096.md: 134.23 MB read + 83.40 MB written (part of the
    # output is still dirty in L2 when the kernel ends)
    "rowwise_softmax_f16_16384x4096": 217628672,
    # profiles/gemm_f16_4096.md: 80.51 MB read + 6.59 MB written (C mostly still in L2)
    "gemm_f16_4096x4096x4096": 87099392,
    # profiles/fa_fwd3_f16_1x16x4096x128.md captured B = 1 (50.42 MB + 1.17 MB); traffic grows
    # in proportion to the batch: x 4 for B = 4
    "fa_fwd_f16_4x16x4096x128": 206323712,
}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:  # noqa: BLE001
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
                "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and clock-event reasons through NVML (read only) while a region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            # honour CUDA_VISIBLE_DEVICES: map the CUDA index to the NVML handle by UUID
            import torch

            uuid = str(torch.cuda.get_device_properties(index).uuid)
            self.h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u:
                    self.h = h
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------
# Workloads: each returns a dict of closures over its tensors.
# ------------------------------------------------------------------------------------------
def rowwise_host_inputs(M, N, seed=1):
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)
    x = 3.0 * torch.randn(M, N, generator=g)
    w = 1.0 + 0.1 * torch.randn(N, generator=g)
    return x, w


class RowwiseWorkload:
    name = "rowwise softmax+rmsnorm X[16384,4096] fp16+bf16"
    metric = "softmax/RMSNorm effective HBM throughput (read x [+ w], write y)"
    unit = "TB/s"
    dtype = "f32 math, f16/bf16 I/O"
    bound = "hbm"
    scaling = "weak"
    M, N, EPS = 16384, 4096, 1e-6

    def __init__(self, rank: int, world: int = 1):
        import torch

        from deca_b200.operators import RMSNorm, Softmax

        self.torch = torch
        x32, w32 = rowwise_host_inputs(self.M, self.N, seed=1 + 1000 * rank)
        self.ops, self.host, self.dev, self.out, self.host_out = [], {}, {}, {}, {}
        for dt, tdt in (("float16", torch.float16), ("bfloat16", torch.bfloat16)):
            self.host[dt] = (x32.to(tdt).pin_memory(), w32.to(tdt).pin_memory())
            self.dev[dt] = tuple(t.cuda() for t in self.host[dt])
        # launch order alternates the dtypes (different buffers)
        for kind, cls in (("softmax", Softmax), ("rmsnorm", RMSNorm)):
            for dt in ("float16", "bfloat16"):
                op = cls(self.M, self.N, dt) if kind == "softmax" else cls(self.M, self.N, dt, self.EPS)
                mod = op.compile(op.build_mod(op.default_config()))
                key = (kind, dt)
                self.out[key] = torch.empty_like(self.dev[dt][0])
                self.host_out[key] = torch.empty_like(self.host[dt][0]).pin_memory()
                self.ops.append((key, op, mod["main"]))
        self.units_per_step = sum(op.num_bytes for _, op, _ in self.ops)  # bytes
        self.launches_per_step = len(self.ops)
        self.dominant = ("softmax", "float16")
        self.dominant_units = self.ops[0][1].num_bytes
        self.traffic_key = "rowwise_softmax_f16_16384x4096"
        self.config = {"workload": self.name, "M": self.M, "N": self.N, "eps": self.EPS,
                       "l2": "inputs larger than L2; dtypes alternate buffers, no flush"}

    def args_for(self, key):
        kind, dt = key
        x, w = self.dev[dt]
        return (x, self.out[key]) if kind == "softmax" else (x, w, self.out[key])

    def step(self):
        for key, _, main in self.ops:
            main(*self.args_for(key))

    dominant_reps = 8

    def dominant_launch(self):
        key, _, main = self.ops[0]
        main(*self.args_for(key))

    E2E_CHUNKS = 8

    def _e2e_setup(self):
        """Row chunks, chunk-sized operators and three streams: host->device copies, kernels and
        device->host copies of different chunks overlap (the copy engines work in both directions
        at once), which is how a caller with host-resident data would drive the operators."""
        torch = self.torch
        from deca_b200.operators import RMSNorm, Softmax

        rows = self.M // self.E2E_CHUNKS
        self._e2e_rows = rows
        self._e2e_ops = {}
        for dt in ("float16", "bfloat16"):
            self._e2e_ops[("softmax", dt)] = Softmax(rows, self.N, dt)
            self._e2e_ops[("rmsnorm", dt)] = RMSNorm(rows, self.N, dt, self.EPS)
        self._s_in, self._s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step_e2e(self):
        """Host pinned inputs -> device -> operator calls -> host pinned outputs, chunked by rows."""
        torch = self.torch
        if not hasattr(self, "_e2e_ops"):
            self._e2e_setup()
        rows, main_stream = self._e2e_rows, torch.cuda.current_stream()
        s_in, s_out = self._s_in, self._s_out
        s_in.wait_stream(main_stream)
        s_out.wait_stream(main_stream)
        h2d = d2h = 0
        for dt in ("float16", "bfloat16"):
            hx, hw = self.host[dt]
            dx, dw = self.dev[dt]
            with torch.cuda.stream(s_in):
                dw.copy_(hw, non_blocking=True)
            h2d += hw.numel() * 2
            for c in range(self.E2E_CHUNKS):
                sl = slice(c * rows, (c + 1) * rows)
                with torch.cuda.stream(s_in):
                    dx[sl].copy_(hx[sl], non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(s_in)
                h2d += rows * self.N * 2
                main_stream.wait_event(ready)
                for kind in ("softmax", "rmsnorm"):
                    op = self._e2e_ops[(kind, dt)]
                    out = self.out[(kind, dt)][sl]
                    if kind == "softmax":
                        op(dx[sl], out=out)
                    else:
                        op(dx[sl], dw, out=out)
                    done = torch.cuda.Event()
                    done.record(main_stream)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(done)
                        self.host_out[(kind, dt)][sl].copy_(out, non_blocking=True)
                    d2h += rows * self.N * 2
        main_stream.wait_stream(s_out)
        return h2d, d2h

    def to_value(self, units_per_s):
        return units_per_s / 1e12  # TB/s

    def roofline_value(self, units_per_s):
        return units_per_s / 1e9  # GB/s

    # ---- CPU arm: the oracle on a bounded sample ----
    def cpu_sample(self, target_s=12.0):
        import numpy as np

        import oracle

        rows = 2048
        x32, w32 = rowwise_host_inputs(rows, self.N, seed=1)
        data = {}
        for dt in ("float16", "bfloat16"):
            data[dt] = (oracle.to_bits(x32.numpy(), dt), oracle.to_bits(w32.numpy(), dt))
        nbytes_once = 2 * (2 * rows * self.N * 2) + 2 * (2 * rows * self.N * 2 + self.N * 2)

        def once():
            for dt in ("float16", "bfloat16"):
                oracle.softmax(data[dt][0], dt)
            for dt in ("float16", "bfloat16"):
                oracle.rmsnorm(data[dt][0], data[dt][1], self.EPS, dt)

        once()
        t0 = time.perf_counter()
        once()
        t1 = time.perf_counter() - t0
        reps = max(1, int(target_s / max(t1, 1e-3)))
        sample = f"{reps} x (softmax+rmsnorm, fp16+bf16) on {rows} of {self.M} rows x {self.N}"
        return once, reps, nbytes_once, sample, np


class GemmWorkload:
    """fp16 tensor-core GEMM, A, B ~ U[-1, 1] (seed 2).  One step = one GEMM on each of
    `sets` rotating (A, B, C) buffer sets, so that more than an L2 of other data passes between
    two uses of a buffer."""

    name = "fp16 GEMM M=N=K=4096"
    metric = "fp16 tensor-core GEMM throughput (2*M*N*K flops)"
    unit = "TFLOPS"
    dtype = "f16 x f16 -> f32 accumulate, f16 out"
    bound = "tensor"
    scaling = "weak"
    shape = (4096, 4096, 4096)
    sets = 4
    shard_m = False
    seed = 2
    tile_override = None

    def __init__(self, rank: int, world: int = 1):
        import torch

        from deca_b200.operators import GEMMTC

        M, N, K = self.shape
        if self.shard_m:
            assert M % world == 0
            M //= world
        self.M, self.N, self.K = M, N, K
        self.op = GEMMTC(M, N, K)
        self.cfg = self.op.default_config()
        if self.tile_override:  # --gemm-tile BMxBN:stages:acc_bufs
            from deca_b200.kernels.gemm_b200 import GemmConfig

            tile, stages, acc = self.tile_override.split(":")
            bm, bn = (int(v) for v in tile.split("x"))
            self.cfg = GemmConfig(BM=bm, BN=bn, stages=int(stages), raster=self.cfg.raster, acc_bufs=int(acc), epi_smem=True)
        self.main = self.op.compile(self.op.build_mod(self.cfg))["main"]
        g = torch.Generator(device="cpu").manual_seed(self.seed + 1000 * rank)
        self.host, self.dev = [], []
        for i in range(self.sets):
            if i == 0 or not self.shard_m:
                a = (torch.rand(M, K, generator=g) * 2 - 1).half()
                b = (torch.rand(K, N, generator=g) * 2 - 1).half()
            self.dev.append((a.cuda(), b.cuda(), torch.empty(M, N, dtype=torch.float16, device="cuda")))
        # e2e uses pinned copies of the first set only
        self.host = (self.dev[0][0].cpu().pin_memory(), self.dev[0][1].cpu().pin_memory(),
                     torch.empty(M, N, dtype=torch.float16).pin_memory())
        self.units_per_step = self.sets * self.op.num_flops
        self.launches_per_step = self.sets
        self.dominant = ("gemm16", str(self.cfg))
        self.dominant_units = self.op.num_flops
        self.traffic_key = f"gemm_f16_{M}x{N}x{K}"
        self.dominant_reps = self.sets
        self._rr = 0
        self.config = {"workload": self.name, "M_per_gpu": M, "N": N, "K": K, "kernel_config": str(self.cfg),
                       "l2": f"{self.sets} rotating buffer sets ({self.sets * (M * K + K * N + M * N) * 2 >> 20} MiB)"}

    def step(self):
        for a, b, c in self.dev:
            self.main(a, b, c)

    def dominant_launch(self):
        a, b, c = self.dev[self._rr % self.sets]
        self._rr += 1
        self.main(a, b, c)

    def step_e2e(self):
        ha, hb, hc = self.host
        a, b, c = self.dev[0]
        h2d = d2h = 0
        for _ in range(self.sets):
            a.copy_(ha, non_blocking=True)
            b.copy_(hb, non_blocking=True)
            self.op(a, b, out=c)
            hc.copy_(c, non_blocking=True)
            h2d += (ha.numel() + hb.numel()) * 2
            d2h += hc.numel() * 2
        return h2d, d2h

    def to_value(self, units_per_s):
        return units_per_s / 1e12

    roofline_value = to_value

    def cpu_sample(self, target_s=12.0):
        import numpy as np
        import torch

        import oracle

        _, N, K = self.shape
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        rows = 64
        a = oracle.to_bits((torch.rand(rows, K, generator=g) * 2 - 1).numpy(), "float16")
        b = oracle.to_bits((torch.rand(K, N, generator=g) * 2 - 1).numpy(), "float16")

        def once():
            oracle.gemm16(a, b, "float16")

        once()
        t0 = time.perf_counter()
        once()
        t1 = time.perf_counter() - t0
        reps = max(1, int(target_s / max(t1, 1e-3)))
        sample = f"{reps} x ({rows} rows of A) @ B[{K},{N}], fp32 accumulate"
        return once, reps, 2 * rows * N * K, sample, np


class GemmShardedWorkload(GemmWorkload):
    """The multi-GPU GEMM configuration: M = 65536 split along M across the ranks (strong
    scaling), B replicated, no collective."""

    name = "fp16 GEMM M=65536 N=8192 K=8192 split along M"
    shape = (65536, 8192, 8192)
    sets = 1
    shard_m = True
    scaling = "strong"
    seed = 4


class GemmGatherWorkload(GemmShardedWorkload):
    """The M-split GEMM followed by the all-gather of C, fused: the kernel's epilogue stores
    every output panel into all ranks' copies of the gathered C (peer stores over NVLink, no
    separate collective).  `comparison` in the output line times the unfused form (the same
    kernel into a local shard, then an NCCL all-gather) in the same process."""

    name = "fp16 GEMM M=65536 N=8192 K=8192 split along M, C all-gathered by the epilogue"

    def __init__(self, rank: int, world: int = 1):
        import torch

        from deca_b200.sharding import GatheredOutput

        super().__init__(rank, world)
        self.rank, self.world = rank, world
        a, b, c = self.dev[0]
        if world > 1:
            self.out = GatheredOutput.symmetric(self.M, self.N, torch.float16, a.device)
        else:
            self.out = GatheredOutput.from_tensors([c], 0)
        self.dominant = ("gemm16 + peer stores", str(self.cfg))
        self.config["gather"] = f"epilogue TMA stores into {world} copies of C[{world * self.M},{self.N}]"
        self.config["nvlink_bytes_per_step"] = (world - 1) * self.M * self.N * 2

    def step(self):
        from deca_b200.sharding import gemm_gather

        a, b, _ = self.dev[0]
        gemm_gather(a, b, self.out, self.cfg)

    dominant_launch = step

    def step_e2e(self):
        from deca_b200.sharding import gemm_gather

        ha, hb, hc = self.host
        a, b, _ = self.dev[0]
        a.copy_(ha, non_blocking=True)
        b.copy_(hb, non_blocking=True)
        gemm_gather(a, b, self.out, self.cfg)
        mine = self.out.local[self.rank * self.M : (self.rank + 1) * self.M]
        hc.copy_(mine, non_blocking=True)
        return (ha.numel() + hb.numel()) * 2, hc.numel() * 2

    def comparison(self, steps, barrier):
        """Unfused: GEMM into a local shard, then all_gather_into_tensor (NCCL); max over ranks."""
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return None
        a, b, c = self.dev[0]
        full = torch.empty(self.world * self.M, self.N, dtype=torch.float16, device=a.device)

        def once():
            self.main(a, b, c)
            dist.all_gather_into_tensor(full, c)

        for _ in range(3):
            once()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            once()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item()) / steps
        return {"what": "same GEMM kernel into a local shard + NCCL all_gather_into_tensor", "ms_per_step": ms,
                "value": self.to_value(self.units_per_step * self.world / (ms / 1e3)), "unit": self.unit}


class AttentionWorkload:
    """FlashAttention forward fp16, Q, K, V ~ N(0, 1) (seed 3).  One step = the non-causal and
    the causal kernel, each on its own buffer set."""

    name = "FlashAttention fwd fp16 B=4 H=16 S=4096 D=128 (non-causal + causal)"
    metric = "FlashAttention forward throughput (4*B*H*S^2*D flops, halved when causal)"
    unit = "TFLOPS"
    dtype = "f16 x f16 -> f32 accumulate, f32 softmax, f16 out"
    bound = "tensor"
    scaling = "weak"
    shape = (4, 16, 4096, 128)
    modes = (False, True)
    shard_bh = False
    seed = 3

    def __init__(self, rank: int, world: int = 1):
        import torch

        from deca_b200.operators import FlashAttention

        B, H, S, D = self.shape
        if self.shard_bh:
            assert (B * H) % world == 0
            B, H = 1, B * H // world
        self.B, self.H, self.S, self.D = B, H, S, D
        g = torch.Generator(device="cpu").manual_seed(self.seed + 1000 * rank)
        self.ops, self.dev = [], []
        for causal in self.modes:
            op = FlashAttention(B, H, S, S, D, causal=causal)
            main = op.compile(op.build_mod(op.default_config()))["main"]
            if not self.dev or not self.shard_bh:
                q, k, v = (torch.randn(B, H, S, D, generator=g).half().cuda() for _ in range(3))
            self.dev.append((q, k, v, torch.empty_like(q)))
            self.ops.append((op, main))
        q, k, v, o = self.dev[0]
        self.host = tuple(t.cpu().pin_memory() for t in (q, k, v)) + (torch.empty_like(o, device="cpu").pin_memory(),)
        self.units_per_step = sum(op.num_flops for op, _ in self.ops)
        self.launches_per_step = len(self.ops)
        cfg = self.ops[0][0].default_config()
        self.dominant = ("fa_fwd", f"{'causal' if self.modes[0] else 'non-causal'} {cfg}")
        self.dominant_units = self.ops[0][0].num_flops
        self.traffic_key = f"fa_fwd_f16_{B}x{H}x{S}x{D}"
        self.dominant_reps = 4
        self.config = {"workload": self.name, "B_per_gpu": B, "H_per_gpu": H, "S": S, "D": D, "kernel_config": str(cfg),
                       "l2": f"Q, K, V, O of one launch are {4 * B * H * S * D * 2 >> 20} MiB; launches alternate buffer sets"}

    def step(self):
        for (op, main), (q, k, v, o) in zip(self.ops, self.dev):
            main(q, k, v, o)

    def dominant_launch(self):
        q, k, v, o = self.dev[0]
        self.ops[0][1](q, k, v, o)

    def step_e2e(self):
        hq, hk, hv, ho = self.host
        q, k, v, o = self.dev[0]
        h2d = d2h = 0
        for op, _ in self.ops:
            for src, dst in ((hq, q), (hk, k), (hv, v)):
                dst.copy_(src, non_blocking=True)
                h2d += src.numel() * 2
            op(q, k, v, out=o)
            ho.copy_(o, non_blocking=True)
            d2h += ho.numel() * 2
        return h2d, d2h

    def to_value(self, units_per_s):
        return units_per_s / 1e12

    roofline_value = to_value

    def cpu_sample(self, target_s=12.0):
        import numpy as np
        import torch

        import oracle

        _, _, S, D = self.shape
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        S_s = min(S, 2048)
        q, k, v = (oracle.to_bits(torch.randn(1, 1, S_s, D, generator=g).numpy(), "float16") for _ in range(3))
        causal_modes = self.modes

        def once():
            for causal in causal_modes:
                oracle.attention(q, k, v, causal=causal)

        once()
        t0 = time.perf_counter()
        once()
        t1 = time.perf_counter() - t0
        reps = max(1, int(target_s / max(t1, 1e-3)))
        flops = sum(4 * S_s * S_s * D // (2 if c else 1) for c in causal_modes)
        sample = f"{reps} x one head, S={S_s}, D={D}, modes causal={list(causal_modes)}"
        return once, reps, flops, sample, np


class AttentionShardedWorkload(AttentionWorkload):
    """The multi-GPU attention configuration: B*H = 1024 heads split across the ranks (strong
    scaling), causal, no collective."""

    name = "FlashAttention fwd fp16 B=32 H=32 S=8192 D=128 causal split along B*H"
    shape = (32, 32, 8192, 128)
    modes = (True,)
    shard_bh = True
    scaling = "strong"
    seed = 4


class AttentionGatherWorkload(AttentionShardedWorkload):
    """The head-split causal attention followed by the all-gather of O, fused: the kernel's
    epilogue stores every output panel into all ranks' copies of the gathered O (peer stores over
    NVLink).  `comparison` times the unfused form (same kernel, then an NCCL all-gather)."""

    name = "FlashAttention fwd fp16 B=32 H=32 S=8192 D=128 causal split along B*H, O all-gathered by the epilogue"

    def __init__(self, rank: int, world: int = 1):
        import torch

        from deca_b200.sharding import GatheredOutput

        super().__init__(rank, world)
        self.rank, self.world = rank, world
        q, k, v, o = self.dev[0]
        rows = self.B * self.H * self.S
        if world > 1:
            self.out = GatheredOutput.symmetric(rows, self.D, torch.float16, q.device)
        else:
            self.out = GatheredOutput.from_tensors([o.view(rows, self.D)], 0)
        self.dominant = ("fa_fwd + peer stores", self.dominant[1])
        self.config["gather"] = f"epilogue TMA stores into {world} copies of O[{world * self.B * self.H},{self.S},{self.D}]"
        self.config["nvlink_bytes_per_step"] = (world - 1) * rows * self.D * 2

    def step(self):
        from deca_b200.sharding import attention_gather

        q, k, v, _ = self.dev[0]
        attention_gather(q, k, v, self.out, causal=True)

    dominant_launch = step

    def step_e2e(self):
        from deca_b200.sharding import attention_gather

        hq, hk, hv, ho = self.host
        q, k, v, _ = self.dev[0]
        h2d = 0
        for src, dst in ((hq, q), (hk, k), (hv, v)):
            dst.copy_(src, non_blocking=True)
            h2d += src.numel() * 2
        attention_gather(q, k, v, self.out, causal=True)
        rows = self.B * self.H * self.S
        ho.view(rows, self.D).copy_(self.out.local[self.rank * rows : (self.rank + 1) * rows], non_blocking=True)
        return h2d, ho.numel() * 2

    def comparison(self, steps, barrier):
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return None
        q, k, v, o = self.dev[0]
        main = self.ops[0][1]
        full = torch.empty(self.world * o.numel(), dtype=torch.float16, device=o.device)

        def once():
            main(q, k, v, o)
            dist.all_gather_into_tensor(full, o.view(-1))

        for _ in range(3):
            once()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            once()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item()) / steps
        return {"what": "same attention kernel into a local shard + NCCL all_gather_into_tensor", "ms_per_step": ms,
                "value": self.to_value(self.units_per_step * self.world / (ms / 1e3)), "unit": self.unit}


def clock_summary_ok(c):
    bad = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}
    return not (bad & set(c.get("reasons", [])))


def run_cpu_arm(wl, steps, warmup, as_reference_line, n_gpus):
    import oracle

    oracle.set_num_threads()  # all host cores, whatever OMP_NUM_THREADS the launcher exported

    # reference arm: every step is a bounded sample, sized so that W + K steps take about 2 minutes
    step_s = 12.0 if not as_reference_line else max(0.05, min(4.0, 120.0 / max(1, steps + warmup)))
    once, reps, nbytes_once, sample, _ = wl.cpu_sample(target_s=step_s)
    if as_reference_line:
        for _ in range(warmup):
            once()
        t0 = time.perf_counter()
        for _ in range(steps):
            for _ in range(reps):
                once()
        dt = time.perf_counter() - t0
        per_step = dt / steps
        units = nbytes_once * reps
    else:
        t0 = time.perf_counter()
        for _ in range(reps):
            once()
        per_step = time.perf_counter() - t0
        units = nbytes_once * reps
    value = wl.to_value(units / per_step)
    base = {"value": value, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port", "sample": sample}
    return base, per_step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="rowwise")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--gemm-tile", default=None, help="GEMM workloads: BMxBN:stages:acc_bufs instead of the default config")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        # The reference has no CPU implementation of these kernels (its TIR uses PTX
        # intrinsics); its arithmetic, restated in oracle/, is what runs here, on all host threads.
        if rank != 0:
            return
        wl = WORKLOADS[args.workload].__new__(WORKLOADS[args.workload])
        base, per_step = run_cpu_arm(wl, args.steps, args.warmup, True, world)
        line = {"impl": "reference", "metric": wl.metric, "value": base["value"], "unit": wl.unit, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
                "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype,
                "data": "synthetic", "config": {"workload": wl.name}, "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if args.gemm_tile:
        GemmWorkload.tile_override = args.gemm_tile
    wl = WORKLOADS[args.workload](rank, world)
    peaks = measured_peaks()

    for _ in range(max(args.warmup, 3)):
        wl.step()
    barrier()

    # One step (and, for the roofline, the dominant kernel alone) is captured into a CUDA graph
    # so that the timed region holds kernel launches only, no Python between them.
    step_graph = dom_graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(step_graph, stream=side):
                wl.step()
            dom_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(dom_graph, stream=side):
                for _ in range(wl.dominant_reps):
                    wl.dominant_launch()
        torch.cuda.current_stream().wait_stream(side)
        step_graph.replay()
        dom_graph.replay()
    barrier()

    def run_step():
        step_graph.replay() if step_graph is not None else wl.step()

    def run_dominant():
        if dom_graph is not None:
            dom_graph.replay()
        else:
            for _ in range(wl.dominant_reps):
                wl.dominant_launch()

    # ---- timed region: exactly K steps between two events ----
    L = wl.launches_per_step
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        barrier()
        start.record()
        for _ in range(args.steps):
            run_step()
        end.record()
        torch.cuda.synchronize()
        barrier()
        total_ms = start.elapsed_time(end)
        # ---- the dominant kernel alone, back to back, for the roofline ----
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dom_iters = max(1, args.steps // 4)
        run_dominant()
        torch.cuda.synchronize()
        d0.record()
        for _ in range(dom_iters):
            run_dominant()
        d1.record()
        torch.cuda.synchronize()
        dom_avg_ms = d0.elapsed_time(d1) / (dom_iters * wl.dominant_reps)

    t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    units = wl.units_per_step * args.steps * world
    value = wl.to_value(units / (total_ms / 1e3))

    # ---- e2e: host buffers through the operator API ----
    wl.step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.e2e_steps):
        h2d, d2h = wl.step_e2e()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = wl.to_value(wl.units_per_step * args.e2e_steps * world / (float(te.item()) / 1e3))

    comparison = wl.comparison(min(args.steps, 20), barrier) if hasattr(wl, "comparison") else None

    if rank == 0:
        clocks = clk.summary()
        achieved = wl.roofline_value(wl.dominant_units / (dom_avg_ms / 1e3))
        if wl.bound == "hbm":
            peak, punit, nominal = peaks["hbm_gbs"], "GB/s", 8000.0
        else:
            peak, punit, nominal = peaks["bf16_tflops"], "TFLOP/s", 2250.0
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": L * args.steps, "launch_mode": "python" if args.no_graph else "cuda_graph",
            "roofline": {"bound": wl.bound, "kernel": f"{wl.dominant[0]} {wl.dominant[1]}", "achieved": achieved,
                         "peak": peak, "unit": punit, "frac": achieved / peak, "peak_source": peaks["source"],
                         "nominal_peak": nominal, "frac_nominal": achieved / nominal,
                         "avg_launch_us": dom_avg_ms * 1e3, "traffic": NCU_TRAFFIC_BYTES.get(wl.traffic_key)},
            "clocks": clocks, "clocks_ok": clock_summary_ok(clocks),
        }
        if comparison is not None:
            line["comparison"] = comparison
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"], _ = run_cpu_arm(wl, 1, 0, False, world)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


WORKLOADS = {"rowwise": RowwiseWorkload, "gemm": GemmWorkload, "attention": AttentionWorkload,
             "gemm_sharded": GemmShardedWorkload, "attention_sharded": AttentionShardedWorkload,
             "gemm_gather": GemmGatherWorkload, "attention_gather": AttentionGatherWorkload}

if __name__ == "__main__":
    main()
