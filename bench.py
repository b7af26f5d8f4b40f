"""Benchmark of the hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload gemm_sharded|gemm|attention|attention_sharded|rowwise|gemm_gather|attention_gather]
                    [--records all|none|name,name,...] [--seconds S]

Headline (default ``gemm_sharded``): the fp16 tensor-core GEMM of the multi-GPU configuration,
M = 65536, N = K = 8192, A and B ~ U[-1, 1] (seed 4), split along M over the ranks (strong
scaling: the same problem at every N; B replicated; no collective on the data path).  One step
= ``launches_per_step`` back-to-back launches of the whole problem (each rank its M shard), so
that K = 20 steps keep the tensor pipe loaded for about two seconds at N = 1 and the number is a
sustained, power-capped one.  ``value`` = 2*M*N*K flops x launches / time, time taken with CUDA
events between barriers, max over ranks.

The same JSON line carries ``records``: the other configurations of the metric, each measured
like the headline kernel (device-resident inputs, >= ``--seconds`` of back-to-back launches in
bursts that alternate with the library baseline on the same tensors, clocks sampled while our
kernel runs): GEMM 4096^3 / 8192^3 / 16384^3 (+ 2048^3) against cuBLAS, FlashAttention
B4 H16 S4096 D128 and D64, causal and not, against SDPA-flash, the row-wise step on
X[16384, 4096] against eager torch, and the head-split causal attention B32 H32 S8192 D128.
With more than one rank only the sharded records run (attention split along B*H, row-wise
replicas).

``e2e`` is the headline through the operator API from pinned host memory and back (row chunks
pipelined over three streams); ``roofline`` is the headline kernel against the measured tensor
peak (sustained figure, since the timed region is seconds long; the burst and nominal fractions
are given beside it); ``cpu_baseline`` is the CPU oracle (a port of the reference's arithmetic)
on the host cores on a bounded sample.  ``--impl reference`` times only that CPU arm and prints
the same ``config``.
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
FALLBACK_BF16_TFLOPS_SUSTAINED = 1400.0
NOMINAL_HBM_GBS = 8000.0
NOMINAL_F16_TFLOPS = 2250.0

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each record's kernel, from
# one-launch ncu captures of exactly these shapes with the default configs (read + written).
NCU_TRAFFIC_BYTES = {
    "gemm_f16_65536x8192x8192": 6246289664 + 1060927488,   # A + B + C = 2.28 GB: B streams past bands of A
    "gemm_f16_2048x2048x2048": 16822528 + 0,               # C still in L2 when the kernel ends
    "gemm_f16_4096x4096x4096": 80066816 + 6435584,
    "gemm_f16_8192x8192x8192": 879593984 + 120230912,
    "gemm_f16_16384x16384x16384": 6821973504 + 528499200,
    "fa_fwd_f16_4x16x4096x128": 201451264 + 43802624,      # Q + K + V = 201.3 MB, O = 67.1 MB partly still in L2
    "fa_fwd_f16_4x16x4096x128_causal": 201725952 + 48557568,
    "fa_fwd_f16_4x16x4096x64": 100756224 + 13899520,
    "fa_fwd_f16_4x16x4096x64_causal": 100818688 + 15640576,
    # softmax fp16 X[16384, 4096]: 134.2 MB read + 81.4 MB written (part of the output is still dirty in L2)
    "rowwise_softmax_f16_16384x4096": 134236928 + 81434368,
}

def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:  # noqa: BLE001
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
                "bf16_tflops_sustained": FALLBACK_BF16_TFLOPS_SUSTAINED, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and clock-event reasons through NVML (read only) while ``active`` is set."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.power, self.reasons = [], [], set()
        self.max_mhz = None
        self.active = threading.Event()
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self.nv = pynvml
            # honour CUDA_VISIBLE_DEVICES: map the CUDA index to the NVML handle by UUID
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
            if self.active.is_set():
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                    self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1e3)
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
        s, p = sorted(self.samples), sorted(self.power)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "power_w": round(p[len(p) // 2], 1) if p else None}


def clock_summary_ok(c):
    bad = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}
    return not (bad & set(c.get("reasons", [])))


class Env:
    """Rank, world and the two collective helpers every measurement needs."""

    def __init__(self, rank, local_rank, world, dist):
        self.rank, self.local_rank, self.world, self.dist = rank, local_rank, world, dist

    def barrier(self):
        import torch

        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        import torch

        t = torch.tensor(list(values), dtype=torch.float64, device="cuda")
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]


# ------------------------------------------------------------------------------------------
# Workloads.  `config()` is static (the CPU arm prints the same dict without a GPU); `setup`
# allocates device tensors and fills `launches` (one kernel launch each, on rotating buffer
# sets where one set is smaller than L2) and `baseline` (the library kernel on the same tensors).
# `units` is the whole job's work per round in which every rank does one launch.
# ------------------------------------------------------------------------------------------
class Workload:
    key = ""
    metric = unit = dtype = bound = ""
    scaling = "weak"
    baseline_name = None
    sharded = False      # every rank takes part (else the record runs on a single GPU only)
    traffic_key = None
    launches_per_step = 1

    def to_value(self, units_per_s):
        return units_per_s / 1e12

    def teardown(self):
        import torch

        self.__dict__.clear()
        torch.cuda.empty_cache()


def uniform_pm1(shape, seed, device="cuda"):
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.rand(*shape, generator=g, device=device) * 2 - 1).half()


class GemmWorkload(Workload):
    """fp16 GEMM C = A @ B, A and B ~ U[-1, 1].  ``shard_m``: M is the whole problem's and each rank
    owns M / world rows of A and C (strong scaling); else every rank runs the full shape."""

    metric = "fp16 tensor-core GEMM throughput (2*M*N*K flops)"
    unit = "TFLOPS"
    dtype = "f16 x f16 -> f32 accumulate, f16 out"
    bound = "tensor"
    baseline_name = "cuBLAS (torch.matmul, fp16)"
    tile_override = None

    def __init__(self, M, N, K, seed, shard_m=False, launches_per_step=1, key=None):
        self.shape, self.seed, self.shard_m = (M, N, K), seed, shard_m
        self.sharded = shard_m
        self.scaling = "strong" if shard_m else "weak"
        self.launches_per_step = launches_per_step
        self.key = key or f"gemm_{M}x{N}x{K}"
        self.traffic_key = f"gemm_f16_{M}x{N}x{K}"

    def config(self, world):
        M, N, K = self.shape
        c = {"workload": f"fp16 GEMM M={M} N={N} K={K}" + (" split along M" if self.shard_m else ""),
             "M": M, "N": N, "K": K, "seed": self.seed, "inputs": "U[-1,1]", "launches_per_step": self.launches_per_step}
        if self.shard_m:
            c["M_per_gpu"] = M // world
        set_bytes = ((M // world if self.shard_m else M) * (K + N) + K * N) * 2
        c["l2"] = ("inputs larger than L2, no flush" if set_bytes > (512 << 20)
                   else "rotating buffer sets, more than L2 between two uses of a buffer")
        return c

    def setup(self, env):
        import torch

        from deca_b200.operators import GEMMTC

        M, N, K = self.shape
        if self.shard_m:
            assert M % env.world == 0
            M //= env.world
        self.M, self.N, self.K = M, N, K
        self.op = GEMMTC(M, N, K)
        self.cfg = self.op.default_config()
        if self.tile_override:  # --gemm-tile BMxBN:stages:acc_bufs[:cta_group]
            from deca_b200.kernels.gemm_b200 import GemmConfig

            parts = self.tile_override.split(":")
            bm, bn = (int(v) for v in parts[0].split("x"))
            self.cfg = GemmConfig(BM=bm, BN=bn, stages=int(parts[1]), raster=self.cfg.raster, acc_bufs=int(parts[2]),
                                  epi_smem=True, cta_group=int(parts[3]) if len(parts) > 3 else 1)
        self.main = self.op.compile(self.op.build_mod(self.cfg))["main"]
        set_bytes = (M * K + K * N + M * N) * 2
        n_sets = 1 if set_bytes > (512 << 20) else max(2, min(20, (400 << 20) // set_bytes + 1))
        # B is the same on every rank (it is replicated); A rows are the rank's own
        b = uniform_pm1((K, N), self.seed)
        self.sets = []
        for i in range(n_sets):
            a = uniform_pm1((M, K), self.seed + 1 + 1000 * env.rank + 17 * i)
            bb = b if i == 0 else uniform_pm1((K, N), self.seed + 500 + i)
            self.sets.append((a, bb, torch.empty(M, N, dtype=torch.float16, device="cuda")))
        self.launches = [lambda a=a, b=b, c=c: self.main(a, b, c) for a, b, c in self.sets]
        self.baseline = [lambda a=a, b=b, c=c: torch.matmul(a, b, out=c) for a, b, c in self.sets]
        self.units = self.op.num_flops * (env.world if self.shard_m else 1)
        self.traffic_key = f"gemm_f16_{M}x{N}x{K}"  # the shape one GPU runs
        self.kernel = f"gemm16 {self.cfg}"
        self.env = env

    def reference_kernel_groups(self, rk):
        a, b, c = self.sets[0]
        cands = [(e, (a, b, c)) for e in rk.entries("gemm", (self.M, self.N, self.K))]
        return [("gemm", cands, self.op.num_flops)] if cands and not self.shard_m else []

    # ---- e2e: pinned host A, B -> device -> operator calls on row chunks -> pinned host C ----
    def _e2e_setup(self):
        import torch

        from deca_b200.operators import GEMMTC

        a, b, c = self.sets[0]
        self.host = (a.cpu().pin_memory(), b.cpu().pin_memory(), torch.empty(self.M, self.N, dtype=torch.float16).pin_memory())
        self.e2e_rows = max(256, self.M // 16)  # 16 chunks: the last chunk's kernel and copy-out are the pipeline's tail
        self.e2e_op = GEMMTC(self.e2e_rows, self.N, self.K)
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        # More than one rank: every rank needs all of B, but over the host link each uploads only its
        # 1 / world of B's rows; the ranks then all-gather B over NVLink.  (Eight ranks uploading all of B
        # each doubled the bytes through a host that moves 135 - 146 GB/s in total.)
        world = self.env.world
        self.b_rows = self.K // world if world > 1 and self.shard_m and self.K % world == 0 else 0
        if self.b_rows:
            self.b_part = torch.empty(self.b_rows, self.N, dtype=b.dtype, device=b.device)
            # once, outside every timed region: the gathered B is the B every rank generated
            r = self.env.rank
            want = b.clone()
            self.b_part.copy_(self.host[1][r * self.b_rows : (r + 1) * self.b_rows])
            b.zero_()
            self.env.dist.all_gather_into_tensor(b, self.b_part)
            torch.cuda.synchronize()
            if not torch.equal(b, want):
                raise RuntimeError("B gathered from the ranks' row slices differs from the generated B")

    def step_e2e(self):
        import torch

        if not hasattr(self, "host"):
            self._e2e_setup()
        ha, hb, hc = self.host
        a, b, c = self.sets[0]
        main, s_in, s_out = torch.cuda.current_stream(), self.s_in, self.s_out
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        with torch.cuda.stream(s_in):
            if self.b_rows:
                r = self.env.rank
                self.b_part.copy_(hb[r * self.b_rows : (r + 1) * self.b_rows], non_blocking=True)
                self.env.dist.all_gather_into_tensor(b, self.b_part)
                h2d = self.b_part.numel() * 2
            else:
                b.copy_(hb, non_blocking=True)
                h2d = hb.numel() * 2
        d2h = 0
        for r0 in range(0, self.M, self.e2e_rows):
            sl = slice(r0, r0 + self.e2e_rows)
            with torch.cuda.stream(s_in):
                a[sl].copy_(ha[sl], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            main.wait_event(ready)
            self.e2e_op(a[sl], b, out=c[sl])
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                hc[sl].copy_(c[sl], non_blocking=True)
            h2d += self.e2e_rows * self.K * 2
            d2h += self.e2e_rows * self.N * 2
        main.wait_stream(s_out)
        return h2d, d2h

    def cpu_sample(self, target_s):
        import torch

        import oracle

        _, N, K = self.shape
        rows = 64
        a = oracle.to_bits(uniform_pm1((rows, K), self.seed + 1, "cpu").float().numpy(), "float16")
        b = oracle.to_bits(uniform_pm1((K, N), self.seed, "cpu").float().numpy(), "float16")

        def once():
            oracle.gemm16(a, b, "float16")

        return once, 2 * rows * N * K, f"({rows} rows of A) @ B[{K},{N}], fp32 accumulate"


class GemmGatherWorkload(GemmWorkload):
    """The M-split GEMM with the all-gather of C fused into the epilogue (peer stores over NVLink);
    the baseline is the unfused form: the same kernel into a local shard, then NCCL all-gather."""

    baseline_name = "same GEMM kernel into a local shard + NCCL all_gather_into_tensor"

    def config(self, world):
        c = super().config(world)
        M, N, _ = self.shape
        c["workload"] += ", C all-gathered by the epilogue"
        c["nvlink_bytes_per_launch_per_rank"] = (world - 1) * (M // world) * N * 2
        return c

    def setup(self, env):
        import torch
        import torch.distributed as dist

        from deca_b200.sharding import GatheredOutput, gemm_gather

        super().setup(env)
        a, b, c = self.sets[0]
        if env.world > 1:
            self.out = GatheredOutput.symmetric(self.M, self.N, torch.float16, a.device)
            full = torch.empty(env.world * self.M, self.N, dtype=torch.float16, device=a.device)

            def unfused():
                self.main(a, b, c)
                dist.all_gather_into_tensor(full, c)

            self.baseline = [unfused]
        else:
            self.out = GatheredOutput.from_tensors([c], 0)
            self.baseline = None
        self.launches = [lambda: gemm_gather(a, b, self.out, self.cfg)]
        self.kernel = f"gemm16 + peer stores {self.cfg}"

    def step_e2e(self):
        import torch

        from deca_b200.sharding import gemm_gather

        if not hasattr(self, "host"):
            self._e2e_setup()
        ha, hb, hc = self.host
        a, b, _ = self.sets[0]
        a.copy_(ha, non_blocking=True)
        b.copy_(hb, non_blocking=True)
        gemm_gather(a, b, self.out, self.cfg)
        mine = self.out.local[self.env.rank * self.M : (self.env.rank + 1) * self.M]
        hc.copy_(mine, non_blocking=True)
        return (ha.numel() + hb.numel()) * 2, hc.numel() * 2

    def verify(self):
        """Sampled row bands of EVERY rank's shard in this rank's gathered copy against the plain
        kernel on regenerated inputs of that rank (bit for bit)."""
        import torch

        from deca_b200.operators import GEMMTC

        env = self.env
        _, b, _ = self.sets[0]
        self.launches[0]()
        self.out.barrier()
        ok = True
        band = 256
        op = GEMMTC(band, self.N, self.K)
        for r in range(env.world):
            a_r = uniform_pm1((self.M, self.K), self.seed + 1 + 1000 * r)
            for off in (0, ((self.M // 2) // 8) * 8 + 8, self.M - band):
                want = op(a_r[off : off + band].contiguous(), b, cfg=self.cfg)
                got = self.out.local[r * self.M + off : r * self.M + off + band]
                ok = ok and bool(torch.equal(want, got))
            del a_r
        self.out.barrier()
        return max(env.max_over_ranks([0.0 if ok else 1.0])) == 0.0


class AttentionWorkload(Workload):
    """FlashAttention forward fp16, Q, K, V ~ N(0, 1).  ``shard_bh``: B*H is the whole problem's
    and each rank owns B*H / world heads."""

    metric = "FlashAttention forward throughput (4*B*H*S^2*D flops, halved when causal)"
    unit = "TFLOPS"
    dtype = "f16 x f16 -> f32 accumulate, f32 softmax, f16 out"
    bound = "tensor"
    baseline_name = "SDPA-flash (torch scaled_dot_product_attention, flash backend)"

    def __init__(self, B, H, S, D, causal, seed, shard_bh=False, launches_per_step=1, key=None):
        self.shape, self.causal, self.seed, self.shard_bh = (B, H, S, D), causal, seed, shard_bh
        self.sharded = shard_bh
        self.scaling = "strong" if shard_bh else "weak"
        self.launches_per_step = launches_per_step
        self.key = key or f"fa_{B}x{H}x{S}x{D}{'_causal' if causal else ''}"
        self.traffic_key = f"fa_fwd_f16_{B}x{H}x{S}x{D}{'_causal' if causal else ''}"

    def config(self, world):
        B, H, S, D = self.shape
        c = {"workload": f"FlashAttention fwd fp16 B={B} H={H} S={S} D={D} {'causal' if self.causal else 'non-causal'}"
                         + (" split along B*H" if self.shard_bh else ""),
             "B": B, "H": H, "S": S, "D": D, "causal": self.causal, "seed": self.seed, "inputs": "N(0,1)",
             "launches_per_step": self.launches_per_step}
        if self.shard_bh:
            c["heads_per_gpu"] = B * H // world
        set_bytes = 4 * (B * H // (world if self.shard_bh else 1)) * S * D * 2
        c["l2"] = ("inputs larger than L2, no flush" if set_bytes > (512 << 20)
                   else "rotating buffer sets, more than L2 between two uses of a buffer")
        return c

    def setup(self, env):
        import torch

        from deca_b200.kernels.attn_bench import sdpa_flash
        from deca_b200.operators import FlashAttention

        B, H, S, D = self.shape
        if self.shard_bh:
            assert (B * H) % env.world == 0
            B, H = 1, B * H // env.world
        self.B, self.H, self.S, self.D = B, H, S, D
        self.op = FlashAttention(B, H, S, S, D, causal=self.causal)
        self.cfg = self.op.default_config()
        self.main = self.op.compile(self.op.build_mod(self.cfg))["main"]
        set_bytes = 4 * B * H * S * D * 2
        n_sets = 1 if set_bytes > (512 << 20) else max(2, min(4, (400 << 20) // set_bytes + 1))
        self.sets = []
        for i in range(n_sets):
            g = torch.Generator(device="cuda").manual_seed(self.seed + 1000 * env.rank + 17 * i)
            q, k, v = (torch.randn(B, H, S, D, generator=g, device="cuda").half() for _ in range(3))
            self.sets.append((q, k, v, torch.empty_like(q)))
        self.launches = [lambda q=q, k=k, v=v, o=o: self.main(q, k, v, o) for q, k, v, o in self.sets]
        scale, causal = self.op.softmax_scale, self.causal
        self.baseline = [lambda q=q, k=k, v=v: sdpa_flash(q, k, v, causal=causal, scale=scale) for q, k, v, _ in self.sets]
        self.units = self.op.num_flops * (env.world if self.shard_bh else 1)
        self.traffic_key = f"fa_fwd_f16_{B}x{H}x{S}x{D}{'_causal' if self.causal else ''}"  # the shape one GPU runs
        self.kernel = f"fa_fwd {'causal' if self.causal else 'non-causal'} {self.cfg}"
        self.env = env

    def reference_kernel_groups(self, rk):
        q, k, v, o = self.sets[0]
        shape = (self.B, self.H, self.S, self.S, self.D)
        cands = [(e, (q, k, v, o)) for e in rk.entries("flash_attn", shape, causal=self.causal)]
        return [("flash_attn", cands, self.op.num_flops)] if cands and not self.shard_bh else []

    def step_e2e(self):
        import torch

        q, k, v, o = self.sets[0]
        if not hasattr(self, "host"):
            self.host = tuple(t.cpu().pin_memory() for t in (q, k, v)) + (torch.empty_like(o, device="cpu").pin_memory(),)
        hq, hk, hv, ho = self.host
        h2d = 0
        for src, dst in ((hq, q), (hk, k), (hv, v)):
            dst.copy_(src, non_blocking=True)
            h2d += src.numel() * 2
        self.op(q, k, v, out=o)
        ho.copy_(o, non_blocking=True)
        return h2d, ho.numel() * 2

    def cpu_sample(self, target_s):
        import torch

        import oracle

        _, _, S, D = self.shape
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        S_s = min(S, 2048)
        q, k, v = (oracle.to_bits(torch.randn(1, 1, S_s, D, generator=g).numpy(), "float16") for _ in range(3))
        causal = self.causal

        def once():
            oracle.attention(q, k, v, causal=causal)

        return once, 4 * S_s * S_s * D // (2 if causal else 1), f"one head, S={S_s}, D={D}, causal={causal}"


class AttentionGatherWorkload(AttentionWorkload):
    """The head-split attention with the all-gather of O fused into the epilogue."""

    baseline_name = "same attention kernel into a local shard + NCCL all_gather_into_tensor"

    def config(self, world):
        c = super().config(world)
        B, H, S, D = self.shape
        c["workload"] += ", O all-gathered by the epilogue"
        c["nvlink_bytes_per_launch_per_rank"] = (world - 1) * (B * H // world) * S * D * 2
        return c

    def setup(self, env):
        import torch
        import torch.distributed as dist

        from deca_b200.sharding import GatheredOutput, attention_gather

        super().setup(env)
        q, k, v, o = self.sets[0]
        rows = self.B * self.H * self.S
        if env.world > 1:
            self.out = GatheredOutput.symmetric(rows, self.D, torch.float16, q.device)
            full = torch.empty(env.world * o.numel(), dtype=torch.float16, device=o.device)

            def unfused():
                self.main(q, k, v, o)
                dist.all_gather_into_tensor(full, o.view(-1))

            self.baseline = [unfused]
        else:
            self.out = GatheredOutput.from_tensors([o.view(rows, self.D)], 0)
            self.baseline = None
        causal = self.causal
        self.launches = [lambda: attention_gather(q, k, v, self.out, causal=causal)]
        self.kernel = f"fa_fwd + peer stores {self.cfg}"

    def step_e2e(self):
        import torch

        from deca_b200.sharding import attention_gather

        q, k, v, o = self.sets[0]
        if not hasattr(self, "host"):
            self.host = tuple(t.cpu().pin_memory() for t in (q, k, v)) + (torch.empty_like(o, device="cpu").pin_memory(),)
        hq, hk, hv, ho = self.host
        h2d = 0
        for src, dst in ((hq, q), (hk, k), (hv, v)):
            dst.copy_(src, non_blocking=True)
            h2d += src.numel() * 2
        attention_gather(q, k, v, self.out, causal=self.causal)
        rows = self.B * self.H * self.S
        ho.view(rows, self.D).copy_(self.out.local[self.env.rank * rows : (self.env.rank + 1) * rows], non_blocking=True)
        return h2d, ho.numel() * 2

    def verify(self):
        """Two heads of EVERY rank's shard in this rank's gathered copy against the plain kernel on
        regenerated inputs of that rank (bit for bit)."""
        import torch

        env = self.env
        self.launches[0]()
        self.out.barrier()
        ok = True
        rows_head = self.S
        for r in range(env.world):
            g = torch.Generator(device="cuda").manual_seed(self.seed + 1000 * r)
            q, k, v = (torch.randn(self.B, self.H, self.S, self.D, generator=g, device="cuda").half() for _ in range(3))
            want = self.op(q, k, v)
            for h in (0, self.H - 1):
                base = (r * self.B * self.H + h) * rows_head
                ok = ok and bool(torch.equal(want[0, h], self.out.local[base : base + rows_head]))
            del q, k, v, want
        self.out.barrier()
        return max(env.max_over_ranks([0.0 if ok else 1.0])) == 0.0


def rowwise_host_inputs(M, N, seed=1):
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)
    x = 3.0 * torch.randn(M, N, generator=g)
    w = 1.0 + 0.1 * torch.randn(N, generator=g)
    return x, w


class RowwiseWorkload(Workload):
    """X[16384, 4096] ~ 3 N(0, 1) (seed 1), W ~ N(1, 0.1), eps 1e-6.  One round = softmax and RMSNorm,
    each in fp16 and bf16 (4 launches, 1 073 758 208 algorithmic bytes: read x [+ w], write y).  The
    two dtypes use different buffers and alternate, so 384 MB of other traffic passes between two
    reads of one input.  With several ranks every rank runs the same shape on its own rows."""

    key = "rowwise_16384x4096"
    metric = "softmax/RMSNorm effective HBM throughput (read x [+ w], write y)"
    unit = "TB/s"
    dtype = "f32 math, f16/bf16 I/O"
    bound = "hbm"
    scaling = "weak"
    sharded = True
    baseline_name = "eager torch (torch.softmax, F.rms_norm)"
    traffic_key = "rowwise_softmax_f16_16384x4096"
    M, N, EPS = 16384, 4096, 1e-6
    E2E_CHUNKS = 8

    def __init__(self, launches_per_step=4):
        self.launches_per_step = launches_per_step

    def config(self, world):
        return {"workload": "rowwise softmax+rmsnorm X[16384,4096] fp16+bf16", "M": self.M, "N": self.N, "eps": self.EPS,
                "seed": 1, "inputs": "X ~ 3*N(0,1), W ~ N(1,0.1)", "launches_per_step": self.launches_per_step,
                "rows": "every rank its own M rows" if world > 1 else "M rows",
                "l2": "inputs larger than L2; dtypes alternate buffers, no flush"}

    def setup(self, env):
        import torch
        import torch.nn.functional as F

        from deca_b200.operators import RMSNorm, Softmax

        x32, w32 = rowwise_host_inputs(self.M, self.N, seed=1 + 1000 * env.rank)
        self.host, self.dev, self.out, self.host_out, self.ops = {}, {}, {}, {}, []
        for dt, tdt in (("float16", torch.float16), ("bfloat16", torch.bfloat16)):
            self.host[dt] = (x32.to(tdt).pin_memory(), w32.to(tdt).pin_memory())
            self.dev[dt] = tuple(t.cuda() for t in self.host[dt])
        self.launches, self.baseline = [], []
        for kind, cls in (("softmax", Softmax), ("rmsnorm", RMSNorm)):
            for dt in ("float16", "bfloat16"):
                op = cls(self.M, self.N, dt) if kind == "softmax" else cls(self.M, self.N, dt, self.EPS)
                main = op.compile(op.build_mod(op.default_config()))["main"]
                key = (kind, dt)
                self.out[key] = torch.empty_like(self.dev[dt][0])
                x, w = self.dev[dt]
                y = self.out[key]
                if kind == "softmax":
                    self.launches.append(lambda main=main, x=x, y=y: main(x, y))
                    self.baseline.append(lambda x=x, y=y: torch.softmax(x, dim=-1, out=y))
                else:
                    self.launches.append(lambda main=main, x=x, w=w, y=y: main(x, w, y))
                    self.baseline.append(lambda x=x, w=w: F.rms_norm(x, (x.shape[-1],), w, eps=self.EPS))
                self.ops.append((key, op))
        # `units` is per launch on average (the four launches of a round move almost equal bytes)
        self.units = sum(op.num_bytes for _, op in self.ops) / len(self.ops) * env.world
        self.dominant_units = self.ops[0][1].num_bytes
        self.kernel = f"rowwise_reg softmax/rmsnorm {self.ops[0][1].default_config()}"
        self.env = env

    def reference_kernel_groups(self, rk):
        groups = []
        for (kind, dt), op in self.ops:
            x, w = self.dev[dt]
            tensors = (x, self.out[(kind, dt)]) if kind == "softmax" else (x, w, self.out[(kind, dt)])
            cands = [(e, tensors) for e in rk.entries("rowwise", (self.M, self.N), op=kind, dtype=dt)]
            if not cands:
                return []
            groups.append((f"{kind} {dt}", cands, op.num_bytes))
        return groups

    def _e2e_setup(self):
        import torch

        from deca_b200.operators import RMSNorm, Softmax

        rows = self.M // self.E2E_CHUNKS
        self._e2e_rows = rows
        self._e2e_ops = {}
        for dt in ("float16", "bfloat16"):
            self._e2e_ops[("softmax", dt)] = Softmax(rows, self.N, dt)
            self._e2e_ops[("rmsnorm", dt)] = RMSNorm(rows, self.N, dt, self.EPS)
            for kind in ("softmax", "rmsnorm"):
                self.host_out[(kind, dt)] = torch.empty_like(self.host[dt][0]).pin_memory()
        self._s_in, self._s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step_e2e(self):
        """Host pinned inputs -> device -> operator calls -> host pinned outputs, chunked by rows:
        copies in both directions and kernels of different chunks overlap on three streams."""
        import torch

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

    def cpu_sample(self, target_s):
        import oracle

        rows = 2048
        x32, w32 = rowwise_host_inputs(rows, self.N, seed=1)
        data = {dt: (oracle.to_bits(x32.numpy(), dt), oracle.to_bits(w32.numpy(), dt)) for dt in ("float16", "bfloat16")}
        nbytes_once = 2 * (2 * rows * self.N * 2) + 2 * (2 * rows * self.N * 2 + self.N * 2)

        def once():
            for dt in ("float16", "bfloat16"):
                oracle.softmax(data[dt][0], dt)
            for dt in ("float16", "bfloat16"):
                oracle.rmsnorm(data[dt][0], data[dt][1], self.EPS, dt)

        return once, nbytes_once, f"(softmax+rmsnorm, fp16+bf16) on {rows} of {self.M} rows x {self.N}"


def make_workload(name):
    if name == "gemm_sharded":
        return GemmWorkload(65536, 8192, 8192, seed=4, shard_m=True, launches_per_step=16, key="gemm_sharded")
    if name == "gemm_gather":
        return GemmGatherWorkload(65536, 8192, 8192, seed=4, shard_m=True, launches_per_step=4, key="gemm_gather")
    if name == "gemm":
        return GemmWorkload(4096, 4096, 4096, seed=2, launches_per_step=64, key="gemm")
    if name == "attention":
        return AttentionWorkload(4, 16, 4096, 128, False, seed=3, launches_per_step=16, key="attention")
    if name == "attention_sharded":
        return AttentionWorkload(32, 32, 8192, 128, True, seed=4, shard_bh=True, launches_per_step=4, key="attention_sharded")
    if name == "attention_gather":
        return AttentionGatherWorkload(32, 32, 8192, 128, True, seed=4, shard_bh=True, launches_per_step=2, key="attention_gather")
    if name == "rowwise":
        return RowwiseWorkload(launches_per_step=4)
    raise SystemExit(f"unknown workload {name}")


def default_records(world, headline_key):
    recs = []
    if world == 1:
        for n in (4096, 8192, 16384, 2048):
            recs.append(GemmWorkload(n, n, n, seed=2))
        for D in (128, 64):
            for causal in (False, True):
                recs.append(AttentionWorkload(4, 16, 4096, D, causal, seed=3))
    recs.append(RowwiseWorkload())
    recs.append(AttentionWorkload(32, 32, 8192, 128, True, seed=4, shard_bh=True, key="attention_sharded"))
    return [r for r in recs if r.key != headline_key]


# ------------------------------------------------------------------------------------------
# Measurement
# ------------------------------------------------------------------------------------------
def capture_graph(fns, reps=1):
    """One CUDA graph holding `reps` rounds of the launches in `fns`, or None when capture fails
    (the callers then launch directly)."""
    import torch

    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(reps):
                    for fn in fns:
                        fn()
        torch.cuda.current_stream().wait_stream(side)
        g.replay()
        torch.cuda.synchronize()
        return g
    except Exception:  # noqa: BLE001
        torch.cuda.synchronize()
        return None


def burst_runner(fns, use_graph):
    """run(rounds): `rounds` rounds of the launches in `fns`, through a graph of one round if possible."""
    g = capture_graph(fns) if use_graph else None

    def run(rounds):
        if g is not None:
            for _ in range(rounds):
                g.replay()
        else:
            for _ in range(rounds):
                for fn in fns:
                    fn()

    return run, g is not None


def time_ms(run, rounds):
    import torch

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(rounds)
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1)


def roofline_of(wl, achieved_units_per_s, avg_launch_ms, peaks, traffic):
    """`achieved` against the measured peak: HBM copy bandwidth, or the cuBLAS bf16 figure
    (sustained, since every timed region here is seconds of back-to-back launches)."""
    if wl.bound == "hbm":
        a = achieved_units_per_s / 1e9
        return {"bound": "hbm", "kernel": wl.kernel, "achieved": a, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": a / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
                "frac_nominal": a / NOMINAL_HBM_GBS, "avg_launch_us": avg_launch_ms * 1e3, "traffic": traffic}
    a = achieved_units_per_s / 1e12
    return {"bound": "tensor", "kernel": wl.kernel, "achieved": a, "peak": peaks["bf16_tflops_sustained"],
            "unit": "TFLOP/s", "frac": a / peaks["bf16_tflops_sustained"],
            "peak_source": peaks["source"] + " cuBLAS bf16, sustained (seconds-long timed region)",
            "frac_sustained": a / peaks["bf16_tflops_sustained"], "frac_burst": a / peaks["bf16_tflops"],
            "frac_nominal": a / NOMINAL_F16_TFLOPS, "avg_launch_us": avg_launch_ms * 1e3, "traffic": traffic}


def measure_record(wl, env, peaks, seconds, use_graph, bursts=4):
    """Device-resident inputs; `bursts` bursts of our launches alternate with bursts of the
    baseline on the same tensors; clocks are sampled during our bursts only."""
    wl.setup(env)
    n = len(wl.launches)
    run, graphed = burst_runner(wl.launches, use_graph)
    run_base = burst_runner(wl.baseline, use_graph)[0] if wl.baseline else None
    for _ in range(3):
        run(1)
        if run_base:
            run_base(1)
    env.barrier()
    t_round = max(env.max_over_ranks([time_ms(run, 2) / 2])[0], 1e-3)
    rounds = max(1, int(seconds * 1e3 / bursts / t_round + 0.5))
    if run_base:
        t_base = max(env.max_over_ranks([time_ms(run_base, 2) / 2])[0], 1e-3)
        rounds_base = max(1, int(min(seconds, 1.5) * 1e3 / bursts / t_base + 0.5))
    ours, base = [], []
    with ClockSampler(env.local_rank) as clk:
        for _ in range(bursts):
            env.barrier()
            clk.active.set()
            ours.append(time_ms(run, rounds))
            clk.active.clear()
            if run_base:
                env.barrier()
                base.append(time_ms(run_base, rounds_base))
    ours_ms = sum(env.max_over_ranks(ours))
    launches = rounds * bursts * n
    value = wl.to_value(wl.units * launches / (ours_ms / 1e3))
    avg_launch_ms = ours_ms / launches
    clocks = clk.summary()
    rec = {"workload": wl.config(env.world)["workload"], "value": value, "unit": wl.unit,
           "ms": ours_ms, "launches": launches, "launch_mode": "cuda_graph" if graphed else "python",
           "scaling": wl.scaling, "config": wl.config(env.world), "kernel_config": str(getattr(wl, "cfg", "")),
           "roofline": roofline_of(wl, wl.units / (env.world if wl.sharded else 1) / (avg_launch_ms / 1e3), avg_launch_ms,
                                   peaks, NCU_TRAFFIC_BYTES.get(wl.traffic_key)),
           "clocks": clocks, "clocks_ok": clock_summary_ok(clocks)}
    if clocks.get("sm_mhz"):
        rec["value_per_sm_mhz"] = value / clocks["sm_mhz"]
    if run_base:
        base_ms = sum(env.max_over_ranks(base))
        base_value = wl.to_value(wl.units * rounds_base * bursts * n / (base_ms / 1e3))
        rec["comparison"] = {"what": wl.baseline_name + ", timed alternately on the same tensors", "value": base_value,
                             "unit": wl.unit, "ratio": value / base_value}
    if env.world == 1:
        rec["comparison_reference_kernels"] = reference_kernels_leg(wl, value)
    if hasattr(wl, "verify"):
        rec["verified"] = wl.verify()
    return rec


def reference_kernels_leg(wl, value, seconds=0.25):
    """The reference's own mma.sync / cp.async kernels (generated by its TIR generators, prebuilt
    for sm_100a) on the same tensors, beside the timed region: per launch of the workload the
    fastest of the prebuilt configs.  A baseline and a sanity check, never the thing measured."""
    import torch

    try:
        from oracle import ref_kernels as rk

        why = rk.unavailable_reason()
    except Exception as e:  # noqa: BLE001
        why = f"{type(e).__name__}: {str(e)[-120:]}"
    if why:
        return {"unavailable": why}
    groups = wl.reference_kernel_groups(rk) if hasattr(wl, "reference_kernel_groups") else []
    if not groups:
        return {"unavailable": "no prebuilt reference kernel for this shape"}
    total_s, total_units, picks = 0.0, 0.0, []
    for label, cands, units in groups:
        best = None
        for entry, tensors in cands:
            launch = rk.bind(entry, *tensors)
            launch()
            torch.cuda.synchronize()
            t1 = max(time_ms(lambda r: [launch() for _ in range(r)], 2) / 2, 1e-3)
            reps = max(3, int(seconds * 1e3 / t1))
            t = time_ms(lambda r: [launch() for _ in range(r)], reps) / reps / 1e3
            if best is None or t < best[0]:
                best = (t, entry["config_str"])
        total_s += best[0]
        total_units += units
        picks.append(f"{label}: {best[1]}")
    ref_value = wl.to_value(total_units / total_s)
    return {"what": "the reference's own generated kernels (mma.sync, prebuilt for sm_100a), best prebuilt config, same tensors",
            "configs": picks, "value": ref_value, "unit": wl.unit, "ratio": value / ref_value}


def host_link_probe(env, nbytes=256 << 20):
    """Pinned-host <-> device copy rates of this rank, alone (rank 0 while the others wait) and
    with all ranks copying at once: names the ceiling of the end-to-end numbers."""
    import torch

    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dev = torch.empty(nbytes, dtype=torch.uint8, device="cuda")

    def rate(direction):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            (dev.copy_(host, non_blocking=True) if direction == "h2d" else host.copy_(dev, non_blocking=True))
        e1.record()
        e1.synchronize()
        return 4 * nbytes / (e0.elapsed_time(e1) / 1e3) / 1e9

    out = {}
    rate("h2d"), rate("d2h")
    env.barrier()
    if env.rank == 0:
        out["alone_h2d_gbs"], out["alone_d2h_gbs"] = rate("h2d"), rate("d2h")
    env.barrier()
    if env.world > 1:
        h, d = rate("h2d"), rate("d2h")
        env.barrier()
        # slowest rank while all copy
        out["all_ranks_h2d_gbs_min"] = -env.max_over_ranks([-h])[0]
        out["all_ranks_d2h_gbs_min"] = -env.max_over_ranks([-d])[0]
    return out


def run_cpu_arm(wl, steps, warmup, as_reference_line):
    import oracle

    oracle.set_num_threads()  # all host cores, whatever OMP_NUM_THREADS the launcher exported
    # reference arm: every step is a bounded sample, sized so that W + K steps take about 2 minutes
    step_s = 12.0 if not as_reference_line else max(0.05, min(4.0, 120.0 / max(1, steps + warmup)))
    once, units_once, what = wl.cpu_sample(step_s)
    once()
    t0 = time.perf_counter()
    once()
    t1 = time.perf_counter() - t0
    reps = max(1, int(step_s / max(t1, 1e-3)))
    if as_reference_line:
        for _ in range(warmup):
            once()
        t0 = time.perf_counter()
        for _ in range(steps):
            for _ in range(reps):
                once()
        per_step = (time.perf_counter() - t0) / steps
    else:
        t0 = time.perf_counter()
        for _ in range(reps):
            once()
        per_step = time.perf_counter() - t0
    value = wl.to_value(units_once * reps / per_step)
    base = {"value": value, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port", "sample": f"{reps} x {what}"}
    return base, per_step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="gemm_sharded")
    ap.add_argument("--records", default="all", help="all, none, or a comma list of record keys")
    ap.add_argument("--seconds", type=float, default=2.0, help="device time of our kernel per record")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying CUDA graphs")
    ap.add_argument("--gemm-tile", default=None, help="GEMM workloads: BMxBN:stages:acc_bufs[:cta_group] instead of the default config")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl = make_workload(args.workload)

    if args.impl == "reference":
        # The reference has no CPU implementation of these kernels (its TIR uses PTX intrinsics);
        # its arithmetic, restated in oracle/, is what runs here, on all host threads.
        if rank != 0:
            return
        base, per_step = run_cpu_arm(wl, args.steps, args.warmup, True)
        line = {"impl": "reference", "metric": wl.metric, "value": base["value"], "unit": wl.unit, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
                "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype,
                "data": "synthetic", "config": wl.config(args.gpus), "cpu_baseline": base,
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
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    env = Env(rank, local_rank, world, dist)
    if args.gemm_tile:
        GemmWorkload.tile_override = args.gemm_tile
    peaks = measured_peaks()
    use_graph = not args.no_graph
    warmup = max(args.warmup, 3)

    # ---------------- headline: W warm-up steps, then exactly K steps between two events ----------------
    wl.setup(env)
    n = len(wl.launches)
    L = wl.launches_per_step
    step_fns = [wl.launches[i % n] for i in range(L)]
    step_graph = capture_graph(step_fns) if use_graph else None

    def run_step():
        if step_graph is not None:
            step_graph.replay()
        else:
            for fn in step_fns:
                fn()

    for _ in range(warmup):
        run_step()
    env.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        env.barrier()
        clk.active.set()
        start.record()
        for _ in range(args.steps):
            run_step()
        end.record()
        torch.cuda.synchronize()
        clk.active.clear()
        env.barrier()
    total_ms = env.max_over_ranks([start.elapsed_time(end)])[0]
    launches = L * args.steps
    value = wl.to_value(wl.units * launches / (total_ms / 1e3))
    avg_launch_ms = total_ms / launches
    per_gpu_units = wl.units / (world if wl.sharded else 1)
    clocks = clk.summary()

    # comparison: the library baseline on the same tensors, same number of launches, right after
    comparison = None
    if wl.baseline:
        nb = len(wl.baseline)
        base_fns = [wl.baseline[i % nb] for i in range(L)]
        base_graph = capture_graph(base_fns) if use_graph else None

        def run_base(rounds):
            for _ in range(rounds):
                if base_graph is not None:
                    base_graph.replay()
                else:
                    for fn in base_fns:
                        fn()

        run_base(2)
        env.barrier()
        base_ms = env.max_over_ranks([time_ms(run_base, args.steps)])[0]
        env.barrier()
        # and our kernel again after it, so that both saw the same state of the part
        again_ms = env.max_over_ranks([time_ms(lambda r: [run_step() for _ in range(r)], args.steps)])[0]
        base_value = wl.to_value(wl.units * launches / (base_ms / 1e3))
        comparison = {"what": wl.baseline_name + ", same tensors, same launch count, timed between two runs of ours",
                      "value": base_value, "unit": wl.unit, "ms_per_step": base_ms / args.steps,
                      "ours_after_ms_per_step": again_ms / args.steps,
                      "ratio": value / base_value,
                      "ratio_mean_of_before_and_after": (wl.units * launches / ((total_ms + again_ms) / 2e3)) / (wl.units * launches / (base_ms / 1e3))}

    verified = wl.verify() if hasattr(wl, "verify") else None

    # ---------------- e2e: host buffers through the operator API ----------------
    wl.step_e2e()
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.e2e_steps):
        h2d, d2h = wl.step_e2e()
    e1.record()
    torch.cuda.synchronize()
    env.barrier()
    e2e_ms = env.max_over_ranks([e0.elapsed_time(e1)])[0]
    e2e_value = wl.to_value(wl.units * args.e2e_steps / (e2e_ms / 1e3))
    link = host_link_probe(env)

    headline = {
        "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(world),
        "kernel_config": str(getattr(wl, "cfg", "")),
        "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.e2e_steps, "host_link": link},
        "gpu_launches": launches, "launch_mode": "cuda_graph" if step_graph is not None else "python",
        "roofline": roofline_of(wl, per_gpu_units / (avg_launch_ms / 1e3), avg_launch_ms, peaks,
                                NCU_TRAFFIC_BYTES.get(wl.traffic_key)),
        "clocks": clocks, "clocks_ok": clock_summary_ok(clocks),
    }
    if clocks.get("sm_mhz"):
        headline["value_per_sm_mhz"] = value / clocks["sm_mhz"]
    if comparison is not None:
        headline["comparison"] = comparison
    if verified is not None:
        headline["verified"] = verified
    headline_key = wl.key
    del step_graph, run_step
    if wl.baseline:
        del base_graph, run_base
    wl.teardown()

    # ---------------- the other configurations of the metric ----------------
    records = {}
    if args.records != "none":
        wanted = None if args.records == "all" else set(args.records.split(","))
        for rec in default_records(world, headline_key):
            if wanted is not None and rec.key not in wanted:
                continue
            if world > 1 and not rec.sharded:
                continue
            try:
                records[rec.key] = measure_record(rec, env, peaks, args.seconds, use_graph)
            except Exception as e:  # noqa: BLE001  (e.g. out of memory on a shared GPU): keep the line
                records[rec.key] = {"error": f"{type(e).__name__}: {str(e)[-300:]}"}
                torch.cuda.synchronize()
            rec.teardown()

    if rank == 0:
        headline["records"] = records
        if not args.no_cpu_baseline and world == 1:
            headline["cpu_baseline"], _ = run_cpu_arm(make_workload(args.workload), 1, 0, False)
        print(json.dumps(headline), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
