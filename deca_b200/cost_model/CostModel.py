"""Analytic ranking of kernel configurations on B200.

Same entry points as the reference's src/cost_model/CostModel.py -- ``gemm_tc_score`` (:207-271),
``fa_score`` (:37-93), ``rowwise_score`` (:116-164) and the ``rank_*`` helpers (:96-99,
:274-283) -- retargeted to the tcgen05 / TMA kernels: the tensor pipe is modelled by
``arch.peak_tcgen05_flops``, operand traffic by the MMA's shared-memory reads and the TMA's
L2 reads per flop, the epilogue by whether a second tensor-memory accumulator hides it, and
the row-wise kernels by bytes in flight against Little's law.  Scores are "larger is better"
and only meaningful relative to each other.
"""

import math

from ..arch.Arch import Arch


class CostModel:
    def __init__(self):
        pass

    def cost(self, kernel, arch: Arch, compute_pattern):
        pass


# --------------------------------------------------------------------------------------- GEMM
def gemm_tc_occupancy(cfg, arch: Arch):
    """Resident CTAs per SM: the kernel is persistent with one CTA per SM."""
    return 1


def gemm_wave_dram_bytes_per_flop(cfg, arch: Arch, M: int, N: int, K: int, slots: int) -> float:
    """DRAM bytes per flop of A / B for one wave of ``slots`` concurrent tiles walking the
    output in groups of ``raster`` tile rows; operands that fit in half the L2 are fetched once."""
    if (M * K + K * N) * 2 <= 0.5 * arch.l2_bytes:
        return (M * K + K * N) * 2 / (2.0 * M * N * K)
    GM, GN, BM, BN = -(-M // cfg.BM), -(-N // cfg.BN), cfg.BM, cfg.BN
    if getattr(cfg, "raster_n", False):  # groups of tile columns walked down M: the roles of M and N swap
        GM, GN, BM, BN = GN, GM, BN, BM
    g = max(1, min(cfg.raster, GM))
    cols = min(GN, math.ceil(slots / g))
    rows = min(GM, g * math.ceil(slots / (g * GN)))
    tiles = min(slots, GM * GN)
    return (rows * BM + cols * BN) / (tiles * BM * BN)


def gemm_tc_score(cfg, arch: Arch, M: int, N: int, K: int) -> float:
    """Heuristic score of a tcgen05 GEMM config.

    Per-SM time per flop of the main loop as a roofline whose terms overlap almost fully (TMA
    and MMA are asynchronous to each other):
    - tensor pipe at ``arch.peak_tcgen05_flops``
    - shared memory: per 16-deep k step the MMAs read BM*32 bytes of A and, once per 128-row
      half, BN*32 bytes of B, for 2*BM*BN*16 flops, against 128 B/clk
    - L2 -> SM: (BM + BN) * 128 bytes per 64-deep K block for 2*BM*BN*64 flops
    - DRAM: unique A / B bytes of one wave (grouped rasterisation)
    Then wave quantisation of the persistent grid, ring depth against ~1 us of L2 latency,
    the epilogue (hidden by a second accumulator, else serial), wasted columns of partial tiles.
    """
    sm = arch.sm_nums
    halves = cfg.BM // 128
    peak = arch.peak_tcgen05_flops * 1e9
    t_mma = sm / peak
    # CTA pairs: each CTA fetches and reads only its half of the B columns, and a tile (2 BM rows)
    # occupies two SMs
    pair = getattr(cfg, "cta_group", 1) == 2
    bn_own = cfg.BN // 2 if pair else cfg.BN
    smem_bpf = (cfg.BM * 32 + halves * bn_own * 32) / (2.0 * cfg.BM * cfg.BN * 16)
    t_smem = smem_bpf / arch.smem_bw_per_sm
    l2_bpf = (cfg.BM + bn_own) / (cfg.BM * cfg.BN)
    t_l2 = l2_bpf * sm / (arch.l2_bw * 1e9)
    GM, GN = -(-M // cfg.BM), -(-N // cfg.BN)
    if pair:
        GM = 2 * -(-M // (2 * cfg.BM))  # rows come in pair tiles
    tiles = GM * GN
    slots = min(sm, tiles)
    t_dram = gemm_wave_dram_bytes_per_flop(cfg, arch, M, N, K, slots) * sm / (arch.dram_bw * 1e9)
    terms = sorted([t_mma, t_smem, t_l2, t_dram])
    t_flop = terms[-1] + 0.1 * sum(terms[:-1])

    waves = math.ceil(tiles / sm)
    wave_eff = tiles / (waves * sm)
    if getattr(cfg, "stream_k", False):
        from ..kernels.gemm_b200 import stream_k_plan

        plan = stream_k_plan(cfg, M, N, K, sm)
        if plan is not None:
            # equal shares per SM remove the wave tail, but the CTAs then walk k out of step and
            # the operand reads lose their reuse in time (0.85), and every CTA writes one partial
            # tile and reads another, worth about 16 k blocks of its time; fitted to 4096^3
            # (1219 against 1400 TFLOPS whole-tile) and 2048^3 (440 against 610)
            grid, dp_tiles, sk_units = plan
            share = dp_tiles / grid * math.ceil(K / cfg.BK) + sk_units / grid
            wave_eff = 0.85 * share / (share + 16.0)
    useful = (M * N) / (GM * cfg.BM * GN * cfg.BN)  # partial tiles compute zero-filled rows / columns

    # bytes in flight per SM needed to cover ~1 us of L2 latency at the MMA's consumption rate
    need = l2_bpf / t_mma * 1e-6
    in_flight = (cfg.stages - 1) * (cfg.BM + cfg.BN) * 128
    pipe = min(1.0, in_flight / need) ** 0.5
    pipe *= 1.0 - getattr(arch, "gemm_excess_stage_penalty", 0.0) * max(0, cfg.stages - 1 - math.ceil(need / ((cfg.BM + cfg.BN) * 128)))

    # epilogue: ~(BM/32 warps-rows) x (BN/64) panels of ~500 cycles per warp, 4 warps in parallel
    tile_cycles = 2.0 * cfg.BM * cfg.BN * K / (peak / sm / arch.sm_clock_hz)
    epi_cycles = (cfg.BM // 128) * (cfg.BN // 64) * (500 if cfg.epi_smem else 900)
    epi = 1.0 if cfg.acc_bufs == 2 else tile_cycles / (tile_cycles + epi_cycles)
    if cfg.acc_bufs == 2 and not cfg.epi_smem:
        epi = 0.97

    # How far A and B outgrow L2 (0 at half of L2, 1 from twice L2 on).  Kernels of that size run for
    # milliseconds at the part's power limit, and two measured preferences come with it: the tile
    # order matters (groups of 8 tile rows best; 16 re-read more DRAM than 8 in ncu and measure 1 - 3 %
    # lower, 4 about 1 %, 2 and 1 up to 10 %), and the one-CTA 256 x 256 tile overtakes the CTA-pair
    # tile on most GPUs of the pool (by 1.5 - 3 % at 6144^3 ... 16384^3: it does a little less per clock but
    # is given a higher clock; on one box the pair tile led by 1.4 % instead), while at 4096^3, where wave
    # tails leave power to spare, the pair tile leads by up to 1.5 %.
    big = min(1.0, max(0.0, ((M * K + K * N) * 2 / arch.l2_bytes - 0.5) / 1.5))
    order = {1: 0.93, 2: 0.96, 4: 0.985, 8: 1.0, 16: 0.98}.get(cfg.raster, 0.99 if cfg.raster > 8 else 0.97)
    rate = 1.0 - big * (1.0 - order)
    if pair:
        rate *= 1.0 - 0.02 * big  # leaves the pair tile of the best order between the one-CTA tile's two best orders
    if pair:
        # measured: the pair kernel matches the one-CTA kernel tile for tile (512 x 256 pair tile
        # 1312-1371 TFLOPS at 4096^3, 256 x 256 pair tile 1163, narrower ones 700-850), so its
        # smaller tiles are ranked like the one-CTA tiles with the same rows and columns per CTA
        rate *= {(256, 256): 0.97, (128, 256): 0.85, (256, 128): 0.62, (128, 128): 0.52}.get((cfg.BM, cfg.BN), 0.5)
    return rate * wave_eff * useful * pipe * epi / (t_flop / t_mma)


def rank_gemm_configs(configs, arch: Arch, M: int, N: int, K: int, top_n: int | None = None):
    """Sort GEMM configs by ``gemm_tc_score`` (best first)."""
    ranked = sorted(configs, key=lambda c: gemm_tc_score(c, arch, M, N, K), reverse=True)
    return ranked[:top_n] if top_n else ranked


# ---------------------------------------------------------------------------- FlashAttention
def fa_occupancy(cfg, arch: Arch, D: int, grid: int):
    """(resident CTAs per SM, occupancy): shared memory and tensor memory allow one CTA."""
    from ..kernels.flash_attn_b200 import smem_bytes, tmem_columns

    by_smem = (max(arch.shared_mem_config_options) * 1024) // (smem_bytes(cfg, D) + 1024)
    by_tmem = getattr(arch, "tmem_columns", 512) // tmem_columns(cfg, D)
    ctas = max(1, min(by_smem, by_tmem))
    return ctas, ctas * cfg.threads / 32 / arch.max_resident_warps_per_sm


def fa_score(cfg, arch: Arch, shape, causal: bool = False) -> float:
    """Heuristic score of a FlashAttention config.

    Per KV tile and 128-row Q tile the tensor pipe needs 4*128*Bc*D / flops-per-clk cycles; the
    softmax warps need 128*Bc / 16 cycles of the exp2 unit (16 per clk per SM) plus about three
    fp32 instructions per score over 128 lanes.  The MMA of the next score tile and the P V
    product of the previous one overlap the softmax, so the tile time is the larger of the two
    plus a hand-off (barrier round trips, tcgen05.ld latency).  Shared memory is a second
    bound: both MMAs read both operands from it (Q and K, P and V) and P is written to it.
    Causal: the diagonal tile is computed in full, so only the useful share of it counts; the
    wave tail of the grid and the K/V ring depth (latency hiding) complete the model.
    """
    B, H, S_q, S_kv, D = shape
    clk = arch.sm_clock_hz
    fpc = arch.peak_tcgen05_flops * 1e9 / arch.sm_nums / clk  # flops per clock per SM
    flops_tile = 4.0 * 128 * cfg.Bc * D
    mma = flops_tile / fpc
    # softmax: one warp per scheduler, so dependent-instruction latency shows; fitted to B200
    # measurements at B4 H16 S4096 (about 0.20 clk per score at Bc = 64, 0.26 at Bc = 128)
    softmax = 128.0 * cfg.Bc * (0.14 + 0.0009 * cfg.Bc)
    # operand delivery: the K and V tiles of one step and the MMAs' shared-memory reads
    operands = 16.0 * D * (cfg.Bc / 64.0)
    handoff = 300.0
    tile = max(mma, softmax, operands) + handoff
    eff = mma / tile
    # two Q tiles per CTA with P in tensor memory: no P traffic through shared memory and the
    # MMAs of one tile overlap the softmax of the other (measured +25 % at D = 128 and, against
    # the one-tile 128-key schedule, +30 % at D = 64, which is +8 % over the best one-tile config;
    # with P in shared memory the two-tile schedule measured no faster than one tile)
    if getattr(cfg, "p_tmem", False):
        if cfg.q_tiles == 2 and cfg.Bc == 64:
            eff *= 0.6  # two score buffers per tile, but twice the barrier round trips (measured)
        elif cfg.q_tiles == 2:
            eff *= 1.25 if D >= 128 else 1.30
        else:
            # one tile: the softmax warps are the critical path either way; a small gain at D = 64,
            # a small loss at D = 128 (measured)
            eff *= 1.03 if D <= 64 else 0.97

    if getattr(cfg, "persistent", False):
        # no CTA start / end per item: the fixed cost of a pair of Q tiles (about two KV steps)
        # overlaps the neighbouring items (measured +4 % at S = 4096, +30 % at S = 512)
        steps = S_kv / cfg.Bc * (0.5 if causal else 1.0)
        eff *= (steps + 2.0) / (steps + 0.7)
    n_q = S_q // cfg.Br
    grid = n_q * B * H
    ctas, _ = fa_occupancy(cfg, arch, D, grid)
    slots = arch.sm_nums * ctas
    wave_eff = grid / (math.ceil(grid / slots) * slots)
    # ring depth in K/V pairs: the two-tile kernel keeps K and V tiles in one ring
    depth = cfg.stages / 2.0 if cfg.q_tiles == 2 else float(cfg.stages)
    pipe = 1.0 if depth >= 2 else (0.93 if depth <= 1 else 0.96)
    pipe *= 1.0 - 0.01 * max(0.0, depth - 2)
    useful = 1.0
    if causal:
        computed = sum(-(-(i + 1) * cfg.Br // cfg.Bc) * cfg.Bc for i in range(n_q)) * cfg.Br
        useful = S_q * (S_q + 1) / 2 / computed
    sync = 1.0 / (1.0 + getattr(arch, "fa_cta_sync_penalty", 0.0))
    return eff * wave_eff * pipe * useful * sync


def rank_fa_configs(configs, arch: Arch, shape, causal: bool = False, top_n: int | None = None):
    """Sort FlashAttention configs by ``fa_score`` (best first)."""
    ranked = sorted(configs, key=lambda c: fa_score(c, arch, shape, causal), reverse=True)
    return ranked[:top_n] if top_n else ranked


# ---------------------------------------------------------------------------------- row-wise
def rowwise_occupancy(cfg, arch: Arch, op: str, N: int):
    """Resident CTAs per SM of a row-wise config (the bulk-copy mode is one persistent CTA)."""
    from ..kernels.rowwise_b200 import est_regs_per_thread

    if cfg.mode == "tma":
        return 1
    regs = (min(255, est_regs_per_thread(cfg, N, op)) + 7) // 8 * 8
    if cfg.mode == "twopass":
        # ptxas -v: 32 / 40 / 56 registers at 8 / 16 / 32 elements per iteration (the validity rule's
        # estimate is deliberately higher)
        regs = max(32, (24 + cfg.unroll * cfg.vec + 7) // 8 * 8)
    warps = cfg.threads // 32
    ctas = min(arch.max_registers_per_sm // (regs * cfg.threads), arch.max_resident_warps_per_sm // warps,
               arch.max_resident_blocks_per_sm)
    return max(int(ctas), 1)


def rowwise_terms(cfg, arch: Arch, op: str, M: int, N: int, type_size: int = 2) -> dict:
    """The factors of ``rowwise_score`` by name (their product is the score).

    - memory parallelism: bytes of loads in flight per SM against Little's law (DRAM bandwidth
      per SM x ``arch.dram_latency_s``).  reg: every chunk of the row is requested up front by all
      resident threads, but a CTA loads, reduces, then stores, so only part of the residents are
      in their load phase; tma: rows_per_block * unroll whole rows are always in flight
    - issue pressure: the arithmetic costs about 8 instructions per element (softmax) or 5
      (RMSNorm); one persistent 512-thread CTA cannot issue them fast enough at full bandwidth,
      many small resident CTAs can (measured: reg 128-thread CTAs reach 95 % of the copy
      bandwidth at 16384 x 4096, the bulk-copy mode 70 %)
    - block barriers couple the rows of a CTA: rows_per_block > 1 costs (measured -12 % per doubling)
    - wave efficiency, twopass re-read (from L2 when the rows in flight fit), cross-warp
      reductions, tail lanes, 8-byte accesses as in the reference's model
    """
    from ..kernels.rowwise_b200 import num_chunks

    ctas = rowwise_occupancy(cfg, arch, op, N)
    chunks = num_chunks(cfg, N)
    need = arch.dram_bw * 1e9 / arch.sm_nums * getattr(arch, "dram_latency_s", 1e-6)
    grid = 0 if cfg.mode == "tma" else M // cfg.rows_per_block * (cfg.unroll if cfg.mode == "cluster" else 1)
    if cfg.mode == "tma":
        in_flight = cfg.rows_per_block * cfg.unroll * N * type_size
        phase = 1.0
    else:
        # a grid below one wave is resident all at once: fewer CTAs per SM than the limit allows
        ctas = max(1.0, min(float(ctas), grid / arch.sm_nums))
        cached = cfg.mode in ("reg", "cluster")  # the whole row (slice) is requested up front
        per_thread = (chunks if cached else cfg.unroll) * cfg.vec * type_size
        in_flight = ctas * cfg.threads * per_thread
        phase = 1.0 - 0.35 / ctas if cached else 1.0 - 0.1 / ctas
    mem = min(1.0, in_flight / need)
    if cfg.mode == "twopass":
        # streaming loop: a row of few iterations never reaches a steady state of loads in flight
        # (32000 columns, 512 threads: 2 iterations of 4 chunks run at 0.76 of 8 iterations of 2), and
        # more, smaller CTAs make up for fewer chunks per iteration
        its = chunks / cfg.unroll
        mem = mem ** 0.5 * its / (its + 0.75)

    # instruction issue: elements per clock per SM needed at full bandwidth vs what the resident
    # warps can issue (4 schedulers; one CTA's phases serialise on its barriers)
    inst_per_elem = 8.0 if op == "softmax" else 5.0
    elems_per_clk = arch.dram_bw * 1e9 / arch.sm_nums / arch.sm_clock_hz / (2 * type_size)
    warps = ctas * cfg.threads / 32
    issue_capacity = 4.0 * min(1.0, warps / 16.0) * 32
    issue = min(1.0, issue_capacity / (inst_per_elem * elems_per_clk * 2.2))

    if cfg.mode == "tma":
        grid_eff = 1.0
        coupling = 0.72  # per-row barrier round trips of the single persistent CTA (measured 0.78 - 0.88 of the best reg config)
        # a persistent CTA starts later (barriers, tensor maps, the first bulk copy's round trip): about
        # a microsecond more than a register-mode launch, which shows on problems that stream for only
        # a few microseconds (4096 x 2048: 0.91 of the best register config)
        t_stream = 2.0 * M * N * type_size / (arch.dram_bw * 1e9) + 3e-6
        coupling *= t_stream / (t_stream + 1e-6)
    else:
        slots = arch.sm_nums * rowwise_occupancy(cfg, arch, op, N)
        grid_eff = 1.0 if grid <= slots else grid / (math.ceil(grid / slots) * slots)
        if grid >= 4 * slots:
            # many small CTAs per SM drain unevenly anyway: the last partial wave costs a fraction of
            # what whole-wave arithmetic says (fitted to the 4096-row shapes of the sweep)
            grid_eff = 1.0 - 0.3 * (1.0 - grid_eff)
        coupling = 0.88 ** math.log2(cfg.rows_per_block) if cfg.threads > 128 else 1.0

    passes = 1.0
    if cfg.mode == "twopass":
        footprint = arch.sm_nums * ctas * cfg.rows_per_block * N * type_size
        hit = min(1.0, 0.6 * arch.l2_bytes / footprint) ** 2  # the rows in flight thrash L2 quickly once they outgrow it
        passes = 1.0 + 0.5 * (hit * arch.dram_bw / arch.l2_bw + (1.0 - hit))

    nw = cfg.threads_per_row // 32
    reduce = 1.0 / (1.0 + 0.02 * math.log2(nw or 1) + (0.03 if nw > 1 else 0.0))
    if cfg.mode == "twopass" and cfg.threads_per_row < 128:
        reduce *= 0.88  # a warp or two streaming a whole vocabulary row: measured 0.76 - 0.9 of 256 threads
    if cfg.mode == "cluster":
        # load, reduce, combine across the cluster, (exponentials, reduce, combine,) store: the phases
        # of a row serialise on cluster barriers at two or three resident CTAs per SM; measured
        # 3.0 - 3.8 TB/s on vocabulary rows where the two-pass mode streams at 4.2 - 5.1
        reduce *= 0.72 / (1.0 + 0.03 * math.log2(cfg.unroll))
    covered = chunks * cfg.threads_per_row * cfg.vec * (cfg.unroll if cfg.mode == "cluster" else 1)
    tail = N / covered if cfg.mode != "twopass" else 1.0
    lanes = 1.0 if cfg.vec * type_size >= 16 else 0.95
    # no-allocate loads and streaming stores: a hair better on problems that stream through L2, 2 - 12 %
    # worse on problems that fit in it
    # (16384 x 1024: 0.88; a tuning run times the same buffers over and over).  The two-pass mode gains
    # most: its second pass and its stores stream past the rows still to be re-read (+3 ... +11 %)
    if not cfg.hint:
        hint = 1.0
    elif cfg.mode == "twopass":
        hint = 1.05
    elif 2.0 * M * N * type_size <= arch.l2_bytes:
        hint = 0.92
    else:
        hint = 1.005
    # elements cached per thread (measured over the hidden-size grid, 12 configs per shape): 64 per
    # thread (eight 16-byte chunks) are best, 32 lose 5 - 13 %, fewer more, 128 lose about 30 % (the
    # row no longer overlaps its own loads with its reduction)
    depth = 1.0
    if cfg.mode in ("reg", "cluster"):
        per_thread_elems = chunks * cfg.vec
        if cfg.mode == "reg" and cfg.threads >= 512:
            # one or two 512- / 1024-thread CTAs per SM: the whole SM waits in the same phase
            # (32000 columns: 0.70 - 0.80 of the two-pass mode)
            phase *= 0.78
        depth = (0.8 if per_thread_elems <= 8 else 0.86 if per_thread_elems <= 16 else 0.93 if per_thread_elems <= 32
                 else 0.97 if per_thread_elems < 56 else 1.0 if per_thread_elems <= 64 else 0.85 if per_thread_elems <= 96 else 0.7)
    # a CTA costs the SM a fixed slice of time to start and retire, which shows when it moves only a
    # couple of kilobytes (16384 x 1024: CTAs of two or four 2 KB rows are 7.7 % faster than of one)
    small = 1.0
    if cfg.mode in ("reg", "twopass") and 2.0 * M * N * type_size <= arch.l2_bytes:  # seen on L2-resident problems only
        cta_bytes = cfg.rows_per_block * N * type_size
        small = cta_bytes / (cta_bytes + 320.0)
    return {"small": small, "mem": mem, "phase": phase, "issue": issue, "grid": grid_eff, "coupling": coupling, "reduce": reduce,
            "tail": 0.7 + 0.3 * tail, "lanes": lanes, "hint": hint, "depth": depth, "passes": 1.0 / passes}


def rowwise_score(cfg, arch: Arch, op: str, M: int, N: int, type_size: int = 2) -> float:
    """Heuristic score of a memory-bound row-wise config: the product of ``rowwise_terms``."""
    return math.prod(rowwise_terms(cfg, arch, op, M, N, type_size).values())


def rank_rowwise_configs(configs, arch: Arch, op: str, M: int, N: int, top_n: int | None = None):
    """Sort row-wise configs by ``rowwise_score`` (best first)."""
    ranked = sorted(configs, key=lambda c: rowwise_score(c, arch, op, M, N), reverse=True)
    return ranked[:top_n] if top_n else ranked
