"""Z3 enumeration of kernel configurations for B200.

Same entry points and calling convention as the hot functions of the reference's
src/Solver.py -- ``solve_gemm_tc`` (:473-559), ``solve_flash_attn`` (:304-386),
``solve_rowwise`` (:389-470): the arch object comes first, the result is a list of frozen
config dataclasses, every solution satisfies the kernel module's ``check_config``.  The
variables are those of the tcgen05 / TMA kernels (CTA tile = MMA tile, TMA ring depth,
tensor-memory accumulator buffers, bulk-copy row pipelines) instead of warp tiles and
cp.async stages.  Importing this module does not touch the GPU (the reference creates a GPU
instance at import, Solver.py:10).
"""

from __future__ import annotations

from z3 import And, BitVecs, BitVecVal, If, Implies, Or, Solver, UDiv, UGE, ULE, URem, sat


def _all_models(s: Solver, variables, count: int):
    """All-SAT by blocking clauses (the enumeration scheme of the reference)."""
    out = []
    while len(out) < count and s.check() == sat:
        m = s.model()
        vals = [m[x].as_long() for x in variables]
        out.append(vals)
        s.add(Or([x != v for x, v in zip(variables, vals)]))
    return out


def solve_gemm_tc(arch, M: int, N: int, K: int, type_size: int = 2, count: int = 4096, acc_f16: bool = False,
                  acc_splits: int = 1):
    """Enumerates 16-bit tensor-core GEMM tile configurations (see ``GemmConfig``).

    arch supplies ``max_dyn_smem_per_block``, ``tmem_columns`` and ``sm_nums``.  ``acc_f16`` asks
    for configs with fp16 accumulators (one-CTA tiles, no stream-K: an fp16 accumulator takes the
    same tensor-memory columns as an fp32 one, so the tile space is otherwise the same);
    ``acc_splits`` is accepted for call-site compatibility (the accumulator is a single one).
    """
    from .kernels.gemm_b200 import SMEM_RESERVED, GemmConfig, check_config, stream_k_plan

    s = Solver()
    bm, bn, st, epi, acc = BitVecs("bm bn st epi acc", 32)
    k_ = BitVecVal(K, 32)

    s.add(Or(bm == 128, bm == 256))
    s.add(Or(bn == 64, bn == 128, bn == 256))
    s.add(Implies(bm == 256, UGE(bn, 128)))
    s.add(And(UGE(st, 2), ULE(st, 8)))
    s.add(ULE(epi, 1))
    s.add(Or(acc == 1, acc == 2))
    # do not pipeline deeper than the number of 64-deep K blocks (at least 2 slots)
    kb = UDiv(k_ + 63, 64)
    s.add(Or(ULE(st, kb), st == 2))
    # tensor memory: acc_bufs accumulators of (BM / 128) * BN fp32 columns
    s.add(ULE(acc * UDiv(bm, 128) * bn, getattr(arch, "tmem_columns", 512)))
    # shared memory: ring of A and B tiles, epilogue staging, barriers
    smem = st * (bm * 64 + 64 * bn) * type_size + If(epi == 1, BitVecVal(32768, 32), BitVecVal(0, 32)) + SMEM_RESERVED
    s.add(ULE(smem, arch.max_dyn_smem_per_block))
    # a tile at least twice as wide as the problem only wastes MMA columns
    s.add(Or(ULE(bn, BitVecVal(max(2 * N - 1, 64), 32)), bn == 64))

    results = []
    gm_of = {128: -(-M // 128), 256: -(-M // 256)}
    for vals in _all_models(s, (bm, bn, st, epi, acc), count):
        gn = -(-N // vals[1])
        # tile order: groups of `ras` tile rows walked along N, or (tall problems) of `ras` tile columns
        # walked down M, which keeps a band of the smaller operand B in L2
        orders = [(ras, False) for ras in (1, 2, 4, 8, 16) if ras == 1 or ras <= gm_of[vals[0]]]
        if M > N:
            orders += [(ras, True) for ras in (2, 4, 8, 16) if ras <= gn]
        for ras, along_n in orders:
            cfg = GemmConfig(BM=vals[0], BN=vals[1], BK=64, stages=vals[2], raster=ras, epi_smem=bool(vals[3]),
                             cta_group=1, acc_bufs=vals[4], acc_f16=acc_f16, raster_n=along_n)
            try:
                check_config(cfg, M, N, K)
            except AssertionError:
                continue
            results.append(cfg)
            if along_n:
                continue
            # the stream-K form of the config, where whole tiles would leave a quarter of a wave idle
            tiles = gm_of[vals[0]] * -(-N // vals[1])
            sms = arch.sm_nums
            if not acc_f16 and ras == 8 and cfg.epi_smem and tiles / (-(-tiles // sms) * sms) < 0.75:
                sk = GemmConfig(**{**cfg.as_dict(), "stream_k": True})
                if stream_k_plan(sk, M, N, K, sms) is not None:
                    results.append(sk)
    # CTA pairs (tcgen05 cta_group::2): (2 BM) x BN tiles whose CTAs fetch half of the B columns each
    for bm_, bn_, acc_ in ((256, 256, 1), (128, 256, 2), (128, 256, 1), (256, 128, 2), (128, 128, 2)):
        if acc_f16:
            break
        if -(-M // (2 * bm_)) * -(-N // bn_) < 8 or bn_ > max(2 * N - 1, 128):
            continue
        for st in (3, 4, 6, 8):
            for ras in (1, 2, 4, 8, 16):
                if ras > 1 and ras > -(-M // (2 * bm_)):
                    continue
                cfg = GemmConfig(BM=bm_, BN=bn_, BK=64, stages=st, raster=ras, epi_smem=True, cta_group=2, acc_bufs=acc_)
                try:
                    check_config(cfg, M, N, K)
                except AssertionError:
                    continue
                results.append(cfg)
    return results[:count]


def solve_flash_attn(arch, B: int, H: int, S_q: int, S_kv: int, D: int, type_size: int = 2, max_est_regs: int = 320,
                     count: int = 256):
    """Enumerates FlashAttention forward configurations (see ``FAConfig``)."""
    from .kernels.flash_attn_b200 import FAConfig, check_config

    s = Solver()
    bc, st, qt, pt = BitVecs("bc st qt pt", 32)
    s.add(Or(bc == 64, bc == 128))
    s.add(Or(qt == 1, qt == 2))
    s.add(ULE(pt, 1))
    s.add(URem(BitVecVal(S_kv, 32), bc) == 0)
    s.add(URem(BitVecVal(S_q, 32), 128 * qt) == 0)
    n_kv = UDiv(BitVecVal(S_kv, 32), bc)
    # one Q tile per CTA: a K ring and a V ring of `st` slots, double-buffered P, two score buffers
    smem1 = (128 * D + 2 * st * bc * D + If(pt == 1, BitVecVal(0, 32), BitVecVal(2 * 128, 32) * bc)) * type_size + 2048
    s.add(Implies(qt == 1, And(UGE(st, 1), ULE(st, 4), ULE(st, n_kv), ULE(smem1, arch.max_dyn_smem_per_block),
                               ULE(2 * bc + D, getattr(arch, "tmem_columns", 512)))))
    # two Q tiles per CTA: one ring of `st` slots shared by K and V tiles, one P and one score buffer per tile
    smem2 = (2 * 128 * D + st * bc * D + If(pt == 1, BitVecVal(0, 32), BitVecVal(2 * 128, 32) * bc)) * type_size + 2048
    s.add(Implies(qt == 2, And(Or(bc == 128, pt == 1), UGE(st, If(bc == 64, BitVecVal(4, 32), BitVecVal(2, 32))),
                               ULE(st, 8), ULE(st, 2 * n_kv), ULE(smem2, arch.max_dyn_smem_per_block),
                               BitVecVal(int(256 + 2 * D <= getattr(arch, "tmem_columns", 512)), 32) == 1)))

    results = []
    for vals in _all_models(s, (bc, st, qt, pt), count):
        cfg = FAConfig(Br=128, Bc=vals[0], stages=vals[1], q_tiles=vals[2], p_tmem=bool(vals[3]))
        try:
            check_config(cfg, S_q, S_kv, D)
        except AssertionError:
            continue
        results.append(cfg)
        # the persistent form of the two-tile schedule (its O staging panels take 32 KB of the ring's space)
        if cfg.q_tiles == 2 and cfg.Bc == 128 and cfg.p_tmem:
            pers = FAConfig(**{**cfg.as_dict(), "persistent": True})
            try:
                check_config(pers, S_q, S_kv, D)
            except AssertionError:
                continue
            results.append(pers)
    return results


def solve_rowwise(arch, op: str, M: int, N: int, type_size: int = 2, twopass_min_n: int = 16384, count: int = 1024):
    """Enumerates row-wise (softmax / RMSNorm) configurations (see ``RowConfig``).

    Modes: 0 = reg (row in registers), 1 = twopass (row streamed twice), 2 = tma (persistent
    CTAs, rows through shared-memory rings with bulk copies).  As in the reference, twopass is
    only offered for rows of at least ``twopass_min_n`` elements unless nothing else fits.  Rows of
    that length also get the cluster mode (a thread-block cluster of 2, 4 or 8 CTAs per row, each
    caching a slice in registers: one pass where twopass needs two), enumerated directly.
    """
    from .kernels.rowwise_b200 import RowConfig, check_config

    s = Solver()
    tpr, rpb, vec, mode, unroll, hint = BitVecs("tpr rpb vec mode unroll hint", 32)
    n = BitVecVal(N, 32)
    s.add(Or([tpr == v for v in (32, 64, 128, 256, 512, 1024)]))
    s.add(Or([rpb == v for v in (1, 2, 3, 4, 8, 15, 16)]))
    s.add(Or(vec == 4, vec == 8) if N % 4 == 0 else vec == 2)  # 4-byte accesses only for rows that need them
    s.add(ULE(mode, 2))
    s.add(Or(unroll == 1, unroll == 2, unroll == 3, unroll == 4))
    s.add(ULE(hint, 1))
    s.add(URem(n, vec) == 0)
    threads = tpr * rpb
    s.add(ULE(threads, 1024))
    # a row must keep every vector lane of its threads busy at least once
    s.add(Or(ULE(tpr * vec, n), tpr == 32))
    # reg / twopass: one CTA per rows_per_block rows, enough CTAs to fill the SMs, >= 64 threads
    s.add(Implies(mode != 2, And(URem(BitVecVal(M, 32), rpb) == 0, Or(rpb == 1, rpb == 2, rpb == 4, rpb == 8, rpb == 16),
                                 Or(UGE(threads, 64), rpb == 1))))
    s.add(Implies(And(mode != 2, BitVecVal(int(M >= arch.sm_nums), 32) == 1),
                  UGE(UDiv(BitVecVal(M, 32), rpb), arch.sm_nums)))
    s.add(Implies(mode == 0, unroll == 1))
    s.add(Implies(mode == 1, And(Or(unroll == 1, unroll == 2, unroll == 4), ULE(unroll * tpr * vec, n))))
    # tma: power-of-two groups of at most 512 threads per CTA, 16-byte accesses, no hint knob
    s.add(Implies(mode == 2, And(vec == 8, ULE(threads, 512), ULE(rpb, 15), hint == 0, UGE(rpb * unroll, 2))))

    only_short = N < twopass_min_n
    results, fallback = [], []
    for vals in _all_models(s, (tpr, rpb, vec, mode, unroll, hint), 8 * count):
        cfg = RowConfig(threads_per_row=vals[0], rows_per_block=vals[1], vec=vals[2],
                        mode=("reg", "twopass", "tma")[vals[3]], unroll=vals[4], hint=bool(vals[5]))
        try:
            check_config(cfg, op, M, N, "float16")
        except AssertionError:
            continue
        (fallback if (cfg.mode == "twopass" and only_short) else results).append(cfg)
    if not results:
        results = fallback
    results = results[:count]
    if N >= twopass_min_n:
        for cs in (2, 4, 8):
            for threads in (256, 512, 1024):
                for v in ((8, 4) if N % 8 == 0 else (4,) if N % 4 == 0 else (2,)):
                    for h in (False, True):
                        cfg = RowConfig(threads_per_row=threads, rows_per_block=1, vec=v, mode="cluster", unroll=cs, hint=h)
                        try:
                            check_config(cfg, op, M, N, "float16")
                        except AssertionError:
                            continue
                        results.append(cfg)
    return results
