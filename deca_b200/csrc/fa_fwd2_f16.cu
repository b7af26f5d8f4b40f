// FlashAttention forward for B200, two Q tiles per CTA (FAConfig q_tiles = 2).
//
// Same arithmetic as fa_fwd_f16.cu; what changes is the schedule.  A CTA owns two consecutive
// 128-row Q tiles of one head (group A = even tile, group B = odd tile) and 320 threads:
//   warp 0      TMA producer: both Q tiles once, then K_0, V_0, K_1, V_1, ... through ONE ring of
//               `stages` slots; every K / V tile is loaded once and used by both groups.
//   warp 1      MMA issuer.  Tensor memory holds S_A, S_B (128 columns each) and O_A, O_B (D columns
//               each).  Issue order per KV step j: when P_A(j) is ready, S_A(j+1) = Q_A K_{j+1}^T
//               then O_A += P_A(j) V_j; then the same for B.  The MMAs of one group run while the
//               other group is in its softmax.
//   warps 2-5   softmax + epilogue of group A, warps 6-9 of group B: one thread per query row, two
//               softmax warps per scheduler.
// With 64-key tiles (BC = 64, P in tensor memory) every group owns TWO score buffers, so the
// scores of step j+1 are computed while the softmax of step j runs and a group never waits for
// the tensor pipe; with 128-key tiles tensor memory only has room for one buffer per group.
// Causal: each group visits the KV tiles up to its own diagonal and masks the tiles that cross it;
// group A stops 128 keys earlier; pairs are scheduled longest first.
// All mbarrier waits are bounded (ptx.cuh); a wait that runs out raises the CTA's abort flag and
// every role falls through to the common teardown.
#include <atomic>
#include <type_traits>

#include "fa_softmax.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace deca {
namespace {

constexpr int kBr = 128;
constexpr int kThreads2 = 320;

struct Fa2Args {
    int S_q, S_kv;
    int causal;
    int stages;  // K/V ring slots
    float sl2;
    int n_peers;  // every output panel is also stored through peers.m[0 .. n_peers)
    DeviceStatus *status;
};

// PTMEM: P lives in tensor memory (aliasing the first 64 columns of its score tile) and is the
// A operand of the P V product, so neither the P write nor the P read touches shared memory and
// the K/V ring gets the space; the product of step j must then be issued BEFORE the next score
// MMA of the same group overwrites that tile.
template <int D, int BC, bool PTMEM>
__global__ void __launch_bounds__(kThreads2, 1)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
               const __grid_constant__ PeerMaps peers, const Fa2Args g) {
    using P16 = Pack16<DECA_F16>;
    constexpr int kBc = BC;
    constexpr int NSB = (BC == 64) ? 2 : 1;  // score buffers per group
    static_assert(BC == 128 || PTMEM, "64-key tiles keep P in tensor memory");
    constexpr uint32_t kQBytes = kBr * D * 2;
    constexpr uint32_t kKVBytes = kBc * D * 2;
    constexpr uint32_t kPBytes = kBr * kBc * 2;
    constexpr uint32_t kKVBlock = kBc * 128;
    constexpr uint32_t kIdescQK = make_idesc_f16(DECA_F16, false, false, kBr, kBc);
    constexpr uint32_t kIdescPV = make_idesc_f16(DECA_F16, false, true, kBr, D);
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw);

    const int stages = g.stages;
    const uint32_t sQ = base;                   // Q_A, Q_B
    const uint32_t sP = sQ + 2 * kQBytes;       // P_A, P_B (unless P is in tensor memory)
    const uint32_t sKV = sP + (PTMEM ? 0u : 2 * kPBytes);  // ring
    const uint32_t sBar = sKV + stages * kKVBytes;
    const uint32_t q_full = sBar;
    auto kv_full = [&](int i) { return sBar + 8u * (1 + i); };
    auto kv_empty = [&](int i) { return sBar + 8u * (1 + stages + i); };
    const uint32_t fixed0 = sBar + 8u * (1 + 2 * stages);
    auto s_full = [&](int grp, int buf) { return fixed0 + 8u * (grp * 2 + buf); };
    // one "P ready" barrier per score buffer: with two buffers a group may finish two tiles before
    // the MMA warp looks, and a single barrier would then have gone through two phases
    auto p_full = [&](int grp, int buf) { return fixed0 + 8u * (4 + grp * 2 + buf); };
    // likewise one "product done" barrier per score buffer: tile j uses buffer j % NSB, and the
    // product of tile j - NSB is always complete before the softmax of tile j starts, so a wait on
    // the buffer's barrier can only be one phase behind
    auto pv_done = [&](int grp, int buf) { return fixed0 + 8u * (8 + grp * 2 + buf); };
    const uint32_t drain_bar = fixed0 + 8u * 12;
    const uint32_t slot_addr = fixed0 + 8u * 13;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + (slot_addr - base));
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int n_pairs = g.S_q / (2 * kBr);
    const int pair = g.causal ? (n_pairs - 1 - (int)blockIdx.x) : (int)blockIdx.x;
    const int bh = blockIdx.y;
    const int q_row0 = bh * g.S_q + pair * 2 * kBr;  // first row of tile A in the [B*H*S_q, D] view
    const int kv_row0 = bh * g.S_kv;
    // KV tiles visited by group A / B (B always visits at least as many as A)
    const int n_a = g.causal ? ((2 * pair + 1) * kBr + kBc - 1) / kBc : g.S_kv / kBc;
    const int n_b = g.causal ? ((2 * pair + 2) * kBr + kBc - 1) / kBc : g.S_kv / kBc;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        for (int i = 0; i < stages; ++i) {
            mbar_init(kv_full(i), 1);
            mbar_init(kv_empty(i), 1);
        }
        for (int grp = 0; grp < 2; ++grp) {
            mbar_init(s_full(grp, 0), 1);
            mbar_init(s_full(grp, 1), 1);
            mbar_init(p_full(grp, 0), 4);
            mbar_init(p_full(grp, 1), 4);
            mbar_init(pv_done(grp, 0), 1);
            mbar_init(pv_done(grp, 1), 1);
        }
        mbar_init(drain_bar, 1);
        fence_barrier_init();
        // This thread is also the TMA producer: the Q tiles are requested here, before the CTA's
        // set-up barrier, so that their latency overlaps the tensor-memory allocation.
        mbar_arrive_expect_tx(q_full, 2 * kQBytes);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int blk = 0; blk < D / 64; ++blk)
                tma_load_2d(sQ + t * kQBytes + blk * 16384, &tmQ, blk * 64, q_row0 + t * kBr, q_full);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
        prefetch_tensormap(&tmO);
    }
    if (warp == 1) {
        tmem_alloc(slot_addr, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    auto tS = [&](int grp, int buf) { return tmem_base + (uint32_t)((grp * NSB + buf) * kBc); };
    auto tO = [&](int grp) { return tmem_base + 2u * NSB * kBc + (uint32_t)(grp * D); };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            int n_items = 0;
            for (int i = 0; i < 2 * n_b; ++i) {  // item 2j = K_j, 2j + 1 = V_j
                if (!mbar_wait(kv_empty(s), ph ^ 1u, abort_flag)) {
                    report_detail(g.status, 0, 1, i);
                    ok = false;
                    break;
                }
                const int row = kv_row0 + (i >> 1) * kBc;
                const CUtensorMap *tm = (i & 1) ? &tmV : &tmK;
                mbar_arrive_expect_tx(kv_full(s), kKVBytes);
#pragma unroll
                for (int blk = 0; blk < D / 64; ++blk)
                    tma_load_2d(sKV + s * kKVBytes + blk * kKVBlock, tm, blk * 64, row, kv_full(s));
                ++n_items;
                if (++s == stages) s = 0, ph ^= 1u;
            }
            if (!ok) {
                if (*abort_flag == 0) {
                    *abort_flag = 1;
                    report_timeout(g.status, 0x401u);
                }
                __shared__ uint32_t no_abort;
                no_abort = 0;
                (void)mbar_wait(q_full, 0, &no_abort);
                for (int st = 0; st < stages; ++st) {
                    const int n_st = (n_items + stages - 1 - st) / stages;
                    if (n_st > 0) (void)mbar_wait(kv_full(st), (uint32_t)((n_st - 1) & 1), &no_abort);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = true;
            // One thread issues every MMA of the CTA, so its instruction stream is on the critical
            // path: descriptors are a constant upper word plus (address >> 4), the per-step offsets
            // are compile-time constants, and ring positions advance incrementally (no division).
            constexpr uint64_t kDescK = (uint64_t(16 >> 4) << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
            constexpr uint64_t kDescV = (uint64_t((kKVBlock >> 4) & 0x3FFF) << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
            const uint64_t q_desc[2] = {kDescK | (uint64_t)((sQ & 0x3FFFFu) >> 4),
                                        kDescK | (uint64_t)(((sQ + kQBytes) & 0x3FFFFu) >> 4)};
            const uint64_t p_desc[2] = {kDescK | (uint64_t)((sP & 0x3FFFFu) >> 4),
                                        kDescK | (uint64_t)(((sP + kPBytes) & 0x3FFFFu) >> 4)};
            struct RingPos {
                int slot;
                uint32_t par;
            };
            auto advance2 = [&](RingPos &p) {  // two items further (K_t -> K_{t+1}, V_j -> V_{j+1})
                p.slot += 2;
                if (p.slot >= stages) p.slot -= stages, p.par ^= 1u;
            };
            auto issue_qk = [&](int grp, int buf, const RingPos &kp) {  // S_grp[buf] = Q_grp K^T
                const uint64_t kdesc = kDescK | (uint64_t)(((sKV + kp.slot * kKVBytes) & 0x3FFFFu) >> 4);
                const uint32_t d_tmem = tS(grp, buf);
#pragma unroll
                for (int kd = 0; kd < D / 16; ++kd) {
                    umma_f16_ss(d_tmem, q_desc[grp] + (((kd / 4) * 16384 + (kd % 4) * 32) >> 4),
                                kdesc + (((kd / 4) * kKVBlock + (kd % 4) * 32) >> 4), kIdescQK, kd != 0 ? 1u : 0u);
                }
                umma_commit(s_full(grp, buf));
            };
            auto issue_pv = [&](int grp, int buf, const RingPos &vp, uint32_t first) {  // O_grp (+)= P_grp V
                const uint64_t vdesc = kDescV | (uint64_t)(((sKV + vp.slot * kKVBytes) & 0x3FFFFu) >> 4);
                const uint32_t d_tmem = tO(grp);
                const uint32_t a_tmem = tS(grp, buf);
#pragma unroll
                for (int kk = 0; kk < kBc / 16; ++kk) {
                    if constexpr (PTMEM) {
                        // 16 keys = 8 packed columns of the P tile in tensor memory
                        umma_f16_ts(d_tmem, a_tmem + kk * 8, vdesc + kk * (2048 >> 4), kIdescPV, (first | kk) != 0 ? 1u : 0u);
                    } else {
                        umma_f16_ss(d_tmem, p_desc[grp] + (((kk / 4) * 16384 + (kk % 4) * 32) >> 4),
                                    vdesc + kk * (2048 >> 4), kIdescPV, (first | kk) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(pv_done(grp, buf));
            };
            // ring positions: kp = K tile whose scores are issued next, vp = V_j
            RingPos kp{0, 0u}, vp{1 % stages, (uint32_t)((1 / stages) & 1)};
            // prologue: fill every score buffer (tiles 0 .. NSB-1 of both groups)
            ok = mbar_wait(q_full, 0, abort_flag);
            for (int t = 0; t < NSB && t < n_b && ok; ++t) {
                if (!mbar_wait(kv_full(kp.slot), kp.par, abort_flag)) {
                    report_detail(g.status, 1, 2, t);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if (t < n_a) issue_qk(0, t % NSB, kp);
                issue_qk(1, t % NSB, kp);
                umma_commit(kv_empty(kp.slot));
                advance2(kp);
            }
            int buf = 0;
            uint32_t p_par = 0;
            for (int j = 0; j < n_b && ok; ++j) {
                const int jn = j + NSB;  // tile whose scores are issued in this step (its K is at kp)
                // V_j and K_jn (if any) must have landed
                if (!mbar_wait(kv_full(vp.slot), vp.par, abort_flag)) {
                    report_detail(g.status, 1, 4, j);
                    ok = false;
                }
                if (ok && jn < n_b && !mbar_wait(kv_full(kp.slot), kp.par, abort_flag)) {
                    report_detail(g.status, 1, 3, j);
                    ok = false;
                }
                if (!ok) break;
                // group A: once P_A(j) is ready its score buffer is consumed as well
                if (j < n_a) {
                    if (!mbar_wait(p_full(0, buf), p_par, abort_flag)) {
                        report_detail(g.status, 1, 5, j);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    if constexpr (PTMEM) {
                        // the product reads P from the buffer the next score MMA overwrites
                        issue_pv(0, buf, vp, (uint32_t)j);
                        if (jn < n_a) issue_qk(0, buf, kp);
                    } else {
                        if (jn < n_a) issue_qk(0, buf, kp);
                        issue_pv(0, buf, vp, (uint32_t)j);
                    }
                }
                // group B (always the last user of K_jn and V_j)
                if (!mbar_wait(p_full(1, buf), p_par, abort_flag)) {
                    report_detail(g.status, 1, 6, j);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                if constexpr (PTMEM) {
                    issue_pv(1, buf, vp, (uint32_t)j);
                    umma_commit(kv_empty(vp.slot));
                    if (jn < n_b) {
                        issue_qk(1, buf, kp);
                        umma_commit(kv_empty(kp.slot));
                    }
                } else {
                    if (jn < n_b) {
                        issue_qk(1, buf, kp);
                        umma_commit(kv_empty(kp.slot));
                    }
                    issue_pv(1, buf, vp, (uint32_t)j);
                    umma_commit(kv_empty(vp.slot));
                }
                advance2(vp);
                if (jn < n_b) advance2(kp);
                if (++buf == NSB) buf = 0, p_par ^= 1u;
            }
            if (!ok) {
                if (*abort_flag == 0) {
                    *abort_flag = 1;
                    report_timeout(g.status, 0x402u);
                }
                __shared__ uint32_t no_abort2;
                no_abort2 = 0;
                umma_commit(drain_bar);
                (void)mbar_wait(drain_bar, 0, &no_abort2);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        const int grp = (warp - 2) >> 2;  // 0 = tile A, 1 = tile B
        const int q = warp & 3;           // tensor-memory lane quarter
        const int r = q * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const int qt = 2 * pair + grp;
        const int row_abs = qt * kBr + r;
        const int n_kv = grp == 0 ? n_a : n_b;
        const uint32_t tOg = tO(grp) + lane_off;
        const float sl2 = g.sl2;
        float m = kNegInf, l = 0.f;
        bool ok = true;
        auto wait_all = [&](uint32_t bar, uint32_t parity) {
            return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag)) != 0;
        };

        for (int j = 0; j < n_kv; ++j) {
            const int buf = j % NSB;
            if (!wait_all(s_full(grp, buf), (uint32_t)((j / NSB) & 1))) {
                if (lane == 0 && q == 0) report_detail(g.status, 2 + grp, 7, j);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t tSg = tS(grp, buf) + lane_off;
            const uint32_t pb = PTMEM ? tSg : sP + grp * kPBytes;
            const bool diag = g.causal && ((j + 1) * kBc - 1 > qt * kBr);
            const int col0 = j * kBc;

            // P (single buffer per group) was last read by the product of tile j - 1, which is also
            // the product that completes O for a rescale
            auto wait_prev = [&]() {
                return j == 0 || wait_all(pv_done(grp, (j - 1) % NSB), (uint32_t)(((j - 1) / NSB) & 1));
            };
            // P in tensor memory reuses the score buffer that was just filled: free by construction
            auto wait_p = [&]() { return PTMEM || wait_prev(); };
            const bool step_ok = diag ? fa_softmax_step<kBc, D, true, PTMEM>(tSg, tOg, pb, r, col0, row_abs, sl2, j == 0,
                                                                             m, l, wait_p, wait_prev)
                                      : fa_softmax_step<kBc, D, false, PTMEM>(tSg, tOg, pb, r, col0, row_abs, sl2, j == 0,
                                                                              m, l, wait_p, wait_prev);
            if (!step_ok) {
                if (lane == 0 && q == 0) report_detail(g.status, 2 + grp, 8, j);
                ok = false;
                break;
            }
            // S is consumed, P (and a possibly rescaled O) are ready
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(grp, buf));
        }

        if (ok) {
            ok = wait_all(pv_done(grp, (n_kv - 1) % NSB), (uint32_t)(((n_kv - 1) / NSB) & 1));
            if (!ok && lane == 0 && q == 0) report_detail(g.status, 2 + grp, 9, n_kv);
        }
        if (!ok) {
            if (lane == 0 && *abort_flag == 0) {
                *abort_flag = 1;
                report_timeout(g.status, 0x403u);
            }
        } else {
            // ---- epilogue: O / l -> fp16 -> shared (this group's Q tile space) -> TMA store
            tc_fence_after_sync();
            const float inv = 1.0f / l;
            const uint32_t stage0 = sQ + grp * kQBytes;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tOg + c * 32, v);
                tmem_ld_wait();
                const uint32_t rowb = stage0 + (c / 2) * 16384 + q * 4096 + lane * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const int chunk = (c & 1) * 4 + cc;
                    const uint32_t dst = rowb + ((chunk ^ (lane & 7)) << 4);
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        o[i] = P16::pack(__uint_as_float(v[cc * 8 + 2 * i]) * inv,
                                         __uint_as_float(v[cc * 8 + 2 * i + 1]) * inv);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                                 "r"(o[3])
                                 : "memory");
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int blk = 0; blk < D / 64; ++blk)
                    tma_store_2d(&tmO, stage0 + blk * 16384 + q * 4096, blk * 64, q_row0 + grp * kBr + q * 32);
                // gather: the same rows of O go to the other ranks' copies (plain TMA stores to peer memory)
                for (int pr = 0; pr < g.n_peers; ++pr)
#pragma unroll
                    for (int blk = 0; blk < D / 64; ++blk)
                        tma_store_2d(&peers.m[pr], stage0 + blk * 16384 + q * 4096, blk * 64, q_row0 + grp * kBr + q * 32);
                tma_store_commit();
                // the CTA may leave once its stores have read shared memory (the writes complete with
                // the grid); stores to peers are waited for in full
                if (g.n_peers > 0)
                    tma_store_wait<0>();
                else
                    tma_store_wait_read<0>();
            }
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int D, int BC, bool PTMEM>
int launch_fa2(const CUtensorMap &tmQ, const CUtensorMap &tmK, const CUtensorMap &tmV, const CUtensorMap &tmO,
               const PeerMaps &peers,
               const Fa2Args &g, dim3 grid, size_t smem, cudaStream_t st) {
    static SmemLimitCache configured;
    if (int rc = ensure_dynamic_smem(fa_fwd2_kernel<D, BC, PTMEM>, smem, configured)) return rc;
    fa_fwd2_kernel<D, BC, PTMEM><<<grid, kThreads2, smem, st>>>(tmQ, tmK, tmV, tmO, peers, g);
    return (int)cudaGetLastError();
}

}  // namespace

size_t fa2_smem_bytes(int D, int BC, int stages, bool ptmem) {
    return 1024 + 2 * (size_t)kBr * D * 2 + (ptmem ? 0 : 2 * (size_t)kBr * BC * 2) + (size_t)stages * BC * D * 2 +
           8 * (2 * (size_t)stages + 20);
}

// Host rules of the two-tile schedule; shared with deca_fa_fwd_f16_check_config.
int fa2_check(int S_q, int S_kv, int D, const deca_fa_cfg &c) {
    if (c.Br != kBr || (c.Bc != 128 && c.Bc != 64)) return DECA_ERR_CONFIG;
    if (c.Bc == 64 && !c.p_tmem) return DECA_ERR_CONFIG;  // 64-key tiles keep P in tensor memory
    if (S_q % (2 * kBr) != 0 || S_kv % c.Bc != 0) return DECA_ERR_CONFIG;
    // 64-key tiles keep two score tiles per group in flight: K_{j+2} and V_j live together
    if (c.stages < (c.Bc == 64 ? 4 : 2) || c.stages > 8) return DECA_ERR_CONFIG;
    if (fa2_smem_bytes(D, c.Bc, c.stages, c.p_tmem != 0) > 232448) return DECA_ERR_CONFIG;
    return DECA_OK;
}

int fa2_launch(const CUtensorMap &tmQ, const CUtensorMap &tmK, const CUtensorMap &tmV, const CUtensorMap &tmO,
               const PeerMaps &peers, int n_peers, int B, int H, int S_q, int S_kv, int D, float softmax_scale, int causal,
               const deca_fa_cfg &c, cudaStream_t st) {
    Fa2Args g;
    g.n_peers = n_peers;
    g.S_q = S_q, g.S_kv = S_kv;
    g.causal = causal ? 1 : 0;
    g.stages = c.stages;
    g.sl2 = softmax_scale * kLog2e;
    g.status = device_status_ptr();
    if (!g.status) return (int)cudaErrorUnknown;
    const dim3 grid((unsigned)(S_q / (2 * kBr)), (unsigned)(B * H), 1);
    const bool ptmem = c.p_tmem != 0;
    const size_t smem = fa2_smem_bytes(D, c.Bc, c.stages, ptmem);
    if (c.Bc == 64)
        return D == 128 ? launch_fa2<128, 64, true>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st)
                        : launch_fa2<64, 64, true>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st);
    if (ptmem)
        return D == 128 ? launch_fa2<128, 128, true>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st)
                        : launch_fa2<64, 128, true>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st);
    return D == 128 ? launch_fa2<128, 128, false>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st)
                    : launch_fa2<64, 128, false>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st);
}

}  // namespace deca
