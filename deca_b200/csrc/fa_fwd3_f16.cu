// FlashAttention forward for B200, persistent form of the two-Q-tile schedule (FAConfig
// q_tiles = 2, persistent = 1; 128-key tiles, P in tensor memory).
//
// Same arithmetic and the same roles as fa_fwd2_f16.cu; what changes is that a CTA does not end
// with its pair of Q tiles.  The grid is one CTA per SM and CTA c works through the items
// c, c + grid, c + 2 grid, ... of the list of (head, Q-tile pair) items in launch order (pairs of
// one head adjacent; causal: longest pair first).  Barriers, the K/V ring and tensor memory
// persist, every role carries its own phase counters across items, and the start of item i + 1
// overlaps the end of item i:
//   * K / V tiles of the next item enter the ring as its slots free up;
//   * the next Q pair is loaded as soon as the last score MMA of the current item has completed
//     (tcgen05.commit on `q_free`), because O is staged for its TMA stores in a buffer of its own
//     (4 KB per softmax warp, 64 columns at a time) instead of the Q tiles;
//   * the score MMAs of the next item's first tile are issued while the softmax warps are still in
//     the epilogue of the current one.  The first product of the next item overwrites the O
//     accumulator; it is issued after that item's first P is published, which the same warps do
//     after their epilogue, so no extra barrier guards O.
// The thread that issues the MMAs is the serial resource of the schedule: its MMAs issue at the
// rate they execute, and every mbarrier wait it makes is a dependent round trip of 100 - 200
// clocks even when the phase has long completed.  So it waits for as little as it can:
//   * a relay warp waits for the K / V tiles of a step (which land a whole step ahead) and then
//     arrives on the same barriers as the softmax warps that publish P, so one wait per Q tile and
//     step tells the issuer that P, V_j and K_{j+1} are all there;
//   * a product is committed to a barrier of its own only at the end of an item: within an item
//     the completion of the next score tile (issued behind the product) already implies it.
// All mbarrier waits are bounded (ptx.cuh); a wait that runs out raises the CTA's abort flag and
// every role falls through to the common teardown.
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "fa_softmax.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace deca {
namespace {

constexpr int kBr = 128;
constexpr int kBc = 128;
constexpr int kThreads3 = 352;  // TMA producer, MMA issuer, 2 x 4 softmax warps, relay
constexpr uint32_t kOStageBytes = 8 * 4096;  // one 32 x 64 fp16 panel per softmax warp

struct Fa3Args {
    int S_q, S_kv;
    int causal;
    int stages;  // K/V ring slots
    float sl2;
    int n_peers;
    int n_pairs;    // Q-tile pairs per head
    int n_heads;    // B * H
    int sec_heads;  // causal: heads per section (their K and V together fit in half of L2)
    DeviceStatus *status;
};

struct RingPos {
    int slot;
    uint32_t par;
};

template <int D>
__global__ void __launch_bounds__(kThreads3, 1)
fa_fwd3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
               const __grid_constant__ PeerMaps peers, const Fa3Args g) {
    using P16 = Pack16<DECA_F16>;
    constexpr uint32_t kQBytes = kBr * D * 2;
    constexpr uint32_t kKVBytes = kBc * D * 2;
    constexpr uint32_t kKVBlock = kBc * 128;
    constexpr uint32_t kIdescQK = make_idesc_f16(DECA_F16, false, false, kBr, kBc);
    constexpr uint32_t kIdescPV = make_idesc_f16(DECA_F16, false, true, kBr, D);
    constexpr uint32_t kTmemCols = 512;  // S_A, S_B (128 each), O_A, O_B (D each)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw);

    const int stages = g.stages;
    const uint32_t sQ = base;                    // Q_A, Q_B
    const uint32_t sKV = sQ + 2 * kQBytes;       // ring
    const uint32_t sO = sKV + stages * kKVBytes; // O staging, 4 KB per softmax warp
    const uint32_t sBar = sO + kOStageBytes;
    const uint32_t q_full = sBar;
    const uint32_t q_free = sBar + 8u;
    auto kv_full = [&](int i) { return sBar + 8u * (2 + i); };
    auto kv_empty = [&](int i) { return sBar + 8u * (2 + stages + i); };
    const uint32_t fixed0 = sBar + 8u * (2 + 2 * stages);
    auto s_full = [&](int grp) { return fixed0 + 8u * grp; };
    auto p_full = [&](int grp) { return fixed0 + 8u * (2 + grp); };
    auto pv_done = [&](int grp) { return fixed0 + 8u * (4 + grp); };
    const uint32_t drain_bar = fixed0 + 8u * 6;
    const uint32_t slot_addr = fixed0 + 8u * 7;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + (slot_addr - base));
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // The CTA's items, in the order every role walks them.
    // Non-causal (all items cost the same): items c, c + grid, ... of the head-major list, so the
    // CTAs that run together share a few heads' K and V.
    // Causal (pair p costs 2p + 2 tiles): the heads are cut into sections whose K and V fit in half of
    // L2; within a section the items are sorted longest first (pair n-1 of every head, then pair n-2,
    // ...) and dealt out in rounds of `grid` that alternate direction (CTA c takes position c of an
    // even round and grid - 1 - c of an odd one), which evens out the CTAs' totals.
    struct ItemWalk {
        int sec, round;
    };
    // advances to the CTA's next item (the first one when `first`); false when it has none left
    auto item_next = [&](ItemWalk &w, int &pair, int &bh, bool first) {
        const int G = (int)gridDim.x, c = (int)blockIdx.x;
        if (!first) ++w.round;
        if (!g.causal) {
            const int item = w.round * G + c;
            if (item >= g.n_heads * g.n_pairs) return false;
            bh = item / g.n_pairs;
            pair = item - bh * g.n_pairs;
            return true;
        }
        while (true) {
            const int h0 = w.sec * g.sec_heads;
            if (h0 >= g.n_heads) return false;
            const int heads = min(g.sec_heads, g.n_heads - h0);
            const int n = heads * g.n_pairs;  // positions of the section, longest pairs first
            if (w.round * G >= n) {
                ++w.sec;
                w.round = 0;
                continue;
            }
            const int pos = w.round * G + ((w.round & 1) ? (G - 1 - c) : c);
            if (pos < n) {
                pair = g.n_pairs - 1 - pos / heads;
                bh = h0 + pos % heads;
                return true;
            }
            ++w.round;  // the section's last, partial round has no position for this CTA
        }
    };
    auto tiles_of = [&](int pair, int &n_a, int &n_b) {
        n_a = g.causal ? ((2 * pair + 1) * kBr + kBc - 1) / kBc : g.S_kv / kBc;
        n_b = g.causal ? ((2 * pair + 2) * kBr + kBc - 1) / kBc : g.S_kv / kBc;
    };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        mbar_init(q_free, 1);
        for (int i = 0; i < stages; ++i) {
            mbar_init(kv_full(i), 1);
            mbar_init(kv_empty(i), 1);
        }
        for (int grp = 0; grp < 2; ++grp) {
            mbar_init(s_full(grp), 1);
            mbar_init(p_full(grp), 5);  // four softmax warps + the relay
            mbar_init(pv_done(grp), 1);
        }
        mbar_init(drain_bar, 1);
        fence_barrier_init();
        prefetch_tensormap(&tmQ);
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
    auto tS = [&](int grp) { return tmem_base + (uint32_t)(grp * kBc); };
    auto tO = [&](int grp) { return tmem_base + 2u * kBc + (uint32_t)(grp * D); };

    auto advance = [&](RingPos &p, int n) {
        p.slot += n;
        while (p.slot >= stages) p.slot -= stages, p.par ^= 1u;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            RingPos rp{0, 0u};
            int n_local = 0;
            ItemWalk walk{0, 0};
            int pair, bh;
            for (bool more = item_next(walk, pair, bh, true); more && ok; more = item_next(walk, pair, bh, false), ++n_local) {
                int n_a, n_b;
                tiles_of(pair, n_a, n_b);
                const int q_row0 = bh * g.S_q + pair * 2 * kBr;
                const int kv_row0 = bh * g.S_kv;
                // the Q tiles are free once every score MMA of the previous item has completed
                if (n_local > 0 && !mbar_wait(q_free, (uint32_t)((n_local - 1) & 1), abort_flag)) {
                    report_detail(g.status, 0, 1, n_local);
                    ok = false;
                    break;
                }
                mbar_arrive_expect_tx(q_full, 2 * kQBytes);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int blk = 0; blk < D / 64; ++blk)
                        tma_load_2d(sQ + t * kQBytes + blk * 16384, &tmQ, blk * 64, q_row0 + t * kBr, q_full);
                for (int i = 0; i < 2 * n_b; ++i) {  // ring item 2j = K_j, 2j + 1 = V_j
                    if (!mbar_wait(kv_empty(rp.slot), rp.par ^ 1u, abort_flag)) {
                        report_detail(g.status, 0, 2, i);
                        ok = false;
                        break;
                    }
                    const int row = kv_row0 + (i >> 1) * kBc;
                    const CUtensorMap *tm = (i & 1) ? &tmV : &tmK;
                    mbar_arrive_expect_tx(kv_full(rp.slot), kKVBytes);
#pragma unroll
                    for (int blk = 0; blk < D / 64; ++blk)
                        tma_load_2d(sKV + rp.slot * kKVBytes + blk * kKVBlock, tm, blk * 64, row, kv_full(rp.slot));
                    advance(rp, 1);
                }
            }
            // A wait that ran out lasted a second since this thread's last copy was issued, so none
            // of its copies is still in flight when the CTA leaves.
            if (!ok && *abort_flag == 0) {
                *abort_flag = 1;
                report_timeout(g.status, 0x411u);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = true;
            constexpr uint64_t kDescK = (uint64_t(16 >> 4) << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
            constexpr uint64_t kDescV = (uint64_t((kKVBlock >> 4) & 0x3FFF) << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
            const uint64_t q_desc[2] = {kDescK | (uint64_t)((sQ & 0x3FFFFu) >> 4),
                                        kDescK | (uint64_t)(((sQ + kQBytes) & 0x3FFFFu) >> 4)};
            auto issue_qk = [&](int grp, const RingPos &kp) {  // S_grp = Q_grp K^T
                const uint64_t kdesc = kDescK | (uint64_t)(((sKV + kp.slot * kKVBytes) & 0x3FFFFu) >> 4);
                const uint32_t d_tmem = tS(grp);
#pragma unroll
                for (int kd = 0; kd < D / 16; ++kd)
                    umma_f16_ss(d_tmem, q_desc[grp] + (((kd / 4) * 16384 + (kd % 4) * 32) >> 4),
                                kdesc + (((kd / 4) * kKVBlock + (kd % 4) * 32) >> 4), kIdescQK, kd != 0 ? 1u : 0u);
                umma_commit(s_full(grp));
            };
            auto issue_pv = [&](int grp, const RingPos &vp, uint32_t first, bool last) {  // O_grp (+)= P_grp V
                const uint64_t vdesc = kDescV | (uint64_t)(((sKV + vp.slot * kKVBytes) & 0x3FFFFu) >> 4);
                const uint32_t d_tmem = tO(grp);
                const uint32_t a_tmem = tS(grp);  // P: 16 keys = 8 packed columns of the score tile
#pragma unroll
                for (int kk = 0; kk < kBc / 16; ++kk)
                    umma_f16_ts(d_tmem, a_tmem + kk * 8, vdesc + kk * (2048 >> 4), kIdescPV, (first | kk) != 0 ? 1u : 0u);
                if (last) umma_commit(pv_done(grp));  // the item's O_grp is complete
            };
            // ring positions run on from item to item: kp = K tile whose scores are issued next,
            // vp = V tile of the next product; cnt[grp] = tiles of that group handled so far
            RingPos kp{0, 0u}, vp{1 % stages, (uint32_t)((1 / stages) & 1)};
            uint32_t cnt[2] = {0u, 0u};
            int n_local = 0;
            ItemWalk walk{0, 0};
            int pair, bh;
            for (bool more = item_next(walk, pair, bh, true); more && ok; more = item_next(walk, pair, bh, false), ++n_local) {
                int n_a, n_b;
                tiles_of(pair, n_a, n_b);
                // first tile: Q and K_0
                if (!mbar_wait(q_full, (uint32_t)(n_local & 1), abort_flag) ||
                    !mbar_wait(kv_full(kp.slot), kp.par, abort_flag)) {
                    report_detail(g.status, 1, 3, n_local);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                issue_qk(0, kp);
                issue_qk(1, kp);
                umma_commit(kv_empty(kp.slot));
                if (n_b == 1) umma_commit(q_free);  // that was the item's last score MMA
                advance(kp, 2);
                for (int j = 0; j < n_b && ok; ++j) {
                    const int jn = j + 1;  // tile whose scores are issued in this step (its K is at kp)
                    // V_j and K_jn have landed once p_full completes: the relay arrives there after them
                    if (j < n_a) {
                        if (!mbar_wait(p_full(0), (cnt[0] + (uint32_t)j) & 1u, abort_flag)) {
                            report_detail(g.status, 1, 5, j);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        // the product reads P from the buffer the next score MMA overwrites
                        issue_pv(0, vp, (uint32_t)j, jn == n_a);
                        if (jn < n_a) issue_qk(0, kp);
                    }
                    if (!mbar_wait(p_full(1), (cnt[1] + (uint32_t)j) & 1u, abort_flag)) {
                        report_detail(g.status, 1, 6, j);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    issue_pv(1, vp, (uint32_t)j, jn == n_b);
                    umma_commit(kv_empty(vp.slot));
                    if (jn < n_b) {
                        issue_qk(1, kp);
                        umma_commit(kv_empty(kp.slot));
                        if (jn == n_b - 1) umma_commit(q_free);  // the item's last score MMA
                        advance(kp, 2);
                    }
                    advance(vp, 2);
                }
                cnt[0] += (uint32_t)n_a;
                cnt[1] += (uint32_t)n_b;
            }
            if (!ok) {
                if (*abort_flag == 0) {
                    *abort_flag = 1;
                    report_timeout(g.status, 0x412u);
                }
                __shared__ uint32_t no_abort2;
                no_abort2 = 0;
                umma_commit(drain_bar);
                (void)mbar_wait(drain_bar, 0, &no_abort2);
            }
        }
        __syncwarp();
    } else if (warp == 10) {
        // ------------------------------------------------------------------ relay
        // Step j of an item needs V_j and K_{j+1}; both were requested a step or more earlier.  The
        // relay waits for them and then arrives on p_full of both Q tiles, in the issuer's place.  An
        // arrival must fall into the phase it is meant for, so the relay first sees the previous
        // phase of that barrier complete (it then still runs most of a step ahead of the softmax
        // warps' own arrivals).
        if (lane == 0) {
            bool ok = true;
            RingPos kp{0, 0u}, vp{1 % stages, (uint32_t)((1 / stages) & 1)};
            uint32_t cnt[2] = {0u, 0u};  // tiles of each group arrived for so far (all items)
            ItemWalk walk{0, 0};
            int pair, bh;
            for (bool more = item_next(walk, pair, bh, true); more && ok; more = item_next(walk, pair, bh, false)) {
                int n_a, n_b;
                tiles_of(pair, n_a, n_b);
                advance(kp, 2);  // K_0: the issuer waits for it itself, together with Q
                for (int j = 0; j < n_b && ok; ++j) {
                    const int jn = j + 1;
                    ok = mbar_wait(kv_full(vp.slot), vp.par, abort_flag) &&
                         (jn >= n_b || mbar_wait(kv_full(kp.slot), kp.par, abort_flag));
                    for (int grp = (j < n_a ? 0 : 1); grp < 2 && ok; ++grp) {
                        const uint32_t t = cnt[grp] + (uint32_t)j;
                        if (t > 0) ok = mbar_wait(p_full(grp), (t - 1u) & 1u, abort_flag);
                        if (ok) mbar_arrive(p_full(grp));
                    }
                    if (!ok) report_detail(g.status, 10, 4, j);
                    advance(vp, 2);
                    if (jn < n_b) advance(kp, 2);
                }
                cnt[0] += (uint32_t)n_a;
                cnt[1] += (uint32_t)n_b;
            }
            if (!ok && *abort_flag == 0) {
                *abort_flag = 1;
                report_timeout(g.status, 0x414u);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        const int grp = (warp - 2) >> 2;  // 0 = tile A, 1 = tile B
        const int q = warp & 3;           // tensor-memory lane quarter
        const int r = q * 32 + lane;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const uint32_t tSg = tS(grp) + lane_off;
        const uint32_t tOg = tO(grp) + lane_off;
        const uint32_t my_stage = sO + (uint32_t)(warp - 2) * 4096u;
        const float sl2 = g.sl2;
        bool ok = true;
        uint32_t cnt = 0;     // tiles of this group handled so far (all items)
        uint32_t n_item = 0;  // items handled so far
        auto wait_all = [&](uint32_t bar, uint32_t parity) {
            return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag)) != 0;
        };

        ItemWalk walk{0, 0};
        int pair, bh;
        for (bool more = item_next(walk, pair, bh, true); more && ok; more = item_next(walk, pair, bh, false)) {
            int n_a, n_b;
            tiles_of(pair, n_a, n_b);
            const int qt = 2 * pair + grp;
            const int row_abs = qt * kBr + r;
            const int n_kv = grp == 0 ? n_a : n_b;
            const int q_row0 = bh * g.S_q + pair * 2 * kBr;
            float m = kNegInf, l = 0.f;
            for (int j = 0; j < n_kv; ++j) {
                const uint32_t t = cnt + (uint32_t)j;
                if (!wait_all(s_full(grp), t & 1u)) {
                    if (lane == 0 && q == 0) report_detail(g.status, 2 + grp, 7, j);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const bool diag = g.causal && ((j + 1) * kBc - 1 > qt * kBr);
                const int col0 = j * kBc;
                // a rescale needs the product of the previous tile complete: it was issued before the
                // score MMAs whose completion s_full has just reported, and MMAs complete in order
                auto wait_prev = [&]() { return true; };
                auto wait_p = [&]() { return true; };  // P reuses the score tile that was just filled
                const bool step_ok =
                    diag ? fa_softmax_step<kBc, D, true, true>(tSg, tOg, tSg, r, col0, row_abs, sl2, j == 0, m, l, wait_p,
                                                               wait_prev)
                         : fa_softmax_step<kBc, D, false, true>(tSg, tOg, tSg, r, col0, row_abs, sl2, j == 0, m, l, wait_p,
                                                                wait_prev);
                if (!step_ok) {
                    if (lane == 0 && q == 0) report_detail(g.status, 2 + grp, 8, j);
                    ok = false;
                    break;
                }
                // S is consumed, P (and a possibly rescaled O) are ready
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full(grp));
            }
            if (!ok) break;
            if (!wait_all(pv_done(grp), n_item & 1u)) {
                if (lane == 0 && q == 0) report_detail(g.status, 2 + grp, 9, n_kv);
                ok = false;
                break;
            }
            cnt += (uint32_t)n_kv;
            ++n_item;
            // ---- epilogue: O / l -> fp16 -> this warp's staging panel -> TMA stores, 64 columns at a time
            tc_fence_after_sync();
            const float inv = 1.0f / l;
#pragma unroll 1
            for (int blk = 0; blk < D / 64; ++blk) {
                uint32_t v0[32], v1[32];
                tmem_ld_32x32b_x32(tOg + blk * 64, v0);
                tmem_ld_32x32b_x32(tOg + blk * 64 + 32, v1);
                tmem_ld_wait();
                if (lane == 0) tma_store_wait_read<0>();  // the panel's previous stores have read it
                __syncwarp();
                const uint32_t rowb = my_stage + lane * 128;
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    const uint32_t *v = cc < 4 ? &v0[cc * 8] : &v1[(cc - 4) * 8];
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        o[i] = P16::pack(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
                    const uint32_t dst = rowb + ((cc ^ (lane & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                                 "r"(o[3])
                                 : "memory");
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const int row = q_row0 + grp * kBr + q * 32;
                    tma_store_2d(&tmO, my_stage, blk * 64, row);
                    // gather: the same rows of O go to the other ranks' copies (plain TMA stores to peer memory)
                    for (int pr = 0; pr < g.n_peers; ++pr) tma_store_2d(&peers.m[pr], my_stage, blk * 64, row);
                    tma_store_commit();
                }
            }
            // the next item's first P is published only after these loads of O: that orders its
            // first product (which overwrites O) behind them
            tc_fence_before_sync();
        }
        if (!ok && lane == 0 && *abort_flag == 0) {
            *abort_flag = 1;
            report_timeout(g.status, 0x413u);
        }
        // the CTA may leave once its stores have read shared memory (the writes complete with the
        // grid); stores to peers are waited for in full
        if (lane == 0) {
            if (g.n_peers > 0)
                tma_store_wait<0>();
            else
                tma_store_wait_read<0>();
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

template <int D>
int launch_fa3(const CUtensorMap &tmQ, const CUtensorMap &tmK, const CUtensorMap &tmV, const CUtensorMap &tmO,
               const PeerMaps &peers, const Fa3Args &g, unsigned grid, size_t smem, cudaStream_t st) {
    static SmemLimitCache configured;
    if (int rc = ensure_dynamic_smem(fa_fwd3_kernel<D>, smem, configured)) return rc;
    fa_fwd3_kernel<D><<<grid, kThreads3, smem, st>>>(tmQ, tmK, tmV, tmO, peers, g);
    return (int)cudaGetLastError();
}

}  // namespace

namespace {

// Causal schedules deal the items of one section of heads (longest pairs first) to the CTAs in
// rounds of alternating direction, exactly as the kernel's item walk does; this is the largest
// CTA total that results, in tiles.
double causal_balance(int grid, int n_heads, int n_pairs, int sec_heads) {
    std::vector<long long> load(grid, 0);
    long long total = 0;
    for (int h0 = 0; h0 < n_heads; h0 += sec_heads) {
        const int heads = sec_heads < n_heads - h0 ? sec_heads : n_heads - h0;
        const int n = heads * n_pairs;
        for (int pos = 0; pos < n; ++pos) {
            const int r = pos / grid, k = pos % grid;
            const int cost = 2 * (n_pairs - 1 - pos / heads) + 2;
            load[(r & 1) ? grid - 1 - k : k] += cost;
            total += cost;
        }
    }
    long long mx = 1;
    for (long long v : load) mx = v > mx ? v : mx;
    return (double)total / grid / (double)mx;
}

// Heads per section for a causal problem: the candidate with the best product of the balance of
// its static schedule and an L2 term (measured on B200: the K and V of a section cost nothing up
// to a quarter of L2, about 14 % at a full L2, more beyond).  Cached per problem.
int choose_sec_heads(int grid, int n_heads, int n_pairs, long long kv_bytes_per_head, long long l2_bytes) {
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, long long, long long>, int> cache;
    const auto key = std::make_tuple(grid, n_heads, n_pairs, kv_bytes_per_head, l2_bytes);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int best = n_heads;
    double best_score = -1.0;
    for (int h = 1; h <= n_heads; h = (h < 64 ? h + 1 : (h < 256 ? h + 8 : h * 2))) {
        const int hh = h > n_heads ? n_heads : h;
        if ((long long)n_heads * n_pairs * (n_heads / hh + 1) > 50000000ll) continue;  // keep the search cheap
        const double frac = (double)hh * (double)kv_bytes_per_head / (double)l2_bytes;
        double f = 1.0;
        if (frac > 0.25) f -= 0.14 * ((frac < 1.0 ? frac : 1.0) - 0.25) / 0.75;
        if (frac > 1.0) f -= 0.05 * ((frac < 4.0 ? frac : 4.0) - 1.0);
        const double score = causal_balance(grid, n_heads, n_pairs, hh) * f;
        if (score > best_score + 1e-9) best_score = score, best = hh;
    }
    {
        // the whole problem as one section is always a candidate
        const double frac = (double)n_heads * (double)kv_bytes_per_head / (double)l2_bytes;
        double f = 1.0;
        if (frac > 0.25) f -= 0.14 * ((frac < 1.0 ? frac : 1.0) - 0.25) / 0.75;
        if (frac > 1.0) f -= 0.05 * ((frac < 4.0 ? frac : 4.0) - 1.0);
        if ((long long)n_heads * n_pairs <= 50000000ll && causal_balance(grid, n_heads, n_pairs, n_heads) * f > best_score + 1e-9)
            best = n_heads;
    }
    cache[key] = best;
    return best;
}

}  // namespace

size_t fa3_smem_bytes(int D, int stages) {
    return 1024 + 2 * (size_t)kBr * D * 2 + (size_t)stages * kBc * D * 2 + kOStageBytes + 8 * (2 * (size_t)stages + 16);
}

// Host rules of the persistent two-tile schedule; shared with deca_fa_fwd_f16_check_config.
int fa3_check(int S_q, int S_kv, int D, const deca_fa_cfg &c) {
    if (c.Br != kBr || c.Bc != kBc || c.q_tiles != 2 || !c.p_tmem) return DECA_ERR_CONFIG;
    if (S_q % (2 * kBr) != 0 || S_kv % kBc != 0) return DECA_ERR_CONFIG;
    if (c.stages < 2 || c.stages > 8) return DECA_ERR_CONFIG;
    if (fa3_smem_bytes(D, c.stages) > 232448) return DECA_ERR_CONFIG;
    return DECA_OK;
}

int fa3_launch(const CUtensorMap &tmQ, const CUtensorMap &tmK, const CUtensorMap &tmV, const CUtensorMap &tmO,
               const PeerMaps &peers, int n_peers, int B, int H, int S_q, int S_kv, int D, float softmax_scale, int causal,
               const deca_fa_cfg &c, cudaStream_t st) {
    Fa3Args g;
    g.n_peers = n_peers;
    g.S_q = S_q, g.S_kv = S_kv;
    g.causal = causal ? 1 : 0;
    g.stages = c.stages;
    g.sl2 = softmax_scale * kLog2e;
    g.n_pairs = S_q / (2 * kBr);
    const int64_t items = (int64_t)g.n_pairs * B * H;
    if (items > 2147483647ll) return DECA_ERR_SHAPE;
    g.n_heads = B * H;
    g.status = device_status_ptr();
    if (!g.status) return (int)cudaErrorUnknown;
    DeviceInfo di;
    const int rc = current_device_info(&di);
    if (rc) return rc;
    const int sms = di.sms, l2 = di.l2_bytes;
    const unsigned grid = (unsigned)(items < sms ? items : sms);
    g.sec_heads = g.n_heads;
    if (causal) g.sec_heads = choose_sec_heads((int)grid, g.n_heads, g.n_pairs, 2ll * S_kv * D * 2, l2);
    const size_t smem = fa3_smem_bytes(D, c.stages);
    return D == 128 ? launch_fa3<128>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st)
                    : launch_fa3<64>(tmQ, tmK, tmV, tmO, peers, g, grid, smem, st);
}

}  // namespace deca
