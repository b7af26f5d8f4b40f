// Per-row online softmax of one 128 x BC score tile held in tensor memory; shared by the two
// FlashAttention schedules.  One thread owns one query row (one tensor-memory lane).
//
// Recurrence of the reference kernel (flash_attn_tir.py:403-438: finite -1e30 mask value, scale
// folded into the exp2 argument, fp32 sum of the unrounded probabilities, P rounded to fp16) with
// a lazily updated running max: as long as the tile's row max exceeds the running max m by at
// most 2^8 in the exponent, m is kept (P <= 256 is exact enough in fp16 and everything is
// normalised by l at the end), so the common case is ONE pass over the scores: exponentials with
// the old max, the row sum and the tile max together (with P in tensor memory not even the max:
// a row sum of at most 2^8 already bounds every probability of the tile).  Only when some row of
// the warp grew by more (always on the first tile) the slow path runs: raise m, rescale l and the
// O accumulator in tensor memory, and redo the exponentials with the new max.
#pragma once

#include <type_traits>

#include "ptx.cuh"

namespace deca {


constexpr float kFaRescaleThreshold = 8.0f;  // log2 units
constexpr float kFaSumLimit = 256.0f;        // 2^threshold: bound of a tile's row sum on the fast path

// Exponentials of the row with max term `ms` (= m * sl2): writes P (fp16) into the K-major,
// 128-byte swizzled shared tile at `p_base` (64-key blocks of 128 rows x 128 bytes) and returns
// the row sum; with TRACK also folds the (masked) raw scores into `mx`.
// With PTMEM the fp16 P tile goes to tensor memory instead, packed two keys per 32-bit column
// into the first BC / 2 columns of the score tile it was computed from (`p_base` is then that
// tile's tensor-memory address): the 64 scores of a chunk are in registers before the 32 columns
// that receive their probabilities are overwritten, and no other thread touches this lane.
template <int BC, bool MASKED, bool TRACK, bool PTMEM>
__device__ __forceinline__ float fa_exp_tile(uint32_t tS, uint32_t p_base, int r, int col0, int row_abs, float sl2,
                                             float ms, float &mx) {
    using P16 = Pack16<DECA_F16>;
    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
    float max4[4] = {kNegInf, kNegInf, kNegInf, kNegInf};
#pragma unroll 1
    for (int h = 0; h < BC / 64; ++h) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(tS + h * 64, v0);
        tmem_ld_32x32b_x32(tS + h * 64 + 32, v1);
        tmem_ld_wait();
        uint32_t p[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float s0 = __uint_as_float(v0[2 * i]), s1 = __uint_as_float(v0[2 * i + 1]);
            float s2 = __uint_as_float(v1[2 * i]), s3 = __uint_as_float(v1[2 * i + 1]);
            if constexpr (MASKED) {
                const int cb = col0 + h * 64 + 2 * i;
                if (cb > row_abs) s0 = kNegInf;
                if (cb + 1 > row_abs) s1 = kNegInf;
                if (cb + 32 > row_abs) s2 = kNegInf;
                if (cb + 33 > row_abs) s3 = kNegInf;
            }
            if constexpr (TRACK) {
                max4[0] = fmaxf(max4[0], s0), max4[1] = fmaxf(max4[1], s1);
                max4[2] = fmaxf(max4[2], s2), max4[3] = fmaxf(max4[3], s3);
            }
            const float p0 = ex2_approx(fmaf(s0, sl2, -ms)), p1 = ex2_approx(fmaf(s1, sl2, -ms));
            const float p2 = ex2_approx(fmaf(s2, sl2, -ms)), p3 = ex2_approx(fmaf(s3, sl2, -ms));
            sum4[0] += p0, sum4[1] += p1, sum4[2] += p2, sum4[3] += p3;
            p[i] = P16::pack(p0, p1);
            p[16 + i] = P16::pack(p2, p3);
        }
        if constexpr (PTMEM) {
            // p[i] holds keys (2i, 2i+1) of the first 32 and p[16 + i] of the second 32: 32 columns
            tmem_st_32x32b_x32(p_base + h * 32, p);
        } else {
            const uint32_t rowb = p_base + h * 16384 + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t dst = rowb + ((c ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[4 * c]), "r"(p[4 * c + 1]),
                             "r"(p[4 * c + 2]), "r"(p[4 * c + 3])
                             : "memory");
            }
        }
    }
    if constexpr (PTMEM) tmem_st_wait();
    if constexpr (TRACK) mx = fmaxf(fmaxf(max4[0], max4[1]), fmaxf(max4[2], max4[3]));
    return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

// 2^x for two scores on the FMA pipe instead of the exp2 unit (x = s * sl2 - ms):
//   t = sat(x / 256 + 126 / 256) clamps to x' = 256 t - 126 in [-126, 130) (one saturating fma per
//   score: what lies below 2^-126 counts as 2^-126), r = x' + 1.5 * 2^23 rounds x' to the nearest
//   integer j in r's low mantissa bits, a degree-3 polynomial (relative error 7.6e-5, a sixth of
//   an fp16 ulp) gives 2^(x' - j) on [-0.5, 0.5], and one integer multiply-add puts j into the
//   exponent (r's bits times 2^23 is j * 2^23 modulo 2^32).  The additions and the polynomial
//   run as packed pairs.
struct FaPolyConst {
    float sl2_256, off;  // sl2 / 256, 126 / 256 - ms / 256
};
__device__ __forceinline__ void fa_exp2_poly_pair(float s0, float s1, const FaPolyConst &k, float &p0, float &p1) {
    float t0, t1;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(t0) : "f"(s0), "f"(k.sl2_256), "f"(k.off));
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(t1) : "f"(s1), "f"(k.sl2_256), "f"(k.off));
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
    const uint64_t x = f32x2_fma(f32x2_pack(t0, t1), f32x2_pack(256.0f, 256.0f), f32x2_pack(-126.0f, -126.0f));
    const uint64_t r = f32x2_add(x, f32x2_pack(kMagic, kMagic));
    const uint64_t j = f32x2_add(r, f32x2_pack(-kMagic, -kMagic));
    const uint64_t f = f32x2_fma(j, f32x2_pack(-1.0f, -1.0f), x);
    uint64_t q = f32x2_fma(f32x2_pack(0.05520550534f, 0.05520550534f), f, f32x2_pack(0.24261397123f, 0.24261397123f));
    q = f32x2_fma(q, f, f32x2_pack(0.69325476885f, 0.69325476885f));
    q = f32x2_fma(q, f, f32x2_pack(0.99992769957f, 0.99992769957f));
    uint32_t q0, q1, r0, r1;
    f32x2_unpack_bits(q, q0, q1);
    f32x2_unpack_bits(r, r0, r1);
    uint32_t e0, e1;
    asm("mad.lo.s32 %0, %1, 8388608, %2;" : "=r"(e0) : "r"(r0), "r"(q0));
    asm("mad.lo.s32 %0, %1, 8388608, %2;" : "=r"(e1) : "r"(r1), "r"(q1));
    p0 = __uint_as_float(e0), p1 = __uint_as_float(e1);
}

// Share of the exponentials of an unmasked tile that is taken on the FMA pipe: every EVERY-th pair
// of scores (0: none).  At D = 64 the exp2 unit alone bounds the kernel (half the tensor work per
// exponential) and a share on the FMA pipe pays: 682 -> 728 ... 747 TFLOPS back to back and 700 -> 798
// in isolated launches with every fourth pair (every fifth or eighth measure the same, every third
// 708, every second 684).  At D = 128, where the step is a dependency chain and the pass only a part
// of it, the longer instruction stream costs what the unit gains (1 147 -> 1 143, 1 282 -> 1 258).
template <int D>
constexpr int kFaPolyEveryFor = D == 64 ? 4 : 0;

// 32 scores of one row (keys cb0 .. cb0 + 31): adds the exponentials 2^(s * sl2 - ms) of the
// (masked) scores to the packed sums and packs them to fp16, keys (2i, 2i + 1) in pk[i].
template <bool MASKED, int EVERY>
__device__ __forceinline__ void fa_exp_chunk32(const uint32_t (&v)[32], int cb0, int row_abs, uint64_t sl2x2,
                                               uint64_t nmsx2, const FaPolyConst &pc, uint64_t (&sum2)[2], uint32_t *pk) {
    using P16 = Pack16<DECA_F16>;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float s0 = __uint_as_float(v[2 * i]), s1 = __uint_as_float(v[2 * i + 1]);
        if constexpr (MASKED) {
            if (cb0 + 2 * i > row_abs) s0 = kNegInf;
            if (cb0 + 2 * i + 1 > row_abs) s1 = kNegInf;
        }
        float p0, p1;
        if (!MASKED && EVERY > 0 && i % (EVERY > 0 ? EVERY : 1) == (EVERY > 0 ? EVERY : 1) - 1) {
            fa_exp2_poly_pair(s0, s1, pc, p0, p1);
        } else {
            float x0, x1;
            f32x2_unpack(f32x2_fma(f32x2_pack(s0, s1), sl2x2, nmsx2), x0, x1);
            p0 = ex2_approx(x0), p1 = ex2_approx(x1);
        }
        sum2[i & 1] = f32x2_add(sum2[i & 1], f32x2_pack(p0, p1));
        pk[i] = P16::pack(p0, p1);
    }
}

// Fast-path variant for P in tensor memory: the exponentials (with the running max) are packed
// into registers `pk` and NOT stored, because storing would overwrite the scores that a redo with
// a raised max still needs; the caller stores them once the warp has voted that no row grew by
// more than the threshold.  No maximum is tracked: the caller tests the returned row sum instead.
// The tensor-memory load of the next 32 columns is in flight while the current 32 are processed.
template <int BC, bool MASKED, int EVERY>
__device__ __forceinline__ float fa_exp_tile_hold(uint32_t tS, int col0, int row_abs, float sl2, float ms,
                                                  uint32_t (&pk)[BC / 2]) {
    constexpr int kChunks = BC / 32;
    const uint64_t sl2x2 = f32x2_pack(sl2, sl2), nmsx2 = f32x2_pack(-ms, -ms);
    const FaPolyConst pc = {sl2 * (1.0f / 256.0f), 126.0f / 256.0f - ms * (1.0f / 256.0f)};
    uint64_t sum2[2] = {0ull, 0ull};
    uint32_t v[2][32];
    tmem_ld_32x32b_x32(tS, v[0]);
    tmem_ld_wait_regs(v[0]);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        if (c + 1 < kChunks) tmem_ld_32x32b_x32(tS + (c + 1) * 32, v[(c + 1) & 1]);
        // chunk c = keys 32c ..: half h = c / 2 of the tile, words (c % 2) * 16 .. of that half
        fa_exp_chunk32<MASKED, EVERY>(v[c & 1], col0 + c * 32, row_abs, sl2x2, nmsx2, pc, sum2,
                               &pk[(c / 2) * 32 + (c % 2) * 16]);
        if (c + 1 < kChunks) tmem_ld_wait_regs(v[(c + 1) & 1]);
    }
    float a0, a1, b0, b1;
    f32x2_unpack(sum2[0], a0, a1);
    f32x2_unpack(sum2[1], b0, b1);
    return (a0 + a1) + (b0 + b1);
}

// (masked) row maximum of the tile
template <int BC, bool MASKED>
__device__ __forceinline__ float fa_row_max(uint32_t tS, int col0, int row_abs) {
    float mx = kNegInf;
#pragma unroll 1
    for (int c = 0; c < BC / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tS + c * 32, v);
        tmem_ld_wait();
        float part[4] = {kNegInf, kNegInf, kNegInf, kNegInf};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float s = __uint_as_float(v[i]);
            if constexpr (MASKED) {
                if (col0 + c * 32 + i > row_abs) s = kNegInf;
            }
            part[i & 3] = fmaxf(part[i & 3], s);
        }
        mx = fmaxf(mx, fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])));
    }
    return mx;
}

// One KV step of the online softmax for this thread's row.  `tS` / `tO` are the tensor-memory
// addresses of the score tile and of the O accumulator including the warp's lane offset.
// `wait_p_free()` must return once the P tile at `p_base` may be overwritten, `wait_o_ready()`
// once O holds the sum over all previous KV tiles (both return false when a bounded wait ran
// out, and must be warp-uniform).  Updates m and l; returns false on such a failure.
template <int BC, int D, bool MASKED, bool PTMEM, typename WaitP, typename WaitO>
__device__ __forceinline__ bool fa_softmax_step(uint32_t tS, uint32_t tO, uint32_t p_base, int r, int col0, int row_abs,
                                                float sl2, bool first_tile, float &m, float &l, WaitP wait_p_free,
                                                WaitO wait_o_ready) {
    if (!wait_p_free()) return false;
    float mx, lsum = 0.f;
    bool have_p = false, raise;
    if (first_tile && !PTMEM) {
        mx = fa_row_max<BC, MASKED>(tS, col0, row_abs);
        raise = true;
    } else if constexpr (PTMEM) {
        if (first_tile) {
            // nothing accumulated yet (l = 0, O empty): start the running max at the maximum of
            // the first 32 keys (key 0 is visible to every row) and take the fast path; the rest
            // of the tile rarely exceeds it by 2^8, and then the slow path below corrects it
            uint32_t v[32];
            tmem_ld_32x32b_x32(tS, v);
            tmem_ld_wait();
            float part[4] = {kNegInf, kNegInf, kNegInf, kNegInf};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float sc = __uint_as_float(v[i]);
                if constexpr (MASKED) {
                    if (col0 + i > row_abs) sc = kNegInf;
                }
                part[i & 3] = fmaxf(part[i & 3], sc);
            }
            m = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
        }
        // fast path, P to tensor memory: hold the packed probabilities until the vote, because
        // storing them overwrites the scores a redo would need.  The vote is on the row sum: the
        // probabilities are positive, so a sum of at most 2^threshold bounds every one of them
        // (no score grew by more than the threshold) without a max over the scores; a larger sum
        // sends the warp down the slow path, where the exact maximum is taken and m raised.
        uint32_t pk[BC / 2];
        lsum = fa_exp_tile_hold<BC, MASKED, kFaPolyEveryFor<D>>(tS, col0, row_abs, sl2, m * sl2, pk);
        const bool slow = __any_sync(0xFFFFFFFFu, !(lsum <= kFaSumLimit)) != 0;
        if (!slow) {
#pragma unroll
            for (int h = 0; h < BC / 64; ++h) {
                uint32_t part[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) part[i] = pk[h * 32 + i];
                tmem_st_32x32b_x32(p_base + h * 32, part);
            }
            tmem_st_wait();
            l += lsum;
            return true;
        }
        mx = fa_row_max<BC, MASKED>(tS, col0, row_abs);
        raise = true;
    } else {
        // fast path, P to shared memory: exponentials with the running max, tile max on the side
        lsum = fa_exp_tile<BC, MASKED, true, PTMEM>(tS, p_base, r, col0, row_abs, sl2, m * sl2, mx);
        have_p = true;
        raise = __any_sync(0xFFFFFFFFu, (mx - m) * sl2 > kFaRescaleThreshold) != 0;
    }
    if (raise) {
        // raise the max, rescale l and O; exponentials computed with the old max are redone
        const float m_new = fmaxf(m, mx);
        const float alpha = ex2_approx((m - m_new) * sl2);
        l *= alpha;
        m = m_new;
        have_p = false;
        if (!first_tile) {
            if (!wait_o_ready()) return false;
            tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tO + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                tmem_st_32x32b_x32(tO + c * 32, v);
            }
            tmem_st_wait();
        }
    }
    if (!have_p) {
        float unused;
        lsum = fa_exp_tile<BC, MASKED, false, PTMEM>(tS, p_base, r, col0, row_abs, sl2, m * sl2, unused);
    }
    l += lsum;
    return true;
}

}  // namespace deca
