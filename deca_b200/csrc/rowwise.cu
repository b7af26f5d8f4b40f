// Row-wise softmax / RMSNorm for B200: HBM-bound streaming kernels.
//
// Same decomposition as the reference generator make_rowwise (src/kernels/rowwise_tir.py:99-391):
// `threads_per_row` threads own the interleaved 16-byte (or 8-byte) chunks
// (c * threads_per_row + t) * vec of a row, `rows_per_block` rows share a CTA, reductions
// are a warp shuffle butterfly followed by a shared-memory exchange between the warps of a
// row, all math is fp32.  Unlike the reference (one nvcc build per shape and config), the
// kernels take the shape at run time; only the per-thread chunk count of the register mode,
// the vector width, the dtype and the cache-hint flavour are template parameters.
//
//   reg     : the row is read once into registers, reduced, written once
//             (algorithmic traffic 2 * M * N * 2 bytes -- the roofline numerator).
//   twopass : rows too long for registers: pass 1 keeps an online (max, sum) / a sum of
//             squares per thread, pass 2 re-reads the row (from L2 when the rows in flight
//             fit) and writes the result.
//   cluster : rows too long for the registers of ONE CTA stay one-pass: a thread-block cluster
//             of 2, 4 or 8 CTAs shares a row, each CTA caches its contiguous slice in registers
//             as in reg mode, and the row statistics are combined across the cluster through
//             distributed shared memory (every CTA stores its partial value into each peer's
//             slot, one cluster barrier per reduction).  No second pass, no clusters across GPUs.
//
// Softmax keeps exp2(x*log2e - max*log2e) of the cached row in fp32 registers between the
// sum and the output pass, so the MUFU unit sees each element once, and takes the row
// maximum on packed 16-bit pairs before any conversion.
#include <atomic>

#include "common.cuh"

namespace deca {
namespace {

template <int WORDS, bool HINT>
__device__ __forceinline__ void load_words(uint32_t (&d)[WORDS], const void *p) {
    static_assert(WORDS == 4 || WORDS == 2 || WORDS == 1, "16-, 8- or 4-byte accesses");
    if constexpr (WORDS == 1) {
        if constexpr (HINT) {
            asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(d[0]) : "l"(p));
        } else {
            d[0] = *reinterpret_cast<const uint32_t *>(p);
        }
    } else if constexpr (WORDS == 4) {
        if constexpr (HINT) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                         : "l"(p));
        } else {
            uint4 v = *reinterpret_cast<const uint4 *>(p);
            d[0] = v.x, d[1] = v.y, d[2] = v.z, d[3] = v.w;
        }
    } else {
        if constexpr (HINT) {
            asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                         : "=r"(d[0]), "=r"(d[1])
                         : "l"(p));
        } else {
            uint2 v = *reinterpret_cast<const uint2 *>(p);
            d[0] = v.x, d[1] = v.y;
        }
    }
}

template <int WORDS, bool HINT>
__device__ __forceinline__ void store_words(void *p, const uint32_t (&d)[WORDS]) {
    if constexpr (WORDS == 1) {
        if constexpr (HINT) {
            asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(d[0]) : "memory");
        } else {
            *reinterpret_cast<uint32_t *>(p) = d[0];
        }
    } else if constexpr (WORDS == 4) {
        if constexpr (HINT) {
            asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d[0]), "r"(d[1]), "r"(d[2]),
                         "r"(d[3])
                         : "memory");
        } else {
            *reinterpret_cast<uint4 *>(p) = make_uint4(d[0], d[1], d[2], d[3]);
        }
    } else {
        if constexpr (HINT) {
            asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(d[0]), "r"(d[1]) : "memory");
        } else {
            *reinterpret_cast<uint2 *>(p) = make_uint2(d[0], d[1]);
        }
    }
}

struct MaxOp {
    static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};
struct SumOp {
    static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};

// Reduction of `v` over all threads of one row: shuffle butterfly inside each warp, then the
// warps of the row exchange through `red` (one slot per warp of the CTA).  Every thread of
// the CTA must call it (block barrier inside when a row spans more than one warp).
template <typename Op>
__device__ __forceinline__ float row_reduce(float v, float *red, int nw, int row_warp0, int wr, int lane) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = Op::apply(v, __shfl_xor_sync(0xFFFFFFFFu, v, m));
    if (nw > 1) {
        if (lane == 0) red[row_warp0 + wr] = v;
        __syncthreads();
        v = red[row_warp0];
        for (int i = 1; i < nw; ++i) v = Op::apply(v, red[row_warp0 + i]);
    }
    return v;
}

// Elements of a row each CTA of a `cs`-CTA cluster takes: an equal share rounded up to whole vectors.
inline int cluster_slice(int N, int cs, int vec) { return ((N + cs - 1) / cs + vec - 1) / vec * vec; }

struct RowArgs {
    const char *x;
    const char *w;
    char *y;
    long long M;
    int N;
    int tpr;  // threads per row
    float eps;
    float inv_n;
    // optional [M, 2] fp32 output of the row statistics as the kernel computed them (null: off):
    // softmax (row max * log2 e, 1 / sum of exponentials); RMSNorm (rsqrt(mean x^2 + eps), sum x^2)
    float *stats;
};

// ------------------------------------------------------------------------------------------
// Register mode: C chunks of VEC = 2 * WORDS elements per thread, all loads issued up front.
// ------------------------------------------------------------------------------------------
template <int OP, int DT, int WORDS, int C, bool HINT>
__global__ void rowwise_reg_kernel(const RowArgs a) {
    using P = Pack16<DT>;
    constexpr int VEC = 2 * WORDS;
    __shared__ float red[2][32];

    const int tpr = a.tpr;
    const int t = threadIdx.x % tpr;
    const int rb = threadIdx.x / tpr;
    const int rpb = blockDim.x / tpr;
    const int lane = threadIdx.x & 31;
    const int wr = t >> 5;
    const int nw = tpr >> 5;
    const int row_warp0 = rb * nw;
    const long long row = (long long)blockIdx.x * rpb + rb;
    const char *xrow = a.x + row * a.N * 2;
    char *yrow = a.y + row * a.N * 2;

    uint32_t cache[C][WORDS];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int col = (c * tpr + t) * VEC;
        if (col < a.N) {
            load_words<WORDS, HINT>(cache[c], xrow + (size_t)col * 2);
        } else {
#pragma unroll
            for (int i = 0; i < WORDS; ++i) cache[c][i] = (OP == DECA_SOFTMAX) ? P::kNegInfPair : 0u;
        }
    }

    if constexpr (OP == DECA_SOFTMAX) {
        // max on packed pairs (exact), one conversion at the end
        uint32_t mx = cache[0][0];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) mx = P::max2(mx, cache[c][i]);
        float2 mf = P::unpack(mx);
        float m = row_reduce<MaxOp>(fmaxf(mf.x, mf.y), red[0], nw, row_warp0, wr, lane);
        const float ml = m * kLog2e;

        // Up to 128 cached elements per thread the exponentials stay in fp32 registers between
        // the sum and the output; longer register rows keep the packed input and recompute.
        constexpr bool KEEP_E = (C * VEC <= 128);
        float e[KEEP_E ? C : 1][VEC];
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                float2 f = P::unpack(cache[c][i]);
                const float e0 = ex2_approx(fmaf(f.x, kLog2e, -ml));
                const float e1 = ex2_approx(fmaf(f.y, kLog2e, -ml));
                if constexpr (KEEP_E) e[c][2 * i] = e0, e[c][2 * i + 1] = e1;
                s += e0 + e1;
            }
        s = row_reduce<SumOp>(s, red[1], nw, row_warp0, wr, lane);
        const float inv = 1.0f / s;
        if (a.stats != nullptr && t == 0) a.stats[2 * row] = ml, a.stats[2 * row + 1] = inv;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = (c * tpr + t) * VEC;
            if (col < a.N) {
                uint32_t o[WORDS];
#pragma unroll
                for (int i = 0; i < WORDS; ++i) {
                    if constexpr (KEEP_E) {
                        o[i] = P::pack(e[c][2 * i] * inv, e[c][2 * i + 1] * inv);
                    } else {
                        float2 f = P::unpack(cache[c][i]);
                        o[i] = P::pack(ex2_approx(fmaf(f.x, kLog2e, -ml)) * inv,
                                       ex2_approx(fmaf(f.y, kLog2e, -ml)) * inv);
                    }
                }
                store_words<WORDS, HINT>(yrow + (size_t)col * 2, o);
            }
        }
    } else {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                float2 f = P::unpack(cache[c][i]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
        ss = row_reduce<SumOp>(ss, red[0], nw, row_warp0, wr, lane);
        const float r = rsqrtf(ss * a.inv_n + a.eps);
        if (a.stats != nullptr && t == 0) a.stats[2 * row] = r, a.stats[2 * row + 1] = ss;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = (c * tpr + t) * VEC;
            if (col < a.N) {
                uint32_t wv[WORDS], o[WORDS];
                load_words<WORDS, false>(wv, a.w + (size_t)col * 2);
#pragma unroll
                for (int i = 0; i < WORDS; ++i) {
                    float2 f = P::unpack(cache[c][i]);
                    // x * r is rounded to the I/O dtype before the weight multiply
                    float2 n = P::unpack(P::pack(f.x * r, f.y * r));
                    float2 g = P::unpack(wv[i]);
                    o[i] = P::pack(n.x * g.x, n.y * g.y);
                }
                store_words<WORDS, HINT>(yrow + (size_t)col * 2, o);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Cluster mode: one row per cluster, one contiguous slice of it per CTA, cached in registers.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t row_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void row_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Every CTA of the cluster holds `v` (its slice's value) in all threads; returns the combination
// over the cluster.  `slots` is this CTA's array of one float per cluster rank: thread i < cs
// stores v into slot [my rank] of CTA i, the cluster barrier publishes the stores.
template <typename Op>
__device__ __forceinline__ float cluster_combine(float v, float *slots, uint32_t rank, uint32_t cs) {
    if (threadIdx.x < cs) {
        const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(slots + rank));
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(threadIdx.x));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
    }
    row_cluster_sync();
    float r = slots[0];
    for (uint32_t i = 1; i < cs; ++i) r = Op::apply(r, slots[i]);
    return r;
}

template <int OP, int DT, int WORDS, int C, bool HINT>
__global__ void rowwise_cluster_kernel(const RowArgs a, int cs, int slice) {
    using P = Pack16<DT>;
    constexpr int VEC = 2 * WORDS;
    __shared__ float red[2][32];
    __shared__ float cl[2][8];

    const int tpr = blockDim.x;  // the whole CTA works on one slice
    const int t = threadIdx.x;
    const int lane = t & 31;
    const int wr = t >> 5;
    const int nw = tpr >> 5;
    const uint32_t rank = row_cluster_rank();
    const long long row = blockIdx.x / cs;
    const int s0 = (int)rank * slice;              // first element of this CTA's slice
    const int s1 = min(a.N, s0 + slice);           // one past its last
    const char *xrow = a.x + row * a.N * 2;
    char *yrow = a.y + row * a.N * 2;

    uint32_t cache[C][WORDS];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int col = s0 + (c * tpr + t) * VEC;
        if (col < s1) {
            load_words<WORDS, HINT>(cache[c], xrow + (size_t)col * 2);
        } else {
#pragma unroll
            for (int i = 0; i < WORDS; ++i) cache[c][i] = (OP == DECA_SOFTMAX) ? P::kNegInfPair : 0u;
        }
    }

    // every CTA of the cluster must be running before a peer stores into its shared memory; the
    // loads above are already in flight while this barrier completes
    row_cluster_sync();

    if constexpr (OP == DECA_SOFTMAX) {
        uint32_t mx = cache[0][0];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) mx = P::max2(mx, cache[c][i]);
        float2 mf = P::unpack(mx);
        float m = row_reduce<MaxOp>(fmaxf(mf.x, mf.y), red[0], nw, 0, wr, lane);
        m = cluster_combine<MaxOp>(m, cl[0], rank, (uint32_t)cs);
        const float ml = m * kLog2e;

        constexpr bool KEEP_E = (C * VEC <= 128);
        float e[KEEP_E ? C : 1][VEC];
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                float2 f = P::unpack(cache[c][i]);
                const float e0 = ex2_approx(fmaf(f.x, kLog2e, -ml));
                const float e1 = ex2_approx(fmaf(f.y, kLog2e, -ml));
                if constexpr (KEEP_E) e[c][2 * i] = e0, e[c][2 * i + 1] = e1;
                s += e0 + e1;
            }
        s = row_reduce<SumOp>(s, red[1], nw, 0, wr, lane);
        s = cluster_combine<SumOp>(s, cl[1], rank, (uint32_t)cs);
        const float inv = 1.0f / s;
        if (a.stats != nullptr && t == 0 && rank == 0) a.stats[2 * row] = ml, a.stats[2 * row + 1] = inv;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = s0 + (c * tpr + t) * VEC;
            if (col < s1) {
                uint32_t o[WORDS];
#pragma unroll
                for (int i = 0; i < WORDS; ++i) {
                    if constexpr (KEEP_E) {
                        o[i] = P::pack(e[c][2 * i] * inv, e[c][2 * i + 1] * inv);
                    } else {
                        float2 f = P::unpack(cache[c][i]);
                        o[i] = P::pack(ex2_approx(fmaf(f.x, kLog2e, -ml)) * inv,
                                       ex2_approx(fmaf(f.y, kLog2e, -ml)) * inv);
                    }
                }
                store_words<WORDS, HINT>(yrow + (size_t)col * 2, o);
            }
        }
    } else {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                float2 f = P::unpack(cache[c][i]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
        ss = row_reduce<SumOp>(ss, red[0], nw, 0, wr, lane);
        ss = cluster_combine<SumOp>(ss, cl[0], rank, (uint32_t)cs);
        const float r = rsqrtf(ss * a.inv_n + a.eps);
        if (a.stats != nullptr && t == 0 && rank == 0) a.stats[2 * row] = r, a.stats[2 * row + 1] = ss;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = s0 + (c * tpr + t) * VEC;
            if (col < s1) {
                uint32_t wv[WORDS], o[WORDS];
                load_words<WORDS, false>(wv, a.w + (size_t)col * 2);
#pragma unroll
                for (int i = 0; i < WORDS; ++i) {
                    float2 f = P::unpack(cache[c][i]);
                    float2 n = P::unpack(P::pack(f.x * r, f.y * r));
                    float2 g = P::unpack(wv[i]);
                    o[i] = P::pack(n.x * g.x, n.y * g.y);
                }
                store_words<WORDS, HINT>(yrow + (size_t)col * 2, o);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Two-pass mode: U chunks in flight per iteration, row streamed twice.
// ------------------------------------------------------------------------------------------
template <int OP, int DT, int WORDS, int U, bool HINT>
__global__ void rowwise_twopass_kernel(const RowArgs a) {
    using P = Pack16<DT>;
    constexpr int VEC = 2 * WORDS;
    __shared__ float red[2][32];

    const int tpr = a.tpr;
    const int t = threadIdx.x % tpr;
    const int rb = threadIdx.x / tpr;
    const int rpb = blockDim.x / tpr;
    const int lane = threadIdx.x & 31;
    const int wr = t >> 5;
    const int nw = tpr >> 5;
    const int row_warp0 = rb * nw;
    const long long row = (long long)blockIdx.x * rpb + rb;
    const char *xrow = a.x + row * a.N * 2;
    char *yrow = a.y + row * a.N * 2;

    const int span = tpr * VEC;
    const int chunks = (a.N + span - 1) / span;
    const int n_loop = (a.N / span) / U;  // iterations whose U chunks are in bounds for every thread

    float m_run = kNegInf, s_run = 0.f;  // softmax: running max (log2 domain) and sum; rmsnorm: s_run = sum x^2

    // pass 1
    auto pass1 = [&](const uint32_t(&buf)[U][WORDS], int n_valid_chunks) {
        if constexpr (OP == DECA_SOFTMAX) {
            float v[U][VEC];
            float gm = m_run;
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int i = 0; i < WORDS; ++i) {
                    float2 f = P::unpack(buf[u][i]);
                    const bool ok = u < n_valid_chunks;
                    v[u][2 * i] = ok ? f.x * kLog2e : kNegInf * kLog2e;
                    v[u][2 * i + 1] = ok ? f.y * kLog2e : kNegInf * kLog2e;
                    gm = fmaxf(gm, fmaxf(v[u][2 * i], v[u][2 * i + 1]));
                }
            float s = 0.f;
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int i = 0; i < VEC; ++i) s += ex2_approx(v[u][i] - gm);
            s_run = s_run * ex2_approx(m_run - gm) + s;
            m_run = gm;
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int i = 0; i < WORDS; ++i) {
                    float2 f = P::unpack(buf[u][i]);
                    if (u < n_valid_chunks) {
                        s_run = fmaf(f.x, f.x, s_run);
                        s_run = fmaf(f.y, f.y, s_run);
                    }
                }
        }
    };

    for (int g = 0; g < n_loop; ++g) {
        uint32_t buf[U][WORDS];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int col = ((g * U + u) * tpr + t) * VEC;
            load_words<WORDS, false>(buf[u], xrow + (size_t)col * 2);
        }
        pass1(buf, U);
    }
    for (int c = n_loop * U; c < chunks; ++c) {
        uint32_t buf[U][WORDS];
        const int col = (c * tpr + t) * VEC;
        const bool ok = col < a.N;
        if (ok) load_words<WORDS, false>(buf[0], xrow + (size_t)col * 2);
#pragma unroll
        for (int u = 1; u < U; ++u)
#pragma unroll
            for (int i = 0; i < WORDS; ++i) buf[u][i] = 0u;
        if (!ok) {
#pragma unroll
            for (int i = 0; i < WORDS; ++i) buf[0][i] = 0u;
        }
        pass1(buf, ok ? 1 : 0);
    }

    float scale0, scale1;  // softmax: (max * log2e, 1 / sum); rmsnorm: (rsqrt, unused)
    if constexpr (OP == DECA_SOFTMAX) {
        const float m = row_reduce<MaxOp>(m_run, red[0], nw, row_warp0, wr, lane);
        const float s = row_reduce<SumOp>(s_run * ex2_approx(m_run - m), red[1], nw, row_warp0, wr, lane);
        scale0 = m;
        scale1 = 1.0f / s;
    } else {
        const float ss = row_reduce<SumOp>(s_run, red[0], nw, row_warp0, wr, lane);
        scale0 = rsqrtf(ss * a.inv_n + a.eps);
        scale1 = ss;
    }
    if (a.stats != nullptr && t == 0) a.stats[2 * row] = scale0, a.stats[2 * row + 1] = scale1;

    // pass 2
    auto emit = [&](const uint32_t(&xin)[WORDS], int col) {
        uint32_t o[WORDS];
        if constexpr (OP == DECA_SOFTMAX) {
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                float2 f = P::unpack(xin[i]);
                o[i] = P::pack(ex2_approx(fmaf(f.x, kLog2e, -scale0)) * scale1,
                               ex2_approx(fmaf(f.y, kLog2e, -scale0)) * scale1);
            }
        } else {
            uint32_t wv[WORDS];
            load_words<WORDS, false>(wv, a.w + (size_t)col * 2);
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                float2 f = P::unpack(xin[i]);
                float2 n = P::unpack(P::pack(f.x * scale0, f.y * scale0));
                float2 g = P::unpack(wv[i]);
                o[i] = P::pack(n.x * g.x, n.y * g.y);
            }
        }
        store_words<WORDS, HINT>(yrow + (size_t)col * 2, o);
    };

    for (int g = 0; g < n_loop; ++g) {
        uint32_t buf[U][WORDS];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int col = ((g * U + u) * tpr + t) * VEC;
            load_words<WORDS, HINT>(buf[u], xrow + (size_t)col * 2);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) emit(buf[u], ((g * U + u) * tpr + t) * VEC);
    }
    for (int c = n_loop * U; c < chunks; ++c) {
        const int col = (c * tpr + t) * VEC;
        if (col < a.N) {
            uint32_t buf[WORDS];
            load_words<WORDS, HINT>(buf, xrow + (size_t)col * 2);
            emit(buf, col);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Host-side dispatch
// ------------------------------------------------------------------------------------------
// One instantiation per kernel: the register budget of a kernel (hence the largest CTA it can
// run with) is a property of the compiled code, so it is queried once and cached.
template <typename K, K kernel>
int launch_checked(const RowArgs &args, unsigned grid, unsigned threads, cudaStream_t st) {
    static std::atomic<int> max_threads{0};
    int mt = max_threads.load(std::memory_order_relaxed);
    if (mt == 0) {
        cudaFuncAttributes fa;
        cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
        if (e != cudaSuccess) return (int)e;
        mt = fa.maxThreadsPerBlock;
        max_threads.store(mt, std::memory_order_relaxed);
    }
    if ((unsigned)mt < threads) return DECA_ERR_CONFIG;  // register budget
    kernel<<<grid, threads, 0, st>>>(args);
    return (int)cudaGetLastError();
}
#define DECA_LAUNCH(KERNEL, ...) launch_checked<decltype(&KERNEL), &KERNEL>(__VA_ARGS__)

template <int OP, int DT, int WORDS, bool HINT>
int launch_reg(int chunks, const RowArgs &a, unsigned grid, unsigned threads, cudaStream_t st) {
#define DECA_REG_CASE(CN) \
    if (chunks <= CN) return DECA_LAUNCH((rowwise_reg_kernel<OP, DT, WORDS, CN, HINT>), a, grid, threads, st);
    DECA_REG_CASE(1)
    DECA_REG_CASE(2)
    DECA_REG_CASE(3)
    DECA_REG_CASE(4)
    DECA_REG_CASE(5)
    DECA_REG_CASE(6)
    DECA_REG_CASE(7)
    DECA_REG_CASE(8)
    DECA_REG_CASE(10)
    DECA_REG_CASE(12)
    DECA_REG_CASE(16)
    DECA_REG_CASE(20)
    DECA_REG_CASE(24)
    DECA_REG_CASE(32)
#undef DECA_REG_CASE
    return DECA_ERR_CONFIG;
}

template <int OP, int DT, int WORDS, bool HINT>
int launch_twopass(int unroll, const RowArgs &a, unsigned grid, unsigned threads, cudaStream_t st) {
    switch (unroll) {
        case 1: return DECA_LAUNCH((rowwise_twopass_kernel<OP, DT, WORDS, 1, HINT>), a, grid, threads, st);
        case 2: return DECA_LAUNCH((rowwise_twopass_kernel<OP, DT, WORDS, 2, HINT>), a, grid, threads, st);
        case 4: return DECA_LAUNCH((rowwise_twopass_kernel<OP, DT, WORDS, 4, HINT>), a, grid, threads, st);
    }
    return DECA_ERR_CONFIG;
}

// Cluster mode: `grid` clusters of `cs` CTAs, one row each; the slice of a CTA is `slice` elements.
template <int OP, int DT, int WORDS, int C, bool HINT>
int launch_cluster_c(const RowArgs &a, unsigned rows, unsigned threads, int cs, int slice, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * (unsigned)cs), cfg.blockDim = dim3(threads), cfg.dynamicSmemBytes = 0, cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)cs, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, rowwise_cluster_kernel<OP, DT, WORDS, C, HINT>, a, cs, slice);
}

template <int OP, int DT, int WORDS, bool HINT>
int launch_cluster(int chunks, const RowArgs &a, unsigned rows, unsigned threads, int cs, int slice, cudaStream_t st) {
#define DECA_CL_CASE(CN) \
    if (chunks <= CN) return launch_cluster_c<OP, DT, WORDS, CN, HINT>(a, rows, threads, cs, slice, st);
    DECA_CL_CASE(1)
    DECA_CL_CASE(2)
    DECA_CL_CASE(3)
    DECA_CL_CASE(4)
    DECA_CL_CASE(6)
    DECA_CL_CASE(8)
#undef DECA_CL_CASE
    return DECA_ERR_CONFIG;
}

template <int OP, int DT, int WORDS, bool HINT>
int launch_mode(const deca_row_cfg &c, int chunks, const RowArgs &a, unsigned grid, unsigned threads,
                cudaStream_t st) {
    if (c.mode == DECA_ROW_REG) return launch_reg<OP, DT, WORDS, HINT>(chunks, a, grid, threads, st);
    if (c.mode == DECA_ROW_CLUSTER) {
        const int slice = cluster_slice(a.N, c.unroll, c.vec);
        const int span = c.threads_per_row * c.vec;
        return launch_cluster<OP, DT, WORDS, HINT>((slice + span - 1) / span, a, (unsigned)a.M, threads, c.unroll, slice, st);
    }
    return launch_twopass<OP, DT, WORDS, HINT>(c.unroll, a, grid, threads, st);
}

template <int OP, int DT>
int launch_vec(const deca_row_cfg &c, int chunks, const RowArgs &a, unsigned grid, unsigned threads,
               cudaStream_t st) {
    if (c.vec == 8)
        return c.hint ? launch_mode<OP, DT, 4, true>(c, chunks, a, grid, threads, st)
                      : launch_mode<OP, DT, 4, false>(c, chunks, a, grid, threads, st);
    if (c.vec == 4)
        return c.hint ? launch_mode<OP, DT, 2, true>(c, chunks, a, grid, threads, st)
                      : launch_mode<OP, DT, 2, false>(c, chunks, a, grid, threads, st);
    // rows whose length is only a multiple of 2: 4-byte accesses
    return c.hint ? launch_mode<OP, DT, 1, true>(c, chunks, a, grid, threads, st)
                  : launch_mode<OP, DT, 1, false>(c, chunks, a, grid, threads, st);
}

}  // namespace

// bulk-copy pipelined mode (rowwise_tma.cu)
int rowwise_tma_check(int op, int64_t M, int64_t N, const deca_row_cfg &c);
int rowwise_tma_launch(int op, int dtype, const void *X, const void *W, void *Y, int64_t M, int64_t N, float eps,
                       const deca_row_cfg &c, cudaStream_t st);
}  // namespace deca

using namespace deca;

extern "C" int deca_rowwise_check_config(int op, int dtype, int64_t M, int64_t N, const deca_row_cfg *cfg) {
    if (!cfg) return DECA_ERR_NULL;
    if (op != DECA_SOFTMAX && op != DECA_RMSNORM) return DECA_ERR_UNSUPPORTED;
    if (dtype != DECA_F16 && dtype != DECA_BF16) return DECA_ERR_UNSUPPORTED;
    if (M <= 0 || N <= 0 || N > (1ll << 30)) return DECA_ERR_SHAPE;
    if (cfg->mode == DECA_ROW_TMA) return rowwise_tma_check(op, M, N, *cfg);
    if (cfg->mode == DECA_ROW_CLUSTER) {
        // a cluster of `unroll` CTAs (2, 4 or 8) of `threads_per_row` threads per row; a CTA caches its
        // slice of the row in registers (at most 8 chunks per thread)
        if (cfg->vec != 8 && cfg->vec != 4 && cfg->vec != 2) return DECA_ERR_CONFIG;
        if (N % cfg->vec != 0) return DECA_ERR_CONFIG;
        if (cfg->unroll != 2 && cfg->unroll != 4 && cfg->unroll != 8) return DECA_ERR_CONFIG;
        if (cfg->rows_per_block != 1) return DECA_ERR_CONFIG;
        if (cfg->threads_per_row < 32 || cfg->threads_per_row % 32 != 0 || cfg->threads_per_row > 1024) return DECA_ERR_CONFIG;
        if (M * cfg->unroll > 2147483647ll) return DECA_ERR_SHAPE;
        const int64_t slice = cluster_slice((int)N, cfg->unroll, cfg->vec);
        const int64_t span = (int64_t)cfg->threads_per_row * cfg->vec;
        const int64_t chunks = (slice + span - 1) / span;
        if (chunks > 8) return DECA_ERR_CONFIG;
        const int64_t elems = chunks * cfg->vec;
        const int64_t regs = (op == DECA_SOFTMAX ? (elems <= 128 ? elems : elems / 2 + cfg->vec) : elems / 2 + cfg->vec) + 28;
        if (regs > 255 || regs * cfg->threads_per_row > 65536) return DECA_ERR_CONFIG;
        return DECA_OK;
    }
    if (cfg->mode != DECA_ROW_REG && cfg->mode != DECA_ROW_TWOPASS) return DECA_ERR_CONFIG;
    if (cfg->vec != 8 && cfg->vec != 4 && cfg->vec != 2) return DECA_ERR_CONFIG;
    if (N % cfg->vec != 0) return DECA_ERR_CONFIG;
    if (cfg->threads_per_row < 32 || cfg->threads_per_row % 32 != 0) return DECA_ERR_CONFIG;
    if (cfg->rows_per_block < 1) return DECA_ERR_CONFIG;
    if ((int64_t)cfg->threads_per_row * cfg->rows_per_block > 1024) return DECA_ERR_CONFIG;
    if (M % cfg->rows_per_block != 0) return DECA_ERR_CONFIG;
    if (M / cfg->rows_per_block > 2147483647ll) return DECA_ERR_SHAPE;
    const int64_t span = (int64_t)cfg->threads_per_row * cfg->vec;
    const int64_t chunks = (N + span - 1) / span;
    // register estimate per thread (fitted to ptxas -v); one CTA must fit the 64 K register file
    int64_t regs;
    if (cfg->mode == DECA_ROW_REG) {
        if (chunks > 32) return DECA_ERR_CONFIG;
        const int64_t elems = chunks * cfg->vec;
        if (op == DECA_SOFTMAX)
            regs = (elems <= 128 ? elems : elems / 2 + cfg->vec) + 24;
        else
            regs = elems / 2 + cfg->vec + 24;
    } else {
        if (cfg->unroll != 1 && cfg->unroll != 2 && cfg->unroll != 4) return DECA_ERR_CONFIG;
        const int64_t elems = (int64_t)cfg->unroll * cfg->vec;
        regs = elems + elems / 2 + 28;
    }
    if (regs > 255 || regs * cfg->threads_per_row * cfg->rows_per_block > 65536) return DECA_ERR_CONFIG;
    return DECA_OK;
}

extern "C" int deca_rowwise_default_config(int op, int dtype, int64_t M, int64_t N, deca_row_cfg *out) {
    if (!out) return DECA_ERR_NULL;
    if (M <= 0 || N <= 0) return DECA_ERR_SHAPE;
    deca_row_cfg c;
    c.vec = (N % 8 == 0) ? 8 : (N % 4 == 0 ? 4 : 2);
    c.hint = 1;  // every byte is touched once: keep it out of L1 and stream the stores
    c.unroll = 1;
    c.mode = DECA_ROW_REG;
    // about eight chunks (64 elements) per thread and CTAs of 64 threads: measured best or within 1 %
    // of it over the hidden-size grid (1024 ... 8192 columns x 4096 ... 65536 rows); four chunks per
    // thread lose 5 - 13 % on the widest rows, sixteen lose 30 %
    int64_t tpr = 32;
    while (tpr < 1024 && tpr * c.vec * 8 < N) tpr *= 2;
    c.threads_per_row = (int)tpr;
    c.rows_per_block = 1;
    int rpb = 1;
    while (rpb * 2 * c.threads_per_row <= 64 && M % (rpb * 2) == 0) rpb *= 2;
    c.rows_per_block = rpb;
    // Softmax rows beyond 16 Ki elements (vocabulary rows) stream twice even where they would fit the
    // registers of a large CTA: measured 3.96 - 4.71 TB/s against 2.76 - 3.32 for a 1024-thread register
    // CTA at 32000 columns (one such CTA per SM hides no latency), and 4.2 - 4.6 at 128256 columns;
    // the cluster mode measures 3.0 - 3.8 there and stays a tunable.  Within the two-pass mode: 256 threads
    // with two chunks per iteration at 32000 columns (4.9 - 5.2 TB/s on 4096 - 8192 rows; four chunks per
    // iteration leave the row too few iterations: 4.6 - 4.7), 512 threads with four chunks at 128256 columns
    // (4.7; two chunks 4.6, 256 threads 4.3: more rows in flight than L2 holds for the second pass).
    const bool long_softmax = op == DECA_SOFTMAX && N > 16384;
    if (long_softmax || deca_rowwise_check_config(op, dtype, M, N, &c) != DECA_OK) {
        // ... or the row does not fit the register file of one CTA
        c.mode = DECA_ROW_TWOPASS;
        c.threads_per_row = N < 65536 ? 256 : 512;
        c.rows_per_block = 1;
        c.unroll = N < 65536 ? 2 : 4;
        while (c.unroll > 1 && (int64_t)c.threads_per_row * c.vec * c.unroll > N) c.unroll /= 2;
        while (c.threads_per_row > 32 && (int64_t)c.threads_per_row * c.vec > N) c.threads_per_row /= 2;
    }
    *out = c;
    return deca_rowwise_check_config(op, dtype, M, N, out);
}

namespace {

int rowwise_impl(int op, int dtype, const void *X, const void *W, void *Y, float *stats, int64_t M, int64_t N, float eps,
                 const deca_row_cfg *cfg, void *stream) {
    if (!X || !Y || (op == DECA_RMSNORM && !W)) return DECA_ERR_NULL;
    deca_row_cfg c;
    int rc;
    if (cfg) {
        c = *cfg;
        rc = deca_rowwise_check_config(op, dtype, M, N, &c);
    } else {
        rc = deca_rowwise_default_config(op, dtype, M, N, &c);
    }
    if (rc != DECA_OK) return rc;
    if (c.mode == DECA_ROW_TMA) {
        if (stats) return DECA_ERR_UNSUPPORTED;  // the bulk-copy mode has no statistics output
        return rowwise_tma_launch(op, dtype, X, W, Y, M, N, eps, c, static_cast<cudaStream_t>(stream));
    }
    const size_t al = (size_t)c.vec * 2;
    if (!aligned_to(X, al) || !aligned_to(Y, al) || (op == DECA_RMSNORM && !aligned_to(W, al))) return DECA_ERR_ALIGN;

    RowArgs a;
    a.x = static_cast<const char *>(X);
    a.w = static_cast<const char *>(W);
    a.y = static_cast<char *>(Y);
    a.M = M;
    a.N = (int)N;
    a.tpr = c.threads_per_row;
    a.eps = eps;
    a.inv_n = 1.0f / (float)N;
    a.stats = stats;
    const unsigned grid = (unsigned)(M / (c.rows_per_block > 0 ? c.rows_per_block : 1));
    const unsigned threads = (unsigned)(c.threads_per_row * c.rows_per_block);
    const int64_t span = (int64_t)c.threads_per_row * c.vec;
    const int chunks = (int)((N + span - 1) / span);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    if (op == DECA_SOFTMAX)
        return dtype == DECA_F16 ? launch_vec<DECA_SOFTMAX, DECA_F16>(c, chunks, a, grid, threads, st)
                                 : launch_vec<DECA_SOFTMAX, DECA_BF16>(c, chunks, a, grid, threads, st);
    return dtype == DECA_F16 ? launch_vec<DECA_RMSNORM, DECA_F16>(c, chunks, a, grid, threads, st)
                             : launch_vec<DECA_RMSNORM, DECA_BF16>(c, chunks, a, grid, threads, st);
}

}  // namespace

extern "C" int deca_rowwise(int op, int dtype, const void *X, const void *W, void *Y, int64_t M, int64_t N,
                            float eps, const deca_row_cfg *cfg, void *stream) {
    return rowwise_impl(op, dtype, X, W, Y, nullptr, M, N, eps, cfg, stream);
}

extern "C" int deca_rowwise_stats(int op, int dtype, const void *X, const void *W, void *Y, float *stats, int64_t M,
                                  int64_t N, float eps, const deca_row_cfg *cfg, void *stream) {
    if (!stats) return DECA_ERR_NULL;
    if (!aligned_to(stats, 8)) return DECA_ERR_ALIGN;
    return rowwise_impl(op, dtype, X, W, Y, stats, M, N, eps, cfg, stream);
}
