// Row-wise softmax / RMSNorm, bulk-copy pipelined variant (mode DECA_ROW_TMA).
//
// One persistent CTA per SM.  The CTA holds `rows_per_block` independent row groups of
// `threads_per_row` threads.  Each group streams its rows through a private shared-memory
// ring: a whole row arrives with one cp.async.bulk (global -> shared, completion counted on
// an mbarrier), is reduced and transformed from registers exactly as in the register mode of
// rowwise.cu, is written to a two-slot output ring and leaves with one cp.async.bulk
// (shared -> global).  The group refills an input slot as soon as its threads have copied the
// row into registers, so `unroll` rows per group are always in flight whatever the occupancy:
// bytes in flight per SM = rows_per_block * unroll * N * 2, set by the config instead of by
// the register budget.  The arithmetic (and therefore the result) is the one of rowwise.cu.
#include <atomic>

#include "ptx.cuh"

namespace deca {
namespace {

constexpr int kOutSlots = 2;
constexpr int kTmaThreadsMax = 512;
constexpr uint32_t kOffBars = 0;      // up to 64 mbarriers
constexpr uint32_t kOffRed = 1024;    // float red[2][16]
constexpr uint32_t kOffAbort = 1280;  // uint32 abort flag
constexpr uint32_t kOffW = 2048;      // weight row (RMSNorm), then the rings

struct RowTmaArgs {
    const char *x;
    const char *w;
    char *y;
    long long M;
    int N;
    int log2_tpr;
    int ng;         // row groups per CTA
    int stages_in;  // input ring slots per group
    uint32_t row_bytes;
    uint32_t row_pitch;  // row_bytes rounded up to 128
    uint32_t w_bytes;    // 0 for softmax, row_pitch for RMSNorm
    float eps;
    float inv_n;
    DeviceStatus *status;
};

__device__ __forceinline__ void bulk_load_row(uint32_t smem_dst, const void *gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
        "l"(gsrc), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_store_row(void *gdst, uint32_t smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
                 : "memory");
}
// Barrier over the group that also ANDs a per-thread flag, so that all threads of a group take
// the same decision after a bounded wait.
__device__ __forceinline__ bool group_all(bool ok, int group, int threads, int nw) {
    if (nw > 1) {
        uint32_t out;
        asm volatile(
            "{\n\t.reg .pred pi, po;\n\tsetp.ne.u32 pi, %1, 0;\n\tbar.red.and.pred po, %2, %3, pi;\n\t"
            "selp.u32 %0, 1, 0, po;\n\t}"
            : "=r"(out)
            : "r"((uint32_t)ok), "r"(group + 1), "r"(threads)
            : "memory");
        return out != 0;
    }
    return __all_sync(0xFFFFFFFFu, ok) != 0;
}
__device__ __forceinline__ void group_sync(int group, int threads, int nw) {
    if (nw > 1)
        asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(threads) : "memory");
    else
        __syncwarp();
}

template <int OP, int DT, int C>
__global__ void __launch_bounds__(kTmaThreadsMax, 1) rowwise_tma_kernel(const RowTmaArgs a) {
    using P = Pack16<DT>;
    extern __shared__ __align__(128) uint8_t smem[];
    float(*red)[16] = reinterpret_cast<float(*)[16]>(smem + kOffRed);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kOffAbort);

    const int tpr = 1 << a.log2_tpr;
    const int t = threadIdx.x & (tpr - 1);
    const int g = threadIdx.x >> a.log2_tpr;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nw = tpr >> 5;
    const int gw0 = g * nw;  // first warp of the group
    const bool leader = (t == 0);

    const uint32_t bar0 = smem_u32(smem + kOffBars) + (uint32_t)(g * a.stages_in) * 8u;
    uint8_t *ring_in = smem + kOffW + a.w_bytes + (size_t)g * (a.stages_in + kOutSlots) * a.row_pitch;
    uint8_t *ring_out = ring_in + (size_t)a.stages_in * a.row_pitch;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < a.ng * a.stages_in; ++i) mbar_init(smem_u32(smem + kOffBars) + 8u * i, 1);
        fence_barrier_init();
    }
    if constexpr (OP == DECA_RMSNORM) {
        for (uint32_t o = threadIdx.x * 16u; o < a.row_bytes; o += blockDim.x * 16u)
            *reinterpret_cast<uint4 *>(smem + kOffW + o) = *reinterpret_cast<const uint4 *>(a.w + o);
    }
    __syncthreads();

    const long long stride = (long long)gridDim.x * a.ng;
    const long long row0 = (long long)blockIdx.x * a.ng + g;
    long long n_issued = 0, n_done = 0;

    if (leader) {
        for (int s = 0; s < a.stages_in; ++s) {
            const long long r = row0 + s * stride;
            if (r < a.M) {
                mbar_arrive_expect_tx(bar0 + 8u * s, a.row_bytes);
                bulk_load_row(smem_u32(ring_in + (size_t)s * a.row_pitch), a.x + r * a.row_bytes, a.row_bytes,
                              bar0 + 8u * s);
                ++n_issued;
            }
        }
    }

    int s = 0;
    uint32_t phase = 0;
    int oslot = 0;
    for (long long r = row0; r < a.M; r += stride) {
        if (!group_all(mbar_wait(bar0 + 8u * s, phase, abort_flag), g, tpr, nw)) {
            if (leader) {
                *abort_flag = 1;
                report_timeout(a.status, 0x100u);
            }
            break;
        }
        ++n_done;
        const uint8_t *in = ring_in + (size_t)s * a.row_pitch;
        uint32_t cache[C][4];
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = ((c << a.log2_tpr) + t) * 8;
            if (col < a.N) {
                const uint4 v = *reinterpret_cast<const uint4 *>(in + (size_t)col * 2);
                cache[c][0] = v.x, cache[c][1] = v.y, cache[c][2] = v.z, cache[c][3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) cache[c][i] = (OP == DECA_SOFTMAX) ? P::kNegInfPair : 0u;
            }
        }

        // ---- first reduction (row max / sum of squares); its sync also frees the input slot
        float v1;
        if constexpr (OP == DECA_SOFTMAX) {
            uint32_t mx = cache[0][0];
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) mx = P::max2(mx, cache[c][i]);
            const float2 mf = P::unpack(mx);
            v1 = fmaxf(mf.x, mf.y);
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) v1 = fmaxf(v1, __shfl_xor_sync(0xFFFFFFFFu, v1, m));
        } else {
            v1 = 0.f;
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = P::unpack(cache[c][i]);
                    v1 = fmaf(f.x, f.x, v1);
                    v1 = fmaf(f.y, f.y, v1);
                }
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, m);
        }
        if (nw > 1 && lane == 0) red[0][warp] = v1;
        // the output slot written below must have been read by the bulk store issued two rows ago
        if (leader) tma_store_wait_read<kOutSlots - 1>();
        group_sync(g, tpr, nw);
        if (nw > 1) {
            v1 = red[0][gw0];
            for (int i = 1; i < nw; ++i) v1 = (OP == DECA_SOFTMAX) ? fmaxf(v1, red[0][gw0 + i]) : v1 + red[0][gw0 + i];
        }
        // every thread of the group has its part of the row in registers: refill the slot
        if (leader) {
            const long long rn = r + (long long)a.stages_in * stride;
            if (rn < a.M) {
                mbar_arrive_expect_tx(bar0 + 8u * s, a.row_bytes);
                bulk_load_row(smem_u32(ring_in + (size_t)s * a.row_pitch), a.x + rn * a.row_bytes, a.row_bytes,
                              bar0 + 8u * s);
                ++n_issued;
            }
        }

        uint8_t *out = ring_out + (size_t)oslot * a.row_pitch;
        if constexpr (OP == DECA_SOFTMAX) {
            const float ml = v1 * kLog2e;
            constexpr bool KEEP_E = (C <= 8);  // longer rows recompute instead of spilling
            float e[KEEP_E ? C : 1][8];
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = P::unpack(cache[c][i]);
                    const float e0 = ex2_approx(fmaf(f.x, kLog2e, -ml));
                    const float e1 = ex2_approx(fmaf(f.y, kLog2e, -ml));
                    if constexpr (KEEP_E) e[c][2 * i] = e0, e[c][2 * i + 1] = e1;
                    sum += e0 + e1;
                }
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, m);
            if (nw > 1) {
                if (lane == 0) red[1][warp] = sum;
                group_sync(g, tpr, nw);
                sum = red[1][gw0];
                for (int i = 1; i < nw; ++i) sum += red[1][gw0 + i];
            }
            const float inv = 1.0f / sum;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int col = ((c << a.log2_tpr) + t) * 8;
                if (col < a.N) {
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if constexpr (KEEP_E) {
                            o[i] = P::pack(e[c][2 * i] * inv, e[c][2 * i + 1] * inv);
                        } else {
                            const float2 f = P::unpack(cache[c][i]);
                            o[i] = P::pack(ex2_approx(fmaf(f.x, kLog2e, -ml)) * inv,
                                           ex2_approx(fmaf(f.y, kLog2e, -ml)) * inv);
                        }
                    }
                    *reinterpret_cast<uint4 *>(out + (size_t)col * 2) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        } else {
            const float rs = rsqrtf(v1 * a.inv_n + a.eps);
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int col = ((c << a.log2_tpr) + t) * 8;
                if (col < a.N) {
                    const uint4 wv = *reinterpret_cast<const uint4 *>(smem + kOffW + (size_t)col * 2);
                    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = P::unpack(cache[c][i]);
                        // x * r is rounded to the I/O dtype before the weight multiply
                        const float2 n = P::unpack(P::pack(f.x * rs, f.y * rs));
                        const float2 gq = P::unpack(ww[i]);
                        o[i] = P::pack(n.x * gq.x, n.y * gq.y);
                    }
                    *reinterpret_cast<uint4 *>(out + (size_t)col * 2) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        }
        fence_proxy_async_smem();
        group_sync(g, tpr, nw);
        if (leader) {
            bulk_store_row(a.y + r * a.row_bytes, smem_u32(out), a.row_bytes);
            tma_store_commit();
        }
        oslot ^= 1;
        if (++s == a.stages_in) s = 0, phase ^= 1;
    }

    if (leader) {
        // After an aborted loop, loads may still be in flight: wait for them (bounded) before
        // the shared memory goes away.  A normal exit has consumed every load it issued.
        __shared__ uint32_t never_abort;
        for (long long k = n_done; k < n_issued; ++k) {
            const int ss = (int)(k % a.stages_in);
            const uint32_t ph = (uint32_t)((k / a.stages_in) & 1);
            never_abort = 0;
            (void)mbar_wait(bar0 + 8u * ss, ph, &never_abort);
        }
        tma_store_wait<0>();
    }
}

size_t tma_smem_bytes(int op, int ng, int stages_in, uint32_t row_pitch) {
    return kOffW + (op == DECA_RMSNORM ? row_pitch : 0) + (size_t)ng * (stages_in + kOutSlots) * row_pitch;
}

template <typename K, K kernel>
int launch_tma(const RowTmaArgs &args, unsigned grid, unsigned threads, size_t smem, cudaStream_t st) {
    static SmemLimitCache configured;
    if (int rc = ensure_dynamic_smem(kernel, smem, configured)) return rc;
    kernel<<<grid, threads, smem, st>>>(args);
    return (int)cudaGetLastError();
}
#define DECA_LAUNCH_TMA(KERNEL, ...) launch_tma<decltype(&KERNEL), &KERNEL>(__VA_ARGS__)

template <int OP, int DT>
int dispatch_chunks(int chunks, const RowTmaArgs &a, unsigned grid, unsigned threads, size_t smem, cudaStream_t st) {
#define DECA_TMA_CASE(CN) \
    if (chunks <= CN) return DECA_LAUNCH_TMA((rowwise_tma_kernel<OP, DT, CN>), a, grid, threads, smem, st);
    DECA_TMA_CASE(1)
    DECA_TMA_CASE(2)
    DECA_TMA_CASE(3)
    DECA_TMA_CASE(4)
    DECA_TMA_CASE(6)
    DECA_TMA_CASE(8)
    DECA_TMA_CASE(12)
    DECA_TMA_CASE(16)
#undef DECA_TMA_CASE
    return DECA_ERR_CONFIG;
}

}  // namespace

// Host-side rules of the bulk-copy mode; shared with deca_rowwise_check_config.
int rowwise_tma_check(int op, int64_t M, int64_t N, const deca_row_cfg &c) {
    if (c.vec != 8 || N % 8 != 0) return DECA_ERR_CONFIG;
    const int tpr = c.threads_per_row;
    if (tpr < 32 || tpr > kTmaThreadsMax || (tpr & (tpr - 1)) != 0) return DECA_ERR_CONFIG;
    if (c.rows_per_block < 1 || c.rows_per_block > 15 || tpr * c.rows_per_block > kTmaThreadsMax)
        return DECA_ERR_CONFIG;
    if (c.unroll < 1 || c.unroll > 8 || c.rows_per_block * c.unroll > 64) return DECA_ERR_CONFIG;
    const int64_t chunks = (N + (int64_t)tpr * 8 - 1) / ((int64_t)tpr * 8);
    if (chunks > 16) return DECA_ERR_CONFIG;
    const uint32_t pitch = (uint32_t)((N * 2 + 127) / 128 * 128);
    if (tma_smem_bytes(op, c.rows_per_block, c.unroll, pitch) > 232448) return DECA_ERR_CONFIG;
    (void)M;
    return DECA_OK;
}

int rowwise_tma_launch(int op, int dtype, const void *X, const void *W, void *Y, int64_t M, int64_t N, float eps,
                       const deca_row_cfg &c, cudaStream_t st) {
    if (!aligned_to(X, 16) || !aligned_to(Y, 16) || (op == DECA_RMSNORM && !aligned_to(W, 16))) return DECA_ERR_ALIGN;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    static std::atomic<int> cached_sms{0};
    sms = cached_sms.load(std::memory_order_relaxed);
    if (sms == 0) {
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        cached_sms.store(sms, std::memory_order_relaxed);
    }
    RowTmaArgs a;
    a.x = static_cast<const char *>(X);
    a.w = static_cast<const char *>(W);
    a.y = static_cast<char *>(Y);
    a.M = M;
    a.N = (int)N;
    a.log2_tpr = 0;
    while ((1 << a.log2_tpr) < c.threads_per_row) ++a.log2_tpr;
    a.ng = c.rows_per_block;
    a.stages_in = c.unroll;
    a.row_bytes = (uint32_t)(N * 2);
    a.row_pitch = (a.row_bytes + 127u) / 128u * 128u;
    a.w_bytes = (op == DECA_RMSNORM) ? a.row_pitch : 0u;
    a.eps = eps;
    a.inv_n = 1.0f / (float)N;
    a.status = device_status_ptr();
    if (!a.status) return (int)cudaErrorUnknown;
    const size_t smem = tma_smem_bytes(op, a.ng, a.stages_in, a.row_pitch);
    const int64_t groups = (M + a.ng - 1) / a.ng;
    const unsigned grid = (unsigned)(groups < sms ? groups : sms);
    const unsigned threads = (unsigned)(c.threads_per_row * a.ng);
    const int chunks = (int)((N + (int64_t)c.threads_per_row * 8 - 1) / ((int64_t)c.threads_per_row * 8));
    if (op == DECA_SOFTMAX)
        return dtype == DECA_F16 ? dispatch_chunks<DECA_SOFTMAX, DECA_F16>(chunks, a, grid, threads, smem, st)
                                 : dispatch_chunks<DECA_SOFTMAX, DECA_BF16>(chunks, a, grid, threads, smem, st);
    return dtype == DECA_F16 ? dispatch_chunks<DECA_RMSNORM, DECA_F16>(chunks, a, grid, threads, smem, st)
                             : dispatch_chunks<DECA_RMSNORM, DECA_BF16>(chunks, a, grid, threads, smem, st);
}

}  // namespace deca
