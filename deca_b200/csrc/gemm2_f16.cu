// 16-bit tensor-core GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] = A[M,K] @ B[K,N], row-major,
// fp32 accumulation in tensor memory.  Same operation and reference counterpart as gemm_f16.cu
// (the mma.sync kernel of src/kernels/gemm_tir.py:123-386); this is the form for large problems.
//
// A cluster of two CTAs owns a (2 BM) x BN output tile, BM = 128 or 256 rows per CTA, BN = 128 or
// 256.  Each CTA holds its BM rows of A and of the accumulator (BM / 128 halves of BN tensor-memory
// columns per accumulator buffer) and BN / 2 of the B columns per 64-deep k block; one thread of
// the even CTA issues MMAs of M = 256 (128 rows from each CTA) x N = BN, and the hardware reads
// the other CTA's operands from that CTA's shared memory.  Against the one-CTA kernel with the
// same rows and columns per CTA this moves a B half less per k block into each SM and reads half
// of B from shared memory per MMA (BM = 256, BN = 256: 48 KB instead of 64 KB and 8 KB instead
// of 12 KB; BM = 128, BN = 256: 32 KB instead of 48 KB and 8 KB instead of 12 KB), which is what
// bounds the narrow one-CTA tiles of small problems.
//   warp 0      TMA producer in both CTAs: own A rows and own B columns into the own ring; the
//               bytes are credited to the even CTA's slot barrier (no multicast).
//   warp 1      tensor-memory allocation (both CTAs); MMA issuer (even CTA): tcgen05.commit
//               arrives on the slot's "empty" barrier and on the "accumulator full" barrier of
//               both CTAs.
//   warps 2-5   epilogue in both CTAs: own 256 x 256 accumulator -> 16 bit -> swizzled staging ->
//               TMA stores; the last tcgen05.ld of a tile arrives on the even CTA's "accumulator
//               empty" barrier (8 arrivals).
// Every mbarrier wait is bounded as in gemm_f16.cu; all paths reach the common teardown (cluster
// barrier, then the pair frees its tensor memory).
#include <atomic>

#include "gemm2.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace deca {
namespace {

constexpr int kBK = 64;
constexpr int kThreads = 192;
constexpr uint32_t kEpiBytes = 4 * 2 * 4096;
constexpr uint32_t kTmemCols = 512;

struct PairArgs {
    int M, N, K;
    int num_kb;
    int gm, gn;  // pair tiles along M and N
    int raster;
    int stages;
    int acc_bufs;
    DeviceStatus *status;
};

__device__ __forceinline__ void pair_tile_coords(int tile, const PairArgs &g, int &m_tile, int &n_tile) {
    const int group_size = g.raster * g.gn;
    const int grp = tile / group_size;
    const int first_m = grp * g.raster;
    const int rows = min(g.raster, g.gm - first_m);
    const int local = tile - grp * group_size;
    m_tile = first_m + local % rows;
    n_tile = local / rows;
}

// HALVES = BM / 128 MMA row halves per CTA, TN = BN.
template <int DT, int HALVES, int TN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const PairArgs g) {
    using P = Pack16<DT>;
    constexpr int kCtaRows = HALVES * 128;  // rows of the tile held by one CTA
    constexpr int kPairRows = 2 * kCtaRows;
    constexpr int kTileN = TN;
    constexpr uint32_t kAStageBytes = kCtaRows * kBK * 2;
    constexpr uint32_t kBStageBytes = (kTileN / 2) * kBK * 2;  // this CTA's half of the columns
    constexpr uint32_t kStageBytes = kAStageBytes + kBStageBytes;
    constexpr uint32_t kAccCols = HALVES * kTileN;  // tensor-memory columns of one accumulator buffer
    constexpr uint32_t kIdesc = make_idesc_f16(DT, false, true, 256, kTileN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw);

    const int stages = g.stages;
    const uint32_t sA = base;
    const uint32_t sB = sA + stages * kAStageBytes;
    const uint32_t sEpi = sB + stages * kBStageBytes;
    const uint32_t sBar = sEpi + kEpiBytes;
    auto full = [&](int i) { return sBar + 8u * i; };
    auto empty = [&](int i) { return sBar + 8u * (stages + i); };
    auto tfull = [&](int i) { return sBar + 8u * (2 * stages + i); };
    auto tempty = [&](int i) { return sBar + 8u * (2 * stages + 2 + i); };
    const uint32_t drain_bar = sBar + 8u * (2 * stages + 4);
    const uint32_t slot_addr = sBar + 8u * (2 * stages + 5);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + (slot_addr - base));
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs, owns the barriers the pair shares
    const int pair_id = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;
    const int total_tiles = g.gm * g.gn;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < stages; ++i) {
            mbar_init(full(i), 1);
            mbar_init(empty(i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tfull(i), 1);
            mbar_init(tempty(i), 8);  // four epilogue warps of each CTA
        }
        mbar_init(drain_bar, 1);
        fence_barrier_init();
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        prefetch_tensormap(&tmC);
    }
    if (warp == 1) {
        tmem_alloc_pair(slot_addr, kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anything arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            long long issued = 0;
            bool ok = true;
            for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
                int mt, nt;
                pair_tile_coords(tile, g, mt, nt);
                const int m0 = mt * kPairRows + (int)rank * kCtaRows;
                const int n0 = nt * kTileN + (int)rank * (kTileN / 2);
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t pair_full = cluster_map(full(s), 0);
                    if (rank == 0) mbar_arrive_expect_tx(full(s), 2 * kStageBytes);  // both CTAs' boxes
                    tma_load_2d_pair(sA + s * kAStageBytes, &tmA, kb * kBK, m0, pair_full);
#pragma unroll
                    for (int b = 0; b < kTileN / 2 / 64; ++b)
                        tma_load_2d_pair(sB + s * kBStageBytes + b * (kBK * 128), &tmB, n0 + b * 64, kb * kBK, pair_full);
                    ++issued;
                    if (++s == stages) s = 0, ph ^= 1u;
                }
            }
            // A wait that ran out lasted a second since this thread's last copy was issued, so no
            // copy of this CTA is still in flight when it leaves.
            if (!ok && *abort_flag == 0) {
                *abort_flag = 1;
                report_timeout(g.status, 0x211u);
            }
            (void)issued;
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA)
        if (lane == 0 && rank == 0) {
            int s = 0, a = 0;
            uint32_t ph = 0, aph = 0;
            bool ok = true;
            for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs) {
                if (!mbar_wait(tempty(a), aph ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)a * kAccCols;
                for (int kb = 0; kb < g.num_kb; ++kb) {
                    if (!mbar_wait(full(s), ph, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = sA + s * kAStageBytes;
                    const uint32_t b_addr = sB + s * kBStageBytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        // A: K-major, 16 k = 32 B inside the swizzled row; B: N-major, this CTA's two
                        // 64-column blocks kBK*128 B apart, 16 k = 2048 B
                        const uint64_t bdesc = make_smem_desc(b_addr, kBK * 128, 1024) + k * (2048 >> 4);
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) {
                            const uint64_t adesc = make_smem_desc(a_addr, 16, 1024) + ((h * (128 * 128) + k * 32) >> 4);
                            umma_f16_ss_pair(d_tmem + h * kTileN, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit_pair(empty(s), 3);  // frees the slot in both CTAs
                    if (++s == stages) s = 0, ph ^= 1u;
                }
                if (!ok) break;
                umma_commit_pair(tfull(a), 3);
                if (++a == g.acc_bufs) a = 0, aph ^= 1u;
            }
            if (!ok) {
                if (*abort_flag == 0) {
                    *abort_flag = 1;
                    report_timeout(g.status, 0x212u);
                }
                __shared__ uint32_t no_abort2;
                no_abort2 = 0;
                umma_commit_pair(drain_bar, 1);
                (void)mbar_wait(drain_bar, 0, &no_abort2);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int q = warp & 3;
        int a = 0;
        uint32_t aph = 0;
        uint32_t panel = 0;
        const uint32_t my_epi = sEpi + q * 8192;
        const uint32_t pair_tempty[2] = {cluster_map(tempty(0), 0), cluster_map(tempty(1), 0)};
        for (int tile = pair_id; tile < total_tiles; tile += n_pairs) {
            int mt, nt;
            pair_tile_coords(tile, g, mt, nt);
            const int m0 = mt * kPairRows + (int)rank * kCtaRows, n0 = nt * kTileN;
            const bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(tfull(a), aph, abort_flag));
            if (!ok) {
                if (lane == 0 && *abort_flag == 0) {
                    *abort_flag = 1;
                    report_timeout(g.status, 0x213u);
                }
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_acc = tmem_base + (uint32_t)a * kAccCols + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int jj = 0; jj < HALVES * (kTileN / 64); ++jj) {
                const int h = jj / (kTileN / 64), j = jj % (kTileN / 64);
                uint32_t r0[32], r1[32];
                tmem_ld_32x32b_x32(t_acc + h * kTileN + j * 64, r0);
                tmem_ld_32x32b_x32(t_acc + h * kTileN + j * 64 + 32, r1);
                tmem_ld_wait();
                if (jj == HALVES * (kTileN / 64) - 1) {
                    // this CTA's half of the accumulator is in registers: tell the issuing CTA
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(pair_tempty[a]);
                }
                uint32_t p[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    p[i] = P::pack(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
                    p[16 + i] = P::pack(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
                }
                const int col0 = n0 + j * 64;
                const int rowq = m0 + h * 128 + q * 32;
                if (col0 >= g.N || rowq >= g.M) continue;  // warp-uniform
                const uint32_t buf = my_epi + (panel & 1u) * 4096u;
                ++panel;
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t dst = buf + lane * 128 + ((c ^ (lane & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[4 * c]), "r"(p[4 * c + 1]),
                                 "r"(p[4 * c + 2]), "r"(p[4 * c + 3])
                                 : "memory");
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tmC, buf, col0, rowq);
                    tma_store_commit();
                }
            }
            if (++a == g.acc_bufs) a = 0, aph ^= 1u;
        }
        if (lane == 0) tma_store_wait_read<0>();  // the writes complete with the grid
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still read its shared or tensor memory
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

size_t pair_smem_bytes(int BM, int BN, int stages) {
    return 1024 + (size_t)stages * ((size_t)BM * kBK * 2 + (size_t)(BN / 2) * kBK * 2) + kEpiBytes + 8 * (2 * (size_t)stages + 8);
}

template <int DT, int HALVES, int TN>
int launch_pair(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC, const PairArgs &g, int64_t tiles,
                size_t smem, cudaStream_t st) {
    // per device: the shared-memory limit set for this instance and how many pairs the device can
    // hold at once with it (SMs pair up inside a GPC)
    static std::atomic<size_t> configured[64];
    static std::atomic<int> max_clusters[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DECA_ERR_UNSUPPORTED;
    if (configured[dev].load(std::memory_order_acquire) < smem) {
        std::lock_guard<std::mutex> lock(smem_limit_mutex());
        if (configured[dev].load(std::memory_order_relaxed) < smem) {
            e = cudaFuncSetAttribute(gemm16_pair_kernel<DT, HALVES, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
            cfg.attrs = &attr, cfg.numAttrs = 1;
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, gemm16_pair_kernel<DT, HALVES, TN>, &cfg);
            if (e != cudaSuccess) return (int)e;
            if (n < 1) return DECA_ERR_UNSUPPORTED;
            max_clusters[dev].store(n, std::memory_order_relaxed);
            configured[dev].store(smem, std::memory_order_release);
        }
    }
    const int64_t max_pairs = max_clusters[dev].load(std::memory_order_relaxed);
    const int64_t pairs = tiles < max_pairs ? tiles : max_pairs;
    gemm16_pair_kernel<DT, HALVES, TN><<<(unsigned)(2 * pairs), kThreads, smem, st>>>(tmA, tmB, tmC, g);
    return (int)cudaGetLastError();
}

template <int DT>
int launch_pair_shape(int BM, int BN, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC,
                      const PairArgs &g, int64_t tiles, size_t smem, cudaStream_t st) {
    if (BM == 256) return BN == 256 ? launch_pair<DT, 2, 256>(tmA, tmB, tmC, g, tiles, smem, st)
                                    : launch_pair<DT, 2, 128>(tmA, tmB, tmC, g, tiles, smem, st);
    return BN == 256 ? launch_pair<DT, 1, 256>(tmA, tmB, tmC, g, tiles, smem, st)
                     : launch_pair<DT, 1, 128>(tmA, tmB, tmC, g, tiles, smem, st);
}

}  // namespace

int gemm16_pair_check(int64_t M, int64_t N, int64_t K, const deca_gemm_cfg *cfg) {
    (void)K;
    if ((cfg->BM != 128 && cfg->BM != 256) || (cfg->BN != 128 && cfg->BN != 256) || cfg->BK != kBK) return DECA_ERR_CONFIG;
    if ((cfg->acc_bufs != 1 && cfg->acc_bufs != 2) || !cfg->epi_smem || cfg->stream_k) return DECA_ERR_CONFIG;
    if (cfg->acc_bufs * (cfg->BM / 128) * cfg->BN > (int)kTmemCols) return DECA_ERR_CONFIG;
    if (cfg->stages < 2 || cfg->stages > 8 || cfg->raster < 1) return DECA_ERR_CONFIG;
    if (pair_smem_bytes(cfg->BM, cfg->BN, cfg->stages) > 232448) return DECA_ERR_CONFIG;
    const int64_t tiles = ((M + 2 * cfg->BM - 1) / (2 * cfg->BM)) * ((N + cfg->BN - 1) / cfg->BN);
    if (tiles > 2147483647ll) return DECA_ERR_SHAPE;
    return DECA_OK;
}

int gemm16_pair_launch(int dtype, const void *A, const void *B, void *C, int64_t M, int64_t N, int64_t K,
                       const deca_gemm_cfg *cfg, void *stream) {
    int rc;
    CUtensorMap tmA, tmB, tmC;
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)K * 2};
        const uint32_t box[2] = {kBK, (uint32_t)cfg->BM};
        if ((rc = make_tmap_16bit(&tmA, dtype, A, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    }
    {
        const uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
        const uint64_t str[1] = {(uint64_t)N * 2};
        const uint32_t box[2] = {64, kBK};
        if ((rc = make_tmap_16bit(&tmB, dtype, B, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    }
    {
        const uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)N * 2};
        const uint32_t box[2] = {64, 32};
        if ((rc = make_tmap_16bit(&tmC, dtype, C, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    }
    PairArgs g;
    g.M = (int)M, g.N = (int)N, g.K = (int)K;
    g.num_kb = (int)((K + kBK - 1) / kBK);
    g.gm = (int)((M + 2 * cfg->BM - 1) / (2 * cfg->BM));
    g.gn = (int)((N + cfg->BN - 1) / cfg->BN);
    g.raster = cfg->raster < g.gm ? cfg->raster : g.gm;
    g.stages = cfg->stages;
    g.acc_bufs = cfg->acc_bufs;
    g.status = device_status_ptr();
    if (!g.status) return (int)cudaErrorUnknown;
    const int64_t tiles = (int64_t)g.gm * g.gn;
    const size_t smem = pair_smem_bytes(cfg->BM, cfg->BN, cfg->stages);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == DECA_F16 ? launch_pair_shape<DECA_F16>(cfg->BM, cfg->BN, tmA, tmB, tmC, g, tiles, smem, st)
                             : launch_pair_shape<DECA_BF16>(cfg->BM, cfg->BN, tmA, tmB, tmC, g, tiles, smem, st);
}

}  // namespace deca
