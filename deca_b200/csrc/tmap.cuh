// Host helper: TMA tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda; the function pointer is fetched from the runtime once).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace deca {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 16-bit row-major tensor of up to 3 dimensions, innermost first in `dims` / `box`;
// `strides_bytes` holds the pitch of dimensions 1..rank-1.  Out-of-bounds reads give zero.
// Returns 0 or a positive error code.
inline int make_tmap_16bit(CUtensorMap *out, int dtype, const void *base, int rank, const uint64_t *dims,
                           const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swizzle) {
    // A tuner calls one kernel thousands of times on the same tensors: the last few maps are kept
    // per thread (a map is a pure function of these arguments), which takes the driver call out of
    // the launch path.
    struct Key {
        const void *base;
        uint64_t dims[3], strides[2];
        uint32_t box[3];
        int dtype, rank, swizzle;
    };
    struct Entry {
        Key key;
        CUtensorMap map;
        bool valid;
    };
    constexpr int kEntries = 16;
    static thread_local Entry cache[kEntries] = {};
    static thread_local int next = 0;
    Key key = {};
    key.base = base, key.dtype = dtype, key.rank = rank, key.swizzle = (int)swizzle;
    for (int i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (i > 0) key.strides[i - 1] = strides_bytes[i - 1];
    }
    for (int i = 0; i < kEntries; ++i)
        if (cache[i].valid && memcmp(&cache[i].key, &key, sizeof(Key)) == 0) {
            *out = cache[i].map;
            return 0;
        }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorSymbolNotFound;
    cuuint64_t gdim[3];
    cuuint64_t gstr[2];
    cuuint32_t bx[3], es[3];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
    }
    CUresult r = fn(out, dtype == DECA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    (cuuint32_t)rank, const_cast<void *>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 200000 + (int)r;
    cache[next].key = key, cache[next].map = *out, cache[next].valid = true;
    next = (next + 1) % kEntries;
    return 0;
}

}  // namespace deca
