// Shared device/host helpers of the deca_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "deca_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ != 1000)
#error "deca_b200 kernels are written for sm_100a only"
#endif

namespace deca {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegInf = -1e30f;  // finite "minus infinity" of the reference kernels

// Device-reported status of the last kernel that gave up on a bounded wait (0 = none).
// Written by kernels through `report_timeout`, read by deca_last_device_status.
struct DeviceStatus {
    unsigned int code;   // 0 ok, else DECA_ERR_DEVICE_TIMEOUT
    unsigned int where;  // kernel-specific site id
    unsigned int block;  // linear block id that reported first
    unsigned int pad;
    // Diagnostics: every role of block (0, 0) that leaves a bounded wait unsuccessfully stores
    // (site << 16 | loop index) in its own slot, whether or not it was the first to time out.
    unsigned int detail[12];
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16-bit storage types as packed pairs in a 32-bit word.
template <int DT>
struct Pack16;

template <>
struct Pack16<DECA_F16> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2 *>(&w));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
        __half2 h = __hmax2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static constexpr uint32_t kNegInfPair = 0xFC00FC00u;
};

template <>
struct Pack16<DECA_BF16> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
        __nv_bfloat162 h =
            __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&a), *reinterpret_cast<const __nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static constexpr uint32_t kNegInfPair = 0xFF80FF80u;
};

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace deca
