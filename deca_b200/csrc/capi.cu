// Library-level entry points of the C ABI: version and status text.
#include <mutex>

#include "ptx.cuh"

namespace deca {

__device__ DeviceStatus g_device_status = {};

DeviceStatus *device_status_ptr() {
    // The symbol has one address per device; cache them.
    static std::mutex mu;
    static DeviceStatus *ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<DeviceStatus *>(p);
    }
    return ptrs[dev];
}

}  // namespace deca

extern "C" int deca_last_device_status(int *code, int *where, int *block, int clear) {
    deca::DeviceStatus *p = deca::device_status_ptr();
    if (!p) return (int)cudaErrorUnknown;
    deca::DeviceStatus h;
    cudaError_t e = cudaMemcpy(&h, p, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    if (code) *code = (int)h.code;
    if (where) *where = (int)h.where;
    if (block) *block = (int)h.block;
    if (clear && h.code != 0) {
        e = cudaMemset(p, 0, sizeof(h));
        if (e != cudaSuccess) return (int)e;
    }
    return DECA_OK;
}

extern "C" int deca_device_status_words(unsigned int *out, int n) {
    deca::DeviceStatus *p = deca::device_status_ptr();
    if (!p || !out) return p ? DECA_ERR_NULL : (int)cudaErrorUnknown;
    deca::DeviceStatus h;
    cudaError_t e = cudaMemcpy(&h, p, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    const unsigned int *w = reinterpret_cast<const unsigned int *>(&h);
    for (int i = 0; i < n && i < (int)(sizeof(h) / 4); ++i) out[i] = w[i];
    return DECA_OK;
}

extern "C" const char *deca_version(void) { return "deca_b200 0.1 (sm_100a)"; }

extern "C" const char *deca_status_string(int status) {
    switch (status) {
        case DECA_OK: return "ok";
        case DECA_ERR_NULL: return "a required pointer is null";
        case DECA_ERR_SHAPE: return "non-positive or unsupported extent";
        case DECA_ERR_ALIGN: return "pointer or pitch is not aligned for this kernel";
        case DECA_ERR_CONFIG: return "kernel config rejected";
        case DECA_ERR_UNSUPPORTED: return "op, dtype or mode not built";
        case DECA_ERR_SCRATCH_LIMIT: return "the problem needs more scratch memory than the built-in buffer holds";
        case DECA_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown status";
}
