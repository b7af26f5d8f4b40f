// Library-level entry points of the C ABI: version and status text.
#include "common.cuh"

extern "C" const char *deca_version(void) { return "deca_b200 0.1 (sm_100a)"; }

extern "C" const char *deca_status_string(int status) {
    switch (status) {
        case DECA_OK: return "ok";
        case DECA_ERR_NULL: return "a required pointer is null";
        case DECA_ERR_SHAPE: return "non-positive or unsupported extent";
        case DECA_ERR_ALIGN: return "pointer or pitch is not aligned for this kernel";
        case DECA_ERR_CONFIG: return "kernel config rejected";
        case DECA_ERR_UNSUPPORTED: return "op, dtype or mode not built";
        case DECA_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown status";
}
