// Library-level entry points of the C ABI: version and status text.
#include <mutex>

#include "ptx.cuh"

namespace deca {

__device__ DeviceStatus g_device_status = {};

constexpr unsigned int kSelfTestSite = 0x7E57u;  // `where` reported by deca_selftest_bounded_wait

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

// Self-test of the bounded-wait path the pipelined kernels rely on, without any of their
// machinery: thread 0 waits on an mbarrier that nothing ever arrives on, with a short limit;
// when the limit passes it raises the CTA's abort flag and reports the timeout exactly as the
// kernels do.  Thread 32 waits on the same barrier with the kernels' default limit and has to
// leave through the abort flag.  Both record how long they waited (microseconds) in the detail
// words 0 and 1.  The kernel returns normally; nothing traps or spins without a bound.
__global__ void bounded_wait_selftest_kernel(DeviceStatus *st, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ uint32_t abort_flag;
    const uint32_t bar_addr = smem_u32(&bar);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(bar_addr, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 || threadIdx.x == 32) {
        const uint64_t t0 = globaltimer_ns();
        const bool done = mbar_wait(bar_addr, 0, &abort_flag, threadIdx.x == 0 ? (uint64_t)limit_ns : kWaitLimitNs);
        const uint64_t waited_us = (globaltimer_ns() - t0) / 1000ull;
        if (!done && threadIdx.x == 0) {
            abort_flag = 1;
            report_timeout(st, kSelfTestSite);
        }
        st->detail[threadIdx.x == 0 ? 0 : 1] = (unsigned int)(waited_us > 0xFFFFFFFFull ? 0xFFFFFFFFull : waited_us);
    }
    __syncthreads();
}

}  // namespace deca

extern "C" int deca_selftest_bounded_wait(unsigned int limit_us, void *stream) {
    if (limit_us < 1 || limit_us > 100000) return DECA_ERR_SHAPE;  // 1 us .. 100 ms
    deca::DeviceStatus *p = deca::device_status_ptr();
    if (!p) return (int)cudaErrorUnknown;
    deca::bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(p, 1000ull * limit_us);
    return (int)cudaGetLastError();
}

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
