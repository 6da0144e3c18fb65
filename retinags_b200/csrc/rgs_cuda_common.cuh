// Small PTX wrappers used by the sm_100a kernels: mbarriers, bulk asynchronous copies (the TMA
// engine's untiled form), proxy fences, system-scope release/acquire accesses for peer flags.
// Every wait takes an iteration limit and reports expiry instead of spinning forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

__device__ __forceinline__ uint32_t rgs_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void rgs_mbar_init(unsigned long long* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(rgs_smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void rgs_fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void rgs_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void rgs_mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rgs_smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void rgs_mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(rgs_smem_addr(bar)) : "memory");
}

// Bounded wait for the phase with the given parity. Returns false when the limit ran out.
__device__ __forceinline__ bool rgs_mbar_wait(unsigned long long* bar, uint32_t parity, uint32_t limit) {
    const uint32_t addr = rgs_smem_addr(bar);
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// global -> shared bulk copy; dst/src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void rgs_bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     rgs_smem_addr(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(rgs_smem_addr(bar))
                 : "memory");
}

// 16-byte asynchronous copy global -> shared (no register in between, so many can be in flight per thread) and the
// wait for all copies this thread has issued.
__device__ __forceinline__ void rgs_cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(rgs_smem_addr(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void rgs_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void rgs_st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t rgs_ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Number of SMs of the current device, queried once per device: launch grids are sized as a multiple of it.
static inline int64_t rgs_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}
#define RGS_SMS rgs_sm_count()

#define RGS_CUDA_CHECK(expr)                          \
    do {                                              \
        cudaError_t _e = (expr);                      \
        if (_e != cudaSuccess) return (int)_e;        \
    } while (0)
