// Allocation-free variant of the (tile, depth) radix sort: see rgs_noalloc.h for who needs it and the rules.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <mutex>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"
#include "rgs_noalloc.h"

// the sort kernels, compiled a second time into a namespace of their own
#define RGS_SORT_KERNELS_ONLY
namespace rgs_noalloc_detail {
#include "rgs_sort.cu"
}
using namespace rgs_noalloc_detail;

// layout of the scratch array, in bytes
#define NA_CHUNKS ((RGS_NOALLOC_MAX_PAIRS + SORT_CHUNK - 1) / SORT_CHUNK)
#define NA_OFF_KEYS 0
#define NA_OFF_VALS (NA_OFF_KEYS + 8ll * RGS_NOALLOC_MAX_PAIRS)
#define NA_OFF_HIST (NA_OFF_VALS + 4ll * RGS_NOALLOC_MAX_PAIRS)
#define NA_OFF_TOTALS (NA_OFF_HIST + 4ll * 256 * NA_CHUNKS)
#define NA_BYTES (NA_OFF_TOTALS + 4ll * 256)

// In host code this name is only a handle for the runtime, not a device address: the address is looked
// up once per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char rgs_noalloc_scratch[NA_BYTES];

#define NA_MAX_DEVICES 64
static unsigned char* g_scratch_ptr[NA_MAX_DEVICES];
static std::mutex g_mutex;
// one message buffer per calling thread: the pointer handed out by rgs_cuda_noalloc_last_error stays valid and
// unchanged while other threads report errors of their own
static thread_local char g_error[256] = "";

static int na_fail(int code, const char* fmt, long long a, long long b) {
    snprintf(g_error, sizeof(g_error), fmt, a, b);
    return code;
}

extern "C" {

const char* rgs_cuda_noalloc_last_error(void) { return g_error; }

int rgs_cuda_sort_ranges_noalloc(uint64_t* keys, uint32_t* vals, int64_t cap_pairs, const int32_t* counters,
                                 int64_t num_tiles, int32_t* ranges, void* stream) {
    if (cap_pairs < 0 || cap_pairs > RGS_NOALLOC_MAX_PAIRS)
        return na_fail(RGS_NOALLOC_ERR_TOO_LARGE,
                       "rgs_cuda_sort_ranges_noalloc: capacity of %lld pairs exceeds the built-in scratch (%lld pairs)",
                       (long long)cap_pairs, (long long)RGS_NOALLOC_MAX_PAIRS);
    int dev = -1;
    RGS_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NA_MAX_DEVICES)
        return na_fail(RGS_NOALLOC_ERR_SYMBOL, "rgs_cuda_sort_ranges_noalloc: device index %lld out of range (max %lld)",
                       (long long)dev, (long long)NA_MAX_DEVICES);
    unsigned char* base;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (g_scratch_ptr[dev] == nullptr) {  // first call on this device: resolve the device address once
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, rgs_noalloc_scratch);
            if (e != cudaSuccess || p == nullptr) {
                snprintf(g_error, sizeof(g_error), "rgs_cuda_sort_ranges_noalloc: cudaGetSymbolAddress failed on device %d: %s",
                         dev, cudaGetErrorString(e));
                return RGS_NOALLOC_ERR_SYMBOL;
            }
            g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
        }
        base = g_scratch_ptr[dev];
    }
    cudaStream_t st = (cudaStream_t)stream;
    uint64_t* keys_tmp = reinterpret_cast<uint64_t*>(base + NA_OFF_KEYS);
    uint32_t* vals_tmp = reinterpret_cast<uint32_t*>(base + NA_OFF_VALS);
    uint32_t* hist = reinterpret_cast<uint32_t*>(base + NA_OFF_HIST);
    uint32_t* totals = reinterpret_cast<uint32_t*>(base + NA_OFF_TOTALS);
    const uint32_t cap = (uint32_t)cap_pairs;
    const uint32_t nchunks_cap = NA_CHUNKS;  // row stride of the histogram table inside the scratch
    int tile_bits = 0;
    while ((1ll << tile_bits) < num_tiles) ++tile_bits;
    const int npass = (32 + tile_bits + 7) / 8;
    const uint32_t need_chunks = (cap + SORT_CHUNK - 1) / SORT_CHUNK;
    const unsigned grid = need_chunks < 1u ? 1u : (need_chunks < (unsigned)(RGS_SMS * 8) ? need_chunks : (unsigned)(RGS_SMS * 8));
    const uint32_t* cnt = reinterpret_cast<const uint32_t*>(counters);
    uint64_t* kin = keys; uint32_t* vin = vals; uint64_t* kout = keys_tmp; uint32_t* vout = vals_tmp;
    for (int p = 0; p < npass; ++p) {
        rgs_sort_hist_kernel<<<grid, SORT_THREADS, 0, st>>>(kin, cnt, cap, 8 * p, hist, nchunks_cap);
        rgs_sort_scan_kernel<<<256, 256, 0, st>>>(hist, totals, cnt, cap, nchunks_cap);
        rgs_sort_scatter_kernel<<<grid, SORT_THREADS, 0, st>>>(kin, vin, kout, vout, cnt, cap, 8 * p, hist, totals,
                                                               nchunks_cap);
        uint64_t* tk = kin; kin = kout; kout = tk;
        uint32_t* tv = vin; vin = vout; vout = tv;
    }
    RGS_CUDA_CHECK(cudaMemsetAsync(ranges, 0, (size_t)num_tiles * 8, st));
    const bool in_tmp = (vin != vals);
    rgs_tile_ranges_kernel<<<(unsigned)(RGS_SMS * 8), 256, 0, st>>>(kin, cnt, cap, reinterpret_cast<int2*>(ranges), (uint32_t)num_tiles,
                                                    in_tmp ? vin : nullptr, in_tmp ? vals : nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        snprintf(g_error, sizeof(g_error), "rgs_cuda_sort_ranges_noalloc: launch failed: %s", cudaGetErrorString(e));
    return (int)e;
}

}  // extern "C"
