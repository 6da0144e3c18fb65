// Hand-written LSD radix sort of (u64 key, u32 value) pairs for sm_100a, plus tile range detection.
//
// Replaces cub::DeviceRadixSort::SortPairs + identifyTileRanges of the reference
// (rasterization_kernels/diff-gaussian-rasterization-half-gaussian/cuda_rasterizer_hgs/
//  rasterizer_impl.cu:116-138,312-323).
//  * The number of pairs is read from device memory (the instance counter written by the
//    projection kernel), so no host round trip sits between emission and sort; grids are sized
//    from the buffer capacity and blocks loop over 4096-pair chunks.
//  * 8-bit digits, bits [0, 32 + ceil(log2(tiles))) only. Each pass = chunk histograms ->
//    per-digit exclusive scan over chunks -> stable scatter. Ranking inside a chunk is done per
//    warp with match.any (no shared-memory atomics), which also keeps the sort stable.
//  * No kernel waits on another block, so nothing here can spin.
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"

#define SORT_THREADS 256
#define SORT_ITEMS 16
#define SORT_CHUNK (SORT_THREADS * SORT_ITEMS)
#define SORT_WARPS (SORT_THREADS / 32)
#define SORT_WARP_SPAN (32 * SORT_ITEMS)

__device__ __forceinline__ uint32_t sort_count(const uint32_t* counters, uint32_t cap) {
    if (counters[RGS_CNT_OVERFLOW]) return 0u;
    uint32_t n = counters[RGS_CNT_INST];
    return n < cap ? n : cap;
}

// hist[d * nchunks_cap + c] = number of keys of chunk c whose digit is d
__global__ void __launch_bounds__(SORT_THREADS) rgs_sort_hist_kernel(const uint64_t* __restrict__ keys,
                                                                    const uint32_t* __restrict__ counters, uint32_t cap,
                                                                    int shift, uint32_t* __restrict__ hist,
                                                                    uint32_t nchunks_cap) {
    __shared__ uint32_t sh[SORT_WARPS][256];
    const uint32_t n = sort_count(counters, cap);
    const uint32_t nchunks = (n + SORT_CHUNK - 1) / SORT_CHUNK;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        for (int k = threadIdx.x; k < SORT_WARPS * 256; k += SORT_THREADS) (&sh[0][0])[k] = 0;
        __syncthreads();
        const uint32_t base = c * SORT_CHUNK + wid * SORT_WARP_SPAN;
#pragma unroll 4
        for (int r = 0; r < SORT_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t digit = valid ? (uint32_t)((keys[idx] >> shift) & 0xffu) : 0xffffffffu;
            const uint32_t m = __match_any_sync(0xffffffffu, digit);
            if (valid && lane == (__ffs(m) - 1)) sh[wid][digit] += __popc(m);
            __syncwarp();
        }
        __syncthreads();
        uint32_t tot = 0;
#pragma unroll
        for (int w = 0; w < SORT_WARPS; ++w) tot += sh[w][threadIdx.x];
        hist[(size_t)threadIdx.x * nchunks_cap + c] = tot;
        __syncthreads();
    }
}

// One block per digit: in-place exclusive scan of hist[d][0..nchunks), total to totals[d].
__global__ void __launch_bounds__(256) rgs_sort_scan_kernel(uint32_t* __restrict__ hist, uint32_t* __restrict__ totals,
                                                            const uint32_t* __restrict__ counters, uint32_t cap,
                                                            uint32_t nchunks_cap) {
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t carry_s;
    const uint32_t n = sort_count(counters, cap);
    const uint32_t nchunks = (n + SORT_CHUNK - 1) / SORT_CHUNK;
    uint32_t* row = hist + (size_t)blockIdx.x * nchunks_cap;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t start = 0; start < nchunks; start += 256 * 4) {
        const uint32_t i0 = start + threadIdx.x * 4;
        uint32_t v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = (i0 + k < nchunks) ? row[i0 + k] : 0u;
        const uint32_t mine = v[0] + v[1] + v[2] + v[3];
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
        uint32_t run = carry_s + wbase + incl - mine;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (i0 + k < nchunks) row[i0 + k] = run;
            run += v[k];
        }
        __syncthreads();
        if (threadIdx.x == 255) carry_s = run;
        __syncthreads();
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = carry_s;
}

__global__ void __launch_bounds__(SORT_THREADS) rgs_sort_scatter_kernel(
    const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out,
    uint32_t* __restrict__ vals_out, const uint32_t* __restrict__ counters, uint32_t cap, int shift,
    const uint32_t* __restrict__ hist, const uint32_t* __restrict__ totals, uint32_t nchunks_cap) {
    __shared__ uint32_t sh[SORT_WARPS][256];
    __shared__ uint32_t digit_base[256];
    __shared__ uint32_t warp_tot[8];
    const uint32_t n = sort_count(counters, cap);
    const uint32_t nchunks = (n + SORT_CHUNK - 1) / SORT_CHUNK;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;
    // exclusive scan of the 256 digit totals
    {
        const uint32_t t = totals[threadIdx.x];
        uint32_t incl = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t u = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += u;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
        digit_base[threadIdx.x] = wbase + incl - t;
    }
    __syncthreads();
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        for (int k = threadIdx.x; k < SORT_WARPS * 256; k += SORT_THREADS) (&sh[0][0])[k] = 0;
        __syncthreads();
        const uint32_t base = c * SORT_CHUNK + wid * SORT_WARP_SPAN;
        uint64_t key[SORT_ITEMS];
        uint32_t val[SORT_ITEMS];
        uint32_t rank[SORT_ITEMS];
#pragma unroll
        for (int r = 0; r < SORT_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            key[r] = valid ? keys_in[idx] : ~0ull;
            val[r] = valid ? vals_in[idx] : 0u;
        }
#pragma unroll
        for (int r = 0; r < SORT_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t digit = valid ? (uint32_t)((key[r] >> shift) & 0xffu) : 0xffffffffu;
            const uint32_t m = __match_any_sync(0xffffffffu, digit);
            const int leader = __ffs(m) - 1;
            uint32_t pre = 0;
            if (valid && lane == leader) { pre = sh[wid][digit]; sh[wid][digit] = pre + __popc(m); }
            pre = __shfl_sync(0xffffffffu, pre, leader);
            rank[r] = pre + __popc(m & lt_mask);
            __syncwarp();
        }
        __syncthreads();
        {
            const int d = threadIdx.x;
            uint32_t run = hist[(size_t)d * nchunks_cap + c] + digit_base[d];
#pragma unroll
            for (int w = 0; w < SORT_WARPS; ++w) { uint32_t t = sh[w][d]; sh[w][d] = run; run += t; }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < SORT_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            if (idx < n) {
                const uint32_t digit = (uint32_t)((key[r] >> shift) & 0xffu);
                const uint32_t dst = sh[wid][digit] + rank[r];
                if (dst < cap) { keys_out[dst] = key[r]; vals_out[dst] = val[r]; }
            }
        }
        __syncthreads();
    }
}

__global__ void rgs_tile_ranges_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ counters,
                                       uint32_t cap, int2* __restrict__ ranges, uint32_t num_tiles,
                                       const uint32_t* __restrict__ vals_src, uint32_t* __restrict__ vals_dst) {
    const uint32_t n = sort_count(counters, cap);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(keys[i] >> 32);
        if (vals_dst) vals_dst[i] = vals_src[i];
        if (t >= num_tiles) continue;
        if (i == 0 || (uint32_t)(keys[i - 1] >> 32) != t) ranges[t].x = (int)i;
        if (i == n - 1 || (uint32_t)(keys[i + 1] >> 32) != t) ranges[t].y = (int)(i + 1);
    }
}

#ifndef RGS_SORT_KERNELS_ONLY  // the kernels above are also compiled into rgs_noalloc.cu (own namespace)
extern "C" {

// Number of uint32 words of scratch needed for a capacity of cap_inst pairs.
int64_t rgs_cuda_sort_scratch_words(int64_t cap_inst) {
    const int64_t nchunks = (cap_inst + SORT_CHUNK - 1) / SORT_CHUNK;
    return 256 * (nchunks > 0 ? nchunks : 1) + 256;
}

// Sorts (keys, vals) by bits [0, 32 + ceil(log2(num_tiles))) and writes per-tile [start,end).
// The sorted values end up in `vals`; `keys` / `*_tmp` contents are unspecified afterwards.
int rgs_cuda_sort_ranges(uint64_t* keys, uint32_t* vals, uint64_t* keys_tmp, uint32_t* vals_tmp, int64_t cap_inst,
                         const int32_t* counters, int64_t num_tiles, int32_t* ranges, uint32_t* scratch, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t cap = (uint32_t)cap_inst;
    const uint32_t nchunks_cap = (uint32_t)((cap_inst + SORT_CHUNK - 1) / SORT_CHUNK > 0 ? (cap_inst + SORT_CHUNK - 1) / SORT_CHUNK : 1);
    uint32_t* hist = scratch;
    uint32_t* totals = scratch + (size_t)256 * nchunks_cap;
    int tile_bits = 0;
    while ((1ll << tile_bits) < num_tiles) ++tile_bits;
    const int end_bit = 32 + tile_bits;
    const int npass = (end_bit + 7) / 8;
    const unsigned grid = nchunks_cap < (unsigned)(RGS_SMS * 8) ? nchunks_cap : (unsigned)(RGS_SMS * 8);
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
    return (int)cudaGetLastError();
}

}  // extern "C"
#endif  // RGS_SORT_KERNELS_ONLY
