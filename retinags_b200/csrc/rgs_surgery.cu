// sm_100a kernels for model surgery: adaptive density control and migration records (see rgs_surgery.h).
//   rgs_densify_classify_kernel  4-bit fate per Gaussian + per-block counts of the four output categories
//   rgs_densify_scan_kernel      exclusive scan of the block counts (one CTA), category totals
//   rgs_densify_gather_kernel    stable compaction: survivors (with moments), clones, split children A, children B
//   rgs_records_pack_kernel      (n,177) row-major records [params, exp_avg, exp_avg_sq] from the column groups
//   rgs_records_unpack_kernel    the inverse, appended at a row offset
// The output of the gather is ordered like the reference's result (kept originals, clones, first children, second
// children; scene/gaussian_nn_module.py:689-751), so that both produce the same model for the same decisions.
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"
#include "rgs_surgery.h"

#define SURGERY_THREADS 256
#define SURGERY_ROWS_PER_THREAD (RGS_SURGERY_BLOCK / SURGERY_THREADS)

__global__ void __launch_bounds__(SURGERY_THREADS) rgs_densify_classify_kernel(
    const RgsConstBlock p, int64_t n, const float* __restrict__ accum, const float* __restrict__ denom,
    const float* __restrict__ maxrad, const __grid_constant__ RgsDensifyCfg cfg, uint8_t* __restrict__ codes,
    int32_t* __restrict__ block_counts, int64_t nblocks) {
    __shared__ int cnt[4];
    for (int64_t b = blockIdx.x; b < nblocks; b += gridDim.x) {
        if (threadIdx.x < 4) cnt[threadIdx.x] = 0;
        __syncthreads();
        int local[4] = {0, 0, 0, 0};
        for (int k = 0; k < SURGERY_ROWS_PER_THREAD; ++k) {
            const int64_t i = b * RGS_SURGERY_BLOCK + k * SURGERY_THREADS + threadIdx.x;
            if (i >= n) continue;
            const float s[3] = {p.scale[3 * i], p.scale[3 * i + 1], p.scale[3 * i + 2]};
            const uint32_t code = rgs_densify_code(cfg, s, p.opacity[i], accum[i], denom[i], maxrad[i]);
            codes[i] = (uint8_t)code;
            for (int c = 0; c < 4; ++c) local[c] += (code >> c) & 1u;
        }
        for (int c = 0; c < 4; ++c) {
            int v = local[c];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((threadIdx.x & 31) == 0 && v) atomicAdd(&cnt[c], v);
        }
        __syncthreads();
        if (threadIdx.x < 4) block_counts[threadIdx.x * nblocks + b] = cnt[threadIdx.x];
        __syncthreads();
    }
}

// one CTA of 1024 threads; per category: block_counts -> exclusive offsets, totals[c] = sum
__global__ void __launch_bounds__(1024) rgs_densify_scan_kernel(int32_t* __restrict__ block_counts, int64_t nblocks,
                                                                int64_t* __restrict__ totals) {
    __shared__ int64_t warp_sum[32];
    __shared__ int64_t carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int c = 0; c < 4; ++c) {
        int32_t* v = block_counts + c * nblocks;
        if (threadIdx.x == 0) carry = 0;
        __syncthreads();
        for (int64_t base = 0; base < nblocks; base += 1024) {
            const int64_t i = base + threadIdx.x;
            const int64_t x = i < nblocks ? v[i] : 0;
            int64_t inc = x;
            for (int o = 1; o < 32; o <<= 1) {
                const int64_t y = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += y;
            }
            if (lane == 31) warp_sum[warp] = inc;
            __syncthreads();
            if (warp == 0) {
                int64_t w = warp_sum[lane], winc = w;
                for (int o = 1; o < 32; o <<= 1) {
                    const int64_t y = __shfl_up_sync(0xffffffffu, winc, o);
                    if (lane >= o) winc += y;
                }
                warp_sum[lane] = winc - w;
            }
            __syncthreads();
            const int64_t excl = carry + warp_sum[warp] + inc - x;
            // offsets inside one category stay below 2^31 rows per buffer, which the 32-bit slot can hold
            if (i < nblocks) v[i] = (int32_t)excl;
            __syncthreads();
            if (threadIdx.x == 1023) carry = excl + x;
            __syncthreads();
        }
        if (threadIdx.x == 0) totals[c] = carry;
        __syncthreads();
    }
}

struct SurgeryItem { int64_t dst; int32_t src_kind; };  // src_kind = (row inside the block) * 4 + kind

__global__ void __launch_bounds__(SURGERY_THREADS) rgs_densify_gather_kernel(
    const RgsConstBlock sp, const RgsConstBlock sm, const RgsConstBlock sv, int64_t n, const uint8_t* __restrict__ codes,
    const int32_t* __restrict__ block_offsets, int64_t nblocks, const int64_t* __restrict__ totals, const RgsBlock dp,
    const RgsBlock dm, const RgsBlock dv, int64_t dcap, uint64_t seed, int* __restrict__ status) {
    __shared__ SurgeryItem items[2 * RGS_SURGERY_BLOCK];
    __shared__ unsigned long long warp_tot[SURGERY_THREADS / 32];
    __shared__ int n_items;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t base_of[4] = {0, totals[0], totals[0] + totals[1], totals[0] + totals[1] + totals[2]};
    if (base_of[3] + totals[3] > dcap) {
        if (threadIdx.x == 0 && blockIdx.x == 0) *status = 1;  // destination too small: nothing is written
        return;
    }
    for (int64_t b = blockIdx.x; b < nblocks; b += gridDim.x) {
        // thread t owns rows 4t..4t+3 of the block, so that a scan over threads is a scan over rows
        uint32_t code[SURGERY_ROWS_PER_THREAD];
        unsigned long long packed = 0;  // five 12-bit counters: categories 0..3 and all items
        for (int k = 0; k < SURGERY_ROWS_PER_THREAD; ++k) {
            const int64_t i = b * RGS_SURGERY_BLOCK + threadIdx.x * SURGERY_ROWS_PER_THREAD + k;
            code[k] = i < n ? codes[i] : 0u;
            for (int c = 0; c < 4; ++c)
                if ((code[k] >> c) & 1u) packed += (1ull << (12 * c)) + (1ull << 48);
        }
        unsigned long long inc = packed;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long y = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += y;
        }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        unsigned long long before = inc - packed;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (threadIdx.x == SURGERY_THREADS - 1) n_items = (int)((before + packed) >> 48);
        int run[4], slot = (int)(before >> 48);
        for (int c = 0; c < 4; ++c) run[c] = (int)((before >> (12 * c)) & 0xfffu);
        for (int k = 0; k < SURGERY_ROWS_PER_THREAD; ++k) {
            for (int c = 0; c < 4; ++c) {
                if (!((code[k] >> c) & 1u)) continue;
                items[slot].dst = base_of[c] + block_offsets[c * nblocks + b] + run[c];
                items[slot].src_kind = (threadIdx.x * SURGERY_ROWS_PER_THREAD + k) * 4 + c;
                ++run[c];
                ++slot;
            }
        }
        __syncthreads();
        const int total = n_items * 15;
        for (int w = threadIdx.x; w < total; w += SURGERY_THREADS) {
            const int it = w / 15, unit = w - it * 15;
            const int64_t o = items[it].dst;
            const int kind = items[it].src_kind & 3;
            const int64_t i = b * RGS_SURGERY_BLOCK + (items[it].src_kind >> 2);
            const bool carry = kind == 0;
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (unit < 12) {
                reinterpret_cast<float4*>(dp.sh + 48 * o)[unit] = reinterpret_cast<const float4*>(sp.sh + 48 * i)[unit];
                reinterpret_cast<float4*>(dm.sh + 48 * o)[unit] = carry ? reinterpret_cast<const float4*>(sm.sh + 48 * i)[unit] : zero4;
                reinterpret_cast<float4*>(dv.sh + 48 * o)[unit] = carry ? reinterpret_cast<const float4*>(sv.sh + 48 * i)[unit] : zero4;
            } else if (unit == 12) {
                float p[3] = {sp.xyz[3 * i], sp.xyz[3 * i + 1], sp.xyz[3 * i + 2]};
                if (kind >= 2) {
                    const float4 q = reinterpret_cast<const float4*>(sp.rot)[i];
                    float nrm[3], R[9];
                    rgs_normal3(seed, i, kind - 2, nrm);
                    const float inv = 1.0f / sqrtf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w);
                    const float qn[4] = {q.x * inv, q.y * inv, q.z * inv, q.w * inv};
                    rgs_quat_to_rot(qn, R);
                    const float e[3] = {expf(sp.scale[3 * i]) * nrm[0], expf(sp.scale[3 * i + 1]) * nrm[1],
                                        expf(sp.scale[3 * i + 2]) * nrm[2]};
                    for (int a = 0; a < 3; ++a) p[a] += R[3 * a] * e[0] + R[3 * a + 1] * e[1] + R[3 * a + 2] * e[2];
                }
                for (int a = 0; a < 3; ++a) {
                    dp.xyz[3 * o + a] = p[a];
                    dm.xyz[3 * o + a] = carry ? sm.xyz[3 * i + a] : 0.f;
                    dv.xyz[3 * o + a] = carry ? sv.xyz[3 * i + a] : 0.f;
                }
            } else if (unit == 13) {
                for (int a = 0; a < 3; ++a) {
                    const float s = sp.scale[3 * i + a];
                    dp.scale[3 * o + a] = kind >= 2 ? logf(expf(s) / 1.6f) : s;
                    dm.scale[3 * o + a] = carry ? sm.scale[3 * i + a] : 0.f;
                    dv.scale[3 * o + a] = carry ? sv.scale[3 * i + a] : 0.f;
                }
                dp.opacity[o] = sp.opacity[i];
                dm.opacity[o] = carry ? sm.opacity[i] : 0.f;
                dv.opacity[o] = carry ? sv.opacity[i] : 0.f;
            } else {
                reinterpret_cast<float4*>(dp.rot)[o] = reinterpret_cast<const float4*>(sp.rot)[i];
                reinterpret_cast<float4*>(dm.rot)[o] = carry ? reinterpret_cast<const float4*>(sm.rot)[i] : zero4;
                reinterpret_cast<float4*>(dv.rot)[o] = carry ? reinterpret_cast<const float4*>(sv.rot)[i] : zero4;
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) rgs_records_pack_kernel(const float* __restrict__ b0, const float* __restrict__ b1,
                                                               const float* __restrict__ b2, int64_t cap,
                                                               const int64_t* __restrict__ index, int64_t row0, int64_t n,
                                                               float* __restrict__ out) {
    const int64_t total = n * 177;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = e / 177;
        const int c = (int)(e - r * 177);
        const int which = c / 59, col = c - which * 59;
        const int64_t i = index ? index[r] : row0 + r;
        const float* src = which == 0 ? b0 : (which == 1 ? b1 : b2);
        out[e] = src[rgs_record_offset(cap, i, col)];
    }
}

__global__ void __launch_bounds__(256) rgs_records_unpack_kernel(const float* __restrict__ rec, int64_t n,
                                                                 float* __restrict__ b0, float* __restrict__ b1,
                                                                 float* __restrict__ b2, int64_t cap, int64_t start) {
    const int64_t total = n * 177;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = e / 177;
        const int c = (int)(e - r * 177);
        const int which = c / 59, col = c - which * 59;
        float* dst = which == 0 ? b0 : (which == 1 ? b1 : b2);
        dst[rgs_record_offset(cap, start + r, col)] = rec[e];
    }
}

static inline unsigned surgery_grid(int64_t work, int per_block) {
    const int64_t want = (work + per_block - 1) / per_block;
    return (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 16 ? RGS_SMS * 16 : want));
}

extern "C" {

// Decide the fate of rows [0,n) and scan it.  block_counts: 4 * ceil(n / RGS_SURGERY_BLOCK) int32 words (holds the
// exclusive per-block offsets afterwards), totals: 4 int64 (survivors, clones, first children, second children).
int rgs_cuda_densify_classify(const float* params, int64_t cap, int64_t n, const float* accum, const float* denom,
                              const float* maxrad, const RgsDensifyCfg* cfg, uint8_t* codes, int32_t* block_counts,
                              int64_t* totals, void* stream) {
    if (n <= 0) return (int)cudaMemsetAsync(totals, 0, 4 * sizeof(int64_t), (cudaStream_t)stream);
    const int64_t nblocks = (n + RGS_SURGERY_BLOCK - 1) / RGS_SURGERY_BLOCK;
    rgs_densify_classify_kernel<<<surgery_grid(nblocks, 1), SURGERY_THREADS, 0, (cudaStream_t)stream>>>(
        rgs_const_block_of(params, cap), n, accum, denom, maxrad, *cfg, codes, block_counts, nblocks);
    rgs_densify_scan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(block_counts, nblocks, totals);
    return (int)cudaGetLastError();
}

// Write the new model into (dparams, dm, dv), buffers of dcap rows.  status (device int, pre-zeroed) becomes 1 when
// dcap is smaller than the new row count; nothing is written then.
int rgs_cuda_densify_gather(const float* params, const float* m, const float* v, int64_t cap, int64_t n,
                            const uint8_t* codes, const int32_t* block_offsets, const int64_t* totals, float* dparams,
                            float* dm, float* dv, int64_t dcap, uint64_t seed, int* status, void* stream) {
    if (n <= 0) return 0;
    const int64_t nblocks = (n + RGS_SURGERY_BLOCK - 1) / RGS_SURGERY_BLOCK;
    rgs_densify_gather_kernel<<<surgery_grid(nblocks, 1), SURGERY_THREADS, 0, (cudaStream_t)stream>>>(
        rgs_const_block_of(params, cap), rgs_const_block_of(m, cap), rgs_const_block_of(v, cap), n, codes, block_offsets,
        nblocks, totals, rgs_block_of(dparams, dcap), rgs_block_of(dm, dcap), rgs_block_of(dv, dcap), dcap, seed, status);
    return (int)cudaGetLastError();
}

// out: (n,177) row-major; rows index[r] (or row0 + r when index is null) of the three buffers.  `out` may be peer-mapped.
int rgs_cuda_records_pack(const float* params, const float* m, const float* v, int64_t cap, const int64_t* index,
                          int64_t row0, int64_t n, float* out, void* stream) {
    if (n <= 0) return 0;
    rgs_records_pack_kernel<<<surgery_grid(n * 177, 256), 256, 0, (cudaStream_t)stream>>>(params, m, v, cap, index, row0, n, out);
    return (int)cudaGetLastError();
}

int rgs_cuda_records_unpack(const float* rec, int64_t n, float* params, float* m, float* v, int64_t cap, int64_t start,
                            void* stream) {
    if (n <= 0) return 0;
    rgs_records_unpack_kernel<<<surgery_grid(n * 177, 256), 256, 0, (cudaStream_t)stream>>>(rec, n, params, m, v, cap, start);
    return (int)cudaGetLastError();
}

}  // extern "C"
