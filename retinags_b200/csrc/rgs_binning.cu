// Depth-ordered tile binning for sm_100a.
//
// The reference sorts every (tile, splat) instance by a 64-bit (tile | depth) key with
// cub::DeviceRadixSort (rasterizer_impl.cu:298-317): 6 radix passes over ~10^8 pairs of 12 bytes.
// Here the order is produced in two much cheaper steps that give the identical result:
//   1. the *visible splats* (10x fewer than instances) are sorted by depth: 4 passes over 8-byte pairs;
//   2. instances are emitted in that order (a block scan fused into the emission gives every splat its
//      output range, the instance total stays on the device), then ONE stable radix sort on the tile id
//      alone (ceil(log2(tiles)/8) = 2 passes, 8-byte pairs) groups them by tile while keeping the depth
//      order inside each tile, because an LSD radix sort is stable.
// All kernels read their element counts from device memory; no kernel waits on another block.
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"

#include <stdlib.h>
#include <string.h>

#define RGS_BIN_WAIT_LIMIT (1u << 22)

#define BS_THREADS 256
#define BS_WARPS (BS_THREADS / 32)
#define BS_MIN_ITEMS 8   // smallest per-thread item count any variant uses: sizes the histogram table

// number of tiles of the rectangle that hold at least one contributing pixel (all of them without tight_rect)
__device__ __forceinline__ uint32_t count_hit_tiles(const RgsCamera& cam, const RgsSplat& sp, const RgsRect& rc) {
    if (cam.tight_rect < 2) return (uint32_t)((rc.x1 - rc.x0) * (rc.y1 - rc.y0));
    const float bound = rgs_alpha_bound(sp.opacity);
    uint32_t n = 0;
    for (int y = rc.y0; y < rc.y1; ++y)
        for (int x = rc.x0; x < rc.x1; ++x)
            n += rgs_tile_hit(sp.px, sp.py, sp.ca, sp.cb, sp.cc, bound, x, y, cam.W, cam.H) ? 1u : 0u;
    return n;
}

// ---------------------------------------------------------------------------------------------
// projection to slots (no instance emission)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rgs_project_slots_kernel(
    const __grid_constant__ RgsCamera cam, const RgsSegment seg, const int64_t id_base, RgsSplat* __restrict__ splats,
    int32_t* __restrict__ vis_ids, uint32_t* __restrict__ aux, const uint32_t cap_vis, uint32_t* __restrict__ slot_depth,
    uint2* __restrict__ slot_rect, uint32_t* __restrict__ slot_cnt, uint32_t* __restrict__ counters,
    RgsSplatGrad* __restrict__ splat_grads) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    bool ok = false;
    RgsSplat sp;
    RgsRect rc;
    int radius = 0;
    unsigned clamped = 0;
    if (i < seg.count) {
        float p[3] = {seg.xyz[3 * i], seg.xyz[3 * i + 1], seg.xyz[3 * i + 2]};
        float s[3] = {seg.scale[3 * i], seg.scale[3 * i + 1], seg.scale[3 * i + 2]};
        float4 q4 = reinterpret_cast<const float4*>(seg.rot)[i];
        float q[4] = {q4.x, q4.y, q4.z, q4.w};
        ok = rgs_project(cam, p, s, q, seg.opacity[i], seg.sh + 48 * i, sp, rc, radius, clamped);
    }
    __shared__ uint32_t warp_vis[8];
    __shared__ uint32_t base_vis;
    __shared__ int drop;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t vmask = __ballot_sync(0xffffffffu, ok);
    if (lane == 0) warp_vis[wid] = __popc(vmask);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t tv = 0;
        for (int w = 0; w < 8; ++w) { uint32_t v = warp_vis[w]; warp_vis[w] = tv; tv += v; }
        uint32_t bv = 0;
        int d = 0;
        if (tv) {
            bv = atomicAdd(&counters[RGS_CNT_VIS], tv);
            if (bv + tv > cap_vis) { atomicExch(&counters[RGS_CNT_OVERFLOW], 1u); d = 1; }
        }
        base_vis = bv; drop = d;
    }
    __syncthreads();
    if (!ok || drop) return;
    const uint32_t slot = base_vis + warp_vis[wid] + __popc(vmask & ((1u << lane) - 1u));
    float4* dst = reinterpret_cast<float4*>(splats + slot);
    dst[0] = make_float4(sp.px, sp.py, sp.ca, sp.cb);
    dst[1] = make_float4(sp.cc, sp.opacity, sp.r, sp.g);
    dst[2] = make_float4(sp.b, sp.w, sp.depth, sp.pmin);
    vis_ids[slot] = (int32_t)(id_base + i);
    aux[slot] = ((uint32_t)radius << 3) | clamped;
    slot_depth[slot] = __float_as_uint(sp.depth);
    slot_rect[slot] = make_uint2((uint32_t)rc.x0 | ((uint32_t)rc.y0 << 16), (uint32_t)rc.x1 | ((uint32_t)rc.y1 << 16));
    slot_cnt[slot] = count_hit_tiles(cam, sp, rc);
    if (splat_grads) {
        float4* gz = reinterpret_cast<float4*>(splat_grads + slot);
        gz[0] = make_float4(0.f, 0.f, 0.f, 0.f); gz[1] = gz[0]; gz[2] = gz[0];
    }
}

// ---------------------------------------------------------------------------------------------
// two-phase projection: a cheap conservative cull over all Gaussians, then the full projection on survivors
// ---------------------------------------------------------------------------------------------
// Phase 1 reads 24 bytes per Gaussian (position, scale) and keeps a Gaussian unless it is provably culled by
// the exact projection: behind the near plane, or its screen rectangle (centre +- an upper bound of the
// 3-sigma radius) misses the image. The radius bound uses ||J W||_2 <= ||J||_F with the clamped Jacobian of
// rgs_ewa and the largest scale; it is never smaller than the exact radius, so no visible splat is lost.
__device__ __forceinline__ bool rgs_cull_keep(const RgsCamera& cam, float p0, float p1, float p2, float s0, float s1, float s2) {
    const float p[3] = {p0, p1, p2};
    float t[3];
    rgs_view_point(cam.view, p, t);
    if (!(t[2] > RGS_NEAR_Z)) return false;
    // exp is monotonic: the largest activated scale is the activation of the largest raw scale (one exp, same value)
    float smax = fmaxf(s0, fmaxf(s1, s2));
    if (cam.raw_params) smax = expf(smax);
    smax *= cam.scale_modifier;
    const float tz = t[2], itz = 1.0f / tz;
    const float limx = 1.3f * cam.tan_fovx, limy = 1.3f * cam.tan_fovy;
    const float ax = fminf(limx, fabsf(t[0] * itz)), ay = fminf(limy, fabsf(t[1] * itz));
    const float fx = cam.focal_x * itz, fy = cam.focal_y * itz;
    const float jf2 = fx * fx * (1.0f + ax * ax) + fy * fy * (1.0f + ay * ay);
    // +0.3 low-pass, +0.32 because rgs_project floors the eigenvalue discriminant at 0.1 (sqrt(0.1) < 0.32)
    const float rad = ceilf(3.0f * sqrtf(smax * smax * jf2 + 0.62f)) * 1.0001f + 1.0f;
    const float* m = cam.proj;
    const float hx = m[0] * p[0] + m[4] * p[1] + m[8] * p[2] + m[12];
    const float hy = m[1] * p[0] + m[5] * p[1] + m[9] * p[2] + m[13];
    const float hw = m[3] * p[0] + m[7] * p[1] + m[11] * p[2] + m[15];
    const float pw = 1.0f / (hw + 0.0000001f);
    const float px = rgs_ndc2pix(hx * pw, cam.W), py = rgs_ndc2pix(hy * pw, cam.H);
    // same rectangle rule as rgs_project, with the enlarged radius; NaNs fall through as "keep"
    return !(px + rad + RGS_TILE - 1 < 0.0f || px - rad >= (float)(cam.tiles_x * RGS_TILE) ||
             py + rad + RGS_TILE - 1 < 0.0f || py - rad >= (float)(cam.tiles_y * RGS_TILE));
}

// Every thread tests four consecutive Gaussians, read as three 128-bit loads per column group (VEC: both arrays
// start on a 16-byte boundary; otherwise scalar loads), and the block appends its survivors in row order.
#define CULL_ROWS 1024  // rows per block: 256 threads x 4
template <bool VEC>
__global__ void __launch_bounds__(256) rgs_cull_kernel(const __grid_constant__ RgsCamera cam, const float* __restrict__ xyz,
                                                       const float* __restrict__ scale, int64_t count, int64_t id_base,
                                                       uint32_t* __restrict__ cand, uint32_t cap_cand,
                                                       uint32_t* __restrict__ counters) {
    const int64_t i0 = (int64_t)blockIdx.x * CULL_ROWS + 4 * (int64_t)threadIdx.x;
    uint32_t keep = 0;  // bit k: row i0 + k survives
    if (i0 + 3 < count && VEC) {
        const float4* xp = reinterpret_cast<const float4*>(xyz + 3 * i0);
        const float4* sp = reinterpret_cast<const float4*>(scale + 3 * i0);
        const float4 a = xp[0], b = xp[1], c = xp[2], d = sp[0], e = sp[1], f = sp[2];
        keep = (rgs_cull_keep(cam, a.x, a.y, a.z, d.x, d.y, d.z) ? 1u : 0u) |
               (rgs_cull_keep(cam, a.w, b.x, b.y, d.w, e.x, e.y) ? 2u : 0u) |
               (rgs_cull_keep(cam, b.z, b.w, c.x, e.z, e.w, f.x) ? 4u : 0u) |
               (rgs_cull_keep(cam, c.y, c.z, c.w, f.y, f.z, f.w) ? 8u : 0u);
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t i = i0 + k;
            if (i < count && rgs_cull_keep(cam, xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2], scale[3 * i], scale[3 * i + 1],
                                           scale[3 * i + 2]))
                keep |= 1u << k;
        }
    }
    __shared__ uint32_t warp_n[8];
    __shared__ uint32_t base_s;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t mine = __popc(keep);
    uint32_t incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) warp_n[wid] = incl;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t tot = 0;
        for (int w = 0; w < 8; ++w) { uint32_t v = warp_n[w]; warp_n[w] = tot; tot += v; }
        uint32_t b = 0;
        if (tot) {
            b = atomicAdd(&counters[RGS_CNT_CAND], tot);
            if (b + tot > cap_cand) { atomicExch(&counters[RGS_CNT_OVERFLOW], 1u); b = 0xffffffffu; }
        }
        base_s = b;
    }
    __syncthreads();
    if (keep && base_s != 0xffffffffu) {
        uint32_t o = base_s + warp_n[wid] + incl - mine;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (keep & (1u << k)) cand[o++] = (uint32_t)(id_base + i0 + k);
    }
}

struct RgsSegs4 { RgsSegment s[4]; int n; };

// Phase 2: full projection of the candidates (dense: every thread has work).  The 192-byte SH row of every
// candidate is fetched by the bulk-copy engine into shared memory (one cp.async.bulk per thread, completing on an
// mbarrier), so that the ~25 KB a block needs are in flight at once without occupying registers; the small columns
// (position, scale, rotation, opacity) are ordinary loads issued before the wait.
#define PC_THREADS 128
#define PC_ROW 52  // floats per staged row: 48 + 4 of padding (conflict-free 128-bit reads, 16-byte aligned rows)

__global__ void __launch_bounds__(PC_THREADS, 6) rgs_project_cand_kernel(
    const __grid_constant__ RgsCamera cam, const __grid_constant__ RgsSegs4 segs, const uint32_t* __restrict__ cand,
    uint32_t cap_cand, RgsSplat* __restrict__ splats, int32_t* __restrict__ vis_ids, uint32_t* __restrict__ aux,
    const uint32_t cap_vis, uint32_t* __restrict__ slot_depth, uint2* __restrict__ slot_rect, uint32_t* __restrict__ slot_cnt,
    uint32_t* __restrict__ counters, RgsSplatGrad* __restrict__ splat_grads, const int lazy) {
    // lazy: geometry only; the SH rows are neither fetched nor evaluated (rgs_colour_slab_kernel does that later for the
    // splats that have tile instances)
    __shared__ __align__(128) float s_sh[PC_THREADS * PC_ROW];
    __shared__ unsigned long long bar;
    __shared__ uint32_t warp_vis[PC_THREADS / 32];
    __shared__ uint32_t base_vis;
    __shared__ int drop;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint32_t n = counters[RGS_CNT_OVERFLOW] ? 0u : counters[RGS_CNT_CAND];
    if (n > cap_cand) n = cap_cand;
    const uint32_t nblk = (n + PC_THREADS - 1) / PC_THREADS;
    if (threadIdx.x == 0) { rgs_mbar_init(&bar, 1); rgs_fence_mbar_init(); }
    __syncthreads();
    uint32_t round = 0;
    bool failed = false;
    for (uint32_t blk = blockIdx.x; blk < nblk; blk += gridDim.x, ++round) {
        const uint32_t c = blk * PC_THREADS + threadIdx.x;
        const uint32_t valid = n - blk * PC_THREADS < PC_THREADS ? n - blk * PC_THREADS : PC_THREADS;
        bool ok = false;
        RgsSplat sp;
        RgsRect rc;
        int radius = 0;
        unsigned clamped = 0;
        uint32_t gid = 0;
        float p[3] = {0.f, 0.f, 0.f}, s[3] = {0.f, 0.f, 0.f}, q[4] = {1.f, 0.f, 0.f, 0.f}, o = 0.f;
        rgs_fence_proxy_async();  // the rows read in the previous round may be overwritten now
        if (threadIdx.x == 0 && !lazy) rgs_mbar_expect_tx(&bar, valid * 192u);
        if (c < n) {
            gid = cand[c];
            int64_t i = gid;
            int sidx = 0;
            while (sidx < segs.n - 1 && i >= segs.s[sidx].count) { i -= segs.s[sidx].count; ++sidx; }
            const RgsSegment& seg = segs.s[sidx];
            if (!lazy) rgs_bulk_g2s(&s_sh[threadIdx.x * PC_ROW], seg.sh + 48 * i, 192u, &bar);
            p[0] = seg.xyz[3 * i]; p[1] = seg.xyz[3 * i + 1]; p[2] = seg.xyz[3 * i + 2];
            s[0] = seg.scale[3 * i]; s[1] = seg.scale[3 * i + 1]; s[2] = seg.scale[3 * i + 2];
            const float4 q4 = reinterpret_cast<const float4*>(seg.rot)[i];
            q[0] = q4.x; q[1] = q4.y; q[2] = q4.z; q[3] = q4.w;
            o = seg.opacity[i];
        }
        if (!lazy) {
            if (!rgs_mbar_wait(&bar, round & 1u, RGS_BIN_WAIT_LIMIT)) failed = true;
            failed = __syncthreads_or(failed) != 0;
            if (failed) break;  // a wait ran out: give up on the remaining candidates, the host reads the status word
        }
        if (c < n) ok = rgs_project(cam, p, s, q, o, lazy ? nullptr : &s_sh[threadIdx.x * PC_ROW], sp, rc, radius, clamped);
        const uint32_t vmask = __ballot_sync(0xffffffffu, ok);
        if (lane == 0) warp_vis[wid] = __popc(vmask);
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t tv = 0;
            for (int w = 0; w < PC_THREADS / 32; ++w) { uint32_t v = warp_vis[w]; warp_vis[w] = tv; tv += v; }
            uint32_t bv = 0;
            int d = 0;
            if (tv) {
                bv = atomicAdd(&counters[RGS_CNT_VIS], tv);
                if (bv + tv > cap_vis) { atomicExch(&counters[RGS_CNT_OVERFLOW], 1u); d = 1; }
            }
            base_vis = bv; drop = d;
        }
        __syncthreads();
        if (ok && !drop) {
            const uint32_t slot = base_vis + warp_vis[wid] + __popc(vmask & ((1u << lane) - 1u));
            float4* dst = reinterpret_cast<float4*>(splats + slot);
            dst[0] = make_float4(sp.px, sp.py, sp.ca, sp.cb);
            dst[1] = make_float4(sp.cc, sp.opacity, sp.r, sp.g);
            dst[2] = make_float4(sp.b, sp.w, sp.depth, sp.pmin);
            vis_ids[slot] = (int32_t)gid;
            aux[slot] = ((uint32_t)radius << 3) | clamped;
            slot_depth[slot] = __float_as_uint(sp.depth);
            slot_rect[slot] = make_uint2((uint32_t)rc.x0 | ((uint32_t)rc.y0 << 16), (uint32_t)rc.x1 | ((uint32_t)rc.y1 << 16));
            slot_cnt[slot] = count_hit_tiles(cam, sp, rc);
            if (splat_grads) {
                float4* gz = reinterpret_cast<float4*>(splat_grads + slot);
                gz[0] = make_float4(0.f, 0.f, 0.f, 0.f); gz[1] = gz[0]; gz[2] = gz[0];
            }
        }
        __syncthreads();
    }
    // the copies of the abandoned round are not waited for again: the limit is far beyond any legitimate latency
    if (failed && threadIdx.x == 0) atomicExch(&counters[RGS_CNT_STATUS], 1u);
}

// ---------------------------------------------------------------------------------------------
// radix sort of (u32 key, u32 value) pairs; count read from counters[which]
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bs_count(const uint32_t* counters, int which, uint32_t cap) {
    if (counters[RGS_CNT_OVERFLOW]) return 0u;
    const uint32_t n = counters[which];
    return n < cap ? n : cap;
}

// When keys_in is null the key of element i is gathered as key_src[vals_in[i]] / the value is i itself
// (first pass of the depth sort: keys live in slot order, values are the slots).
template <int BS_ITEMS>
__global__ void __launch_bounds__(BS_THREADS) rgs_bs_hist_kernel(const uint32_t* __restrict__ keys,
                                                                const uint32_t* __restrict__ counters, int which,
                                                                uint32_t cap, int shift, uint32_t* __restrict__ hist,
                                                                uint32_t nchunks_cap, int aggregate) {
    constexpr uint32_t BS_CHUNK = BS_THREADS * BS_ITEMS, BS_WARP_SPAN = 32 * BS_ITEMS;
    __shared__ uint32_t sh[BS_WARPS][256];
    const uint32_t n = bs_count(counters, which, cap);
    const uint32_t nchunks = (n + BS_CHUNK - 1) / BS_CHUNK;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        for (int k = threadIdx.x; k < BS_WARPS * 256; k += BS_THREADS) (&sh[0][0])[k] = 0;
        __syncthreads();
        const uint32_t base = c * BS_CHUNK + wid * BS_WARP_SPAN;
#pragma unroll 4
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t digit = valid ? ((keys[idx] >> shift) & 0xffu) : 0xffffffffu;
            if (aggregate) {  // digits repeat inside a warp (high bits of sorted-ish keys): one update per distinct digit
                const uint32_t m = __match_any_sync(0xffffffffu, digit);
                if (valid && lane == (__ffs(m) - 1)) sh[wid][digit] += __popc(m);
                __syncwarp();
            } else if (valid) {  // digits mostly distinct inside a warp: conflict-free shared atomics
                atomicAdd(&sh[wid][digit], 1u);
            }
        }
        __syncthreads();
        uint32_t tot = 0;
#pragma unroll
        for (int w = 0; w < BS_WARPS; ++w) tot += sh[w][threadIdx.x];
        hist[(size_t)threadIdx.x * nchunks_cap + c] = tot;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) rgs_bs_scan_kernel(uint32_t* __restrict__ hist, uint32_t* __restrict__ totals,
                                                          const uint32_t* __restrict__ counters, int which, uint32_t cap,
                                                          uint32_t nchunks_cap, uint32_t chunk) {
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t carry_s;
    const uint32_t n = bs_count(counters, which, cap);
    const uint32_t nchunks = (n + chunk - 1) / chunk;
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

template <int BS_ITEMS>
__global__ void __launch_bounds__(BS_THREADS) rgs_bs_scatter_kernel(
    const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint32_t* __restrict__ keys_out,
    uint32_t* __restrict__ vals_out, const uint32_t* __restrict__ counters, int which, uint32_t cap, int shift,
    const uint32_t* __restrict__ hist, const uint32_t* __restrict__ totals, uint32_t nchunks_cap, int iota_vals) {
    constexpr uint32_t BS_CHUNK = BS_THREADS * BS_ITEMS, BS_WARP_SPAN = 32 * BS_ITEMS;
    __shared__ uint32_t sh[BS_WARPS][256];      // per-warp digit counts -> offsets of the warp inside the digit's run
    __shared__ uint32_t digit_base[256];        // first output index of every digit (over the whole array)
    __shared__ uint32_t local_start[256];       // first staged index of every digit inside this chunk
    __shared__ uint32_t global_start[256];      // output index of the chunk's first element of every digit
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t stage_k[BS_CHUNK], stage_v[BS_CHUNK];
    const uint32_t n = bs_count(counters, which, cap);
    const uint32_t nchunks = (n + BS_CHUNK - 1) / BS_CHUNK;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;
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
        for (int k = threadIdx.x; k < BS_WARPS * 256; k += BS_THREADS) (&sh[0][0])[k] = 0;
        __syncthreads();
        const uint32_t base = c * BS_CHUNK + wid * BS_WARP_SPAN;
        uint32_t key[BS_ITEMS], val[BS_ITEMS], rank[BS_ITEMS];
#pragma unroll
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            key[r] = valid ? keys_in[idx] : 0xffffffffu;
            val[r] = valid ? (iota_vals ? idx : vals_in[idx]) : 0u;
        }
#pragma unroll
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t digit = valid ? ((key[r] >> shift) & 0xffu) : 0xffffffffu;
            const uint32_t m = __match_any_sync(0xffffffffu, digit);
            const int leader = __ffs(m) - 1;
            uint32_t pre = 0;
            if (valid && lane == leader) { pre = sh[wid][digit]; sh[wid][digit] = pre + __popc(m); }
            pre = __shfl_sync(0xffffffffu, pre, leader);
            rank[r] = pre + __popc(m & lt_mask);
            __syncwarp();
        }
        __syncthreads();
        // thread d: offsets of the warps inside digit d's run, the chunk's count of d, and a block scan of the counts
        {
            const int d = threadIdx.x;
            uint32_t run = 0;
#pragma unroll
            for (int w = 0; w < BS_WARPS; ++w) { uint32_t t = sh[w][d]; sh[w][d] = run; run += t; }
            uint32_t incl = run;
#pragma unroll
            for (int dd = 1; dd < 32; dd <<= 1) {
                uint32_t u = __shfl_up_sync(0xffffffffu, incl, dd);
                if (lane >= dd) incl += u;
            }
            if (lane == 31) warp_tot[wid] = incl;
            __syncthreads();
            uint32_t wbase = 0;
            for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
            local_start[d] = wbase + incl - run;
            global_start[d] = hist[(size_t)d * nchunks_cap + c] + digit_base[d];
        }
        __syncthreads();
        // stage the chunk in digit order
#pragma unroll
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            if (idx < n) {
                const uint32_t digit = (key[r] >> shift) & 0xffu;
                const uint32_t pos = local_start[digit] + sh[wid][digit] + rank[r];
                stage_k[pos] = key[r]; stage_v[pos] = val[r];
            }
        }
        __syncthreads();
        // consecutive threads now hold consecutive elements of a digit's run: stores come out in full sectors
        const uint32_t chunk_n = min(BS_CHUNK, n - c * BS_CHUNK);
        for (uint32_t i = threadIdx.x; i < chunk_n; i += BS_THREADS) {
            const uint32_t k = stage_k[i];
            const uint32_t digit = (k >> shift) & 0xffu;
            const uint32_t dst = global_start[digit] + (i - local_start[digit]);
            if (dst < cap) { keys_out[dst] = k; vals_out[dst] = stage_v[i]; }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// single-sweep variant of the same sort: one kernel counts the digits of every pass before the first pass, and the
// scatter of a pass finds where its chunk starts inside every digit's run by looking back at the chunks before it
// (decoupled look-back), instead of a histogram and a scan launch per pass.
//   look-back word of (chunk, digit): count << 2 | state; EMPTY: not there yet, AGG: count of this chunk alone,
//   INCL: count of this chunk and all chunks before it.
// Chunks are handed out by a ticket counter, so every chunk a block waits for belongs to a block that is already
// running and publishes its AGG words without waiting for anybody. The wait is bounded all the same: when it runs
// out, bit 2 of the status word is set, the chunk publishes what it has (so that later chunks do not wait as well),
// and the blocks stop taking tickets; the host raises on the status word and the slower three-kernel sort remains
// available (RGS_SORT=3k).
// ---------------------------------------------------------------------------------------------
#define BS_LB_EMPTY 0u
#define BS_LB_AGG 1u
#define BS_LB_INCL 2u
#define BS_LB_SPINS (1u << 20)
#define BS_STATUS_LOOKBACK 4u
#define BS_SWEEP_MAX_PASSES 4
#define BS_SWEEP_SMALL_WORDS (BS_SWEEP_MAX_PASSES * 256 + 8)  // digit totals of every pass + one ticket per pass

__device__ __forceinline__ uint32_t bs_ld_relaxed(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void bs_st_relaxed(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Digit counts of all passes in one read of the keys (the counts of a digit do not depend on the order of the
// keys, so they hold for every later pass), and the look-back words of the first pass are cleared on the way.
// agg_mask: bit p set when the digits of pass p repeat inside a warp (one shared update per distinct digit).
template <int BS_ITEMS>
__global__ void __launch_bounds__(BS_THREADS) rgs_bs_digits_kernel(const uint32_t* __restrict__ keys,
                                                                  const uint32_t* __restrict__ counters, int which,
                                                                  uint32_t cap, int npass, int agg_mask,
                                                                  uint32_t* __restrict__ totals, uint32_t* __restrict__ lb) {
    constexpr uint32_t BS_CHUNK = BS_THREADS * BS_ITEMS, BS_WARP_SPAN = 32 * BS_ITEMS;
    __shared__ uint32_t sh[BS_SWEEP_MAX_PASSES][256];
    const uint32_t n = bs_count(counters, which, cap);
    const uint32_t nchunks = (n + BS_CHUNK - 1) / BS_CHUNK;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < BS_SWEEP_MAX_PASSES * 256; k += BS_THREADS) (&sh[0][0])[k] = 0;
    __syncthreads();
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        lb[(size_t)c * 256 + threadIdx.x] = 0u;
        const uint32_t base = c * BS_CHUNK + wid * BS_WARP_SPAN;
#pragma unroll 4
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t key = valid ? keys[idx] : 0u;
            for (int p = 0; p < npass; ++p) {
                const uint32_t digit = valid ? ((key >> (8 * p)) & 0xffu) : 0xffffffffu;
                if ((agg_mask >> p) & 1) {
                    const uint32_t m = __match_any_sync(0xffffffffu, digit);
                    if (valid && lane == (__ffs(m) - 1)) atomicAdd(&sh[p][digit], (uint32_t)__popc(m));
                } else if (valid) {
                    atomicAdd(&sh[p][digit], 1u);
                }
            }
        }
    }
    __syncthreads();
    for (int p = 0; p < npass; ++p) {
        const uint32_t v = sh[p][threadIdx.x];
        if (v) atomicAdd(&totals[p * 256 + threadIdx.x], v);
    }
}

template <int BS_ITEMS>
__global__ void __launch_bounds__(BS_THREADS) rgs_bs_sweep_kernel(
    const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint32_t* __restrict__ keys_out,
    uint32_t* __restrict__ vals_out, uint32_t* __restrict__ counters, int which, uint32_t cap, int shift,
    const uint32_t* __restrict__ totals, uint32_t* __restrict__ lb, uint32_t* __restrict__ lb_next,
    uint32_t* __restrict__ ticket, int iota_vals) {
    constexpr uint32_t BS_CHUNK = BS_THREADS * BS_ITEMS, BS_WARP_SPAN = 32 * BS_ITEMS;
    __shared__ uint32_t sh[BS_WARPS][256];
    __shared__ uint32_t digit_base[256];
    __shared__ uint32_t local_start[256];
    __shared__ uint32_t global_start[256];
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t chunk_s, fail_s;
    __shared__ uint32_t stage_k[BS_CHUNK], stage_v[BS_CHUNK];
    const uint32_t n = bs_count(counters, which, cap);
    const uint32_t nchunks = (n + BS_CHUNK - 1) / BS_CHUNK;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;
    {
        const uint32_t t = totals[threadIdx.x];
        uint32_t incl = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t u = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += u;
        }
        if (lane == 31) warp_tot[wid] = incl;
        if (threadIdx.x == 0) fail_s = 0u;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
        digit_base[threadIdx.x] = wbase + incl - t;
    }
    __syncthreads();
    for (;;) {
        if (threadIdx.x == 0) chunk_s = atomicAdd(ticket, 1u);
        for (int k = threadIdx.x; k < BS_WARPS * 256; k += BS_THREADS) (&sh[0][0])[k] = 0;
        __syncthreads();
        const uint32_t c = chunk_s;
        if (c >= nchunks || fail_s) break;  // the same for every thread: both words were written before the barrier
        const uint32_t base = c * BS_CHUNK + wid * BS_WARP_SPAN;
        uint32_t key[BS_ITEMS], val[BS_ITEMS], rank[BS_ITEMS];
#pragma unroll
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            key[r] = valid ? keys_in[idx] : 0xffffffffu;
            val[r] = valid ? (iota_vals ? idx : vals_in[idx]) : 0u;
        }
#pragma unroll
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t digit = valid ? ((key[r] >> shift) & 0xffu) : 0xffffffffu;
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
            uint32_t run = 0;
#pragma unroll
            for (int w = 0; w < BS_WARPS; ++w) { uint32_t t = sh[w][d]; sh[w][d] = run; run += t; }
            // tell the later chunks at once how many elements of digit d this chunk holds
            uint32_t* mine = lb + (size_t)c * 256 + d;
            if (c > 0) bs_st_relaxed(mine, (run << 2) | BS_LB_AGG);
            uint32_t incl = run;
#pragma unroll
            for (int dd = 1; dd < 32; dd <<= 1) {
                uint32_t u = __shfl_up_sync(0xffffffffu, incl, dd);
                if (lane >= dd) incl += u;
            }
            if (lane == 31) warp_tot[wid] = incl;
            __syncthreads();
            uint32_t wbase = 0;
            for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
            local_start[d] = wbase + incl - run;
            // elements of digit d in the chunks before this one
            uint32_t excl = 0;
            bool failed = false;
            for (uint32_t j = c; j > 0 && !failed;) {
                --j;
                const uint32_t* theirs = lb + (size_t)j * 256 + d;
                uint32_t w = bs_ld_relaxed(theirs), spins = 0;
                while ((w & 3u) == BS_LB_EMPTY) {
                    if (++spins > BS_LB_SPINS ||
                        ((spins & 1023u) == 0u && (bs_ld_relaxed(counters + RGS_CNT_STATUS) & BS_STATUS_LOOKBACK))) {
                        failed = true;
                        break;
                    }
                    w = bs_ld_relaxed(theirs);
                }
                if (failed) break;
                excl += w >> 2;
                if ((w & 3u) == BS_LB_INCL) break;
            }
            bs_st_relaxed(mine, ((excl + run) << 2) | BS_LB_INCL);
            lb_next[(size_t)c * 256 + d] = 0u;  // the words the next pass starts from
            if (failed) {
                atomicOr(counters + RGS_CNT_STATUS, BS_STATUS_LOOKBACK);
                fail_s = 1u;
            }
            global_start[d] = digit_base[d] + excl;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < BS_ITEMS; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            if (idx < n) {
                const uint32_t digit = (key[r] >> shift) & 0xffu;
                const uint32_t pos = local_start[digit] + sh[wid][digit] + rank[r];
                stage_k[pos] = key[r]; stage_v[pos] = val[r];
            }
        }
        __syncthreads();
        const uint32_t chunk_n = min(BS_CHUNK, n - c * BS_CHUNK);
        for (uint32_t i = threadIdx.x; i < chunk_n; i += BS_THREADS) {
            const uint32_t k = stage_k[i];
            const uint32_t digit = (k >> shift) & 0xffu;
            const uint32_t dst = global_start[digit] + (i - local_start[digit]);
            if (dst < cap) { keys_out[dst] = k; vals_out[dst] = stage_v[i]; }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// instance emission in depth order: per-segment counts -> scan of segment sums -> emit
// ---------------------------------------------------------------------------------------------
#define EM_SEG 1024  // splats per segment (256 threads x 4)

__device__ __forceinline__ uint32_t rect_count(uint2 r) {
    const uint32_t w = (r.y & 0xffffu) - (r.x & 0xffffu), h = (r.y >> 16) - (r.x >> 16);
    return w * h;
}

__global__ void __launch_bounds__(256) rgs_emit_count_kernel(const uint32_t* __restrict__ order,
                                                             const uint32_t* __restrict__ slot_cnt,
                                                             const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                             uint32_t* __restrict__ seg_sums) {
    __shared__ uint32_t red[8];
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    const uint32_t nseg = (n + EM_SEG - 1) / EM_SEG;
    for (uint32_t s = blockIdx.x; s < nseg; s += gridDim.x) {
        uint32_t sum = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t i = s * EM_SEG + k * 256 + threadIdx.x;
            if (i < n) sum += slot_cnt[order[i]];
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t t = 0;
            for (int w = 0; w < 8; ++w) t += red[w];
            seg_sums[s] = t;
        }
        __syncthreads();
    }
}

// single block: exclusive scan of the segment sums in place; total -> counters[CNT_INST], overflow flag.
__global__ void __launch_bounds__(1024) rgs_emit_scan_kernel(uint32_t* __restrict__ seg_sums, uint32_t* __restrict__ counters,
                                                             uint32_t cap_vis, uint32_t cap_inst) {
    __shared__ uint32_t warp_tot[32];
    __shared__ unsigned long long carry_s;  // 64-bit so that a total beyond 2^32 is seen as an overflow, not a wrap
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    const uint32_t nseg = (n + EM_SEG - 1) / EM_SEG;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    unsigned long long total64 = 0;
    for (uint32_t start = 0; start < nseg; start += 1024) {
        const uint32_t i = start + threadIdx.x;
        const uint32_t v = i < nseg ? seg_sums[i] : 0u;
        uint32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
        const uint32_t excl = (uint32_t)carry_s + wbase + incl - v;
        if (i < nseg) seg_sums[i] = excl;
        __syncthreads();
        if (threadIdx.x == 1023) { total64 = carry_s + wbase + incl; carry_s = total64; }
        __syncthreads();
    }
    if (threadIdx.x == 1023) {
        const unsigned long long tot = nseg ? total64 : 0ull;
        counters[RGS_CNT_INST] = tot > 0xffffffffull ? 0xffffffffu : (uint32_t)tot;
        if (tot > (unsigned long long)cap_inst) atomicExch(&counters[RGS_CNT_OVERFLOW], 1u);
    }
}

// Emission: a block scans the tile counts of its 1024 depth-ordered splats, parks (slot, rect, base) in
// shared memory, then every warp walks its 128 splats and the 32 lanes test/write one splat's tiles together
// (consecutive lanes -> consecutive instances: coalesced stores instead of one long loop per thread).
__global__ void __launch_bounds__(256) rgs_emit_kernel(const __grid_constant__ RgsCamera cam, const uint32_t* __restrict__ order,
                                                       const uint2* __restrict__ slot_rect, const uint32_t* __restrict__ slot_cnt,
                                                       const RgsSplat* __restrict__ splats,
                                                       const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                       const uint32_t* __restrict__ seg_excl, uint32_t* __restrict__ tile_keys,
                                                       uint32_t* __restrict__ vals, uint32_t cap_inst) {
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t s_slot[EM_SEG], s_base[EM_SEG];
    __shared__ uint2 s_rect[EM_SEG];
    // an overflow flagged by the scan kernel zeroes the count here, so nothing is written
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    const uint32_t nseg = (n + EM_SEG - 1) / EM_SEG;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int tiles_x = cam.tiles_x;
    for (uint32_t s = blockIdx.x; s < nseg; s += gridDim.x) {
        // thread t owns elements s*1024 + 4t .. 4t+3 (consecutive, so the scan order is the element order)
        uint32_t slot[4], cnt[4];
        uint2 rect[4];
        uint32_t mine = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t i = s * EM_SEG + threadIdx.x * 4 + k;
            if (i < n) { slot[k] = order[i]; rect[k] = slot_rect[slot[k]]; cnt[k] = slot_cnt[slot[k]]; }
            else { slot[k] = 0; rect[k] = make_uint2(0, 0); cnt[k] = 0; }
            mine += cnt[k];
        }
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
        uint32_t base = seg_excl[s] + wbase + incl - mine;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int e = threadIdx.x * 4 + k;
            s_slot[e] = slot[k]; s_base[e] = base;
            s_rect[e] = cnt[k] ? rect[k] : make_uint2(0, 0);  // nothing to emit -> empty rectangle
            base += cnt[k];
        }
        __syncthreads();
        for (int j = 0; j < EM_SEG / 8; ++j) {
            const int e = wid * (EM_SEG / 8) + j;
            const uint2 r = s_rect[e];
            const uint32_t c = rect_count(r);
            if (c == 0) continue;
            const int x0 = r.x & 0xffff, y0 = r.x >> 16, w = (int)(r.y & 0xffff) - x0;
            const uint32_t sl = s_slot[e];
            uint32_t o = s_base[e];
            if (cam.tight_rect < 2) {
                for (uint32_t t = lane; t < c; t += 32) {
                    const uint32_t ty = t / (uint32_t)w, tx = t - ty * (uint32_t)w;
                    if (o + t < cap_inst) { tile_keys[o + t] = (uint32_t)((y0 + (int)ty) * tiles_x + x0 + (int)tx); vals[o + t] = sl; }
                }
                continue;
            }
            // same test, same inputs as count_hit_tiles: the record written by the projection kernel
            const float4 q0 = reinterpret_cast<const float4*>(splats + sl)[0];
            const float2 q1 = reinterpret_cast<const float2*>(splats + sl)[2];
            const float bound = rgs_alpha_bound(q1.y);
            for (uint32_t t0 = 0; t0 < c; t0 += 32) {
                const uint32_t t = t0 + lane;
                bool hit = false;
                uint32_t key = 0;
                if (t < c) {
                    const uint32_t ty = t / (uint32_t)w, tx = t - ty * (uint32_t)w;
                    hit = rgs_tile_hit(q0.x, q0.y, q0.z, q0.w, q1.x, bound, x0 + (int)tx, y0 + (int)ty, cam.W, cam.H);
                    key = (uint32_t)((y0 + (int)ty) * tiles_x + x0 + (int)tx);
                }
                const uint32_t m = __ballot_sync(0xffffffffu, hit);
                if (hit) {
                    const uint32_t dst = o + __popc(m & ((1u << lane) - 1u));
                    if (dst < cap_inst) { tile_keys[dst] = key; vals[dst] = sl; }
                }
                o += __popc(m);
            }
        }
        __syncthreads();
    }
}

__global__ void rgs_bs_tile_ranges_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ counters,
                                          uint32_t cap, int2* __restrict__ ranges, uint32_t num_tiles,
                                          const uint32_t* __restrict__ vals_src, uint32_t* __restrict__ vals_dst) {
    const uint32_t n = bs_count(counters, RGS_CNT_INST, cap);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint32_t t = keys[i];
        if (vals_dst) vals_dst[i] = vals_src[i];
        if (t >= num_tiles) continue;
        if (i == 0 || keys[i - 1] != t) ranges[t].x = (int)i;
        if (i == n - 1 || keys[i + 1] != t) ranges[t].y = (int)(i + 1);
    }
}

// Tile ranges by binary search in the sorted tile keys: one thread per tile, ~2 log2(n) probes, instead of a pass
// over all keys (340 MB per view at 85 M instances).
// `which`: counter word holding the number of sorted keys; `base` is added to the indices written (the keys of a
// depth slab start `base` elements into the instance buffers).
__global__ void __launch_bounds__(128) rgs_bs_tile_ranges_search_kernel(const uint32_t* __restrict__ keys,
                                                                        const uint32_t* __restrict__ counters, uint32_t cap,
                                                                        int2* __restrict__ ranges, uint32_t num_tiles,
                                                                        int which, uint32_t base) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= num_tiles) return;
    const uint32_t n = bs_count(counters, which, cap);
    uint32_t lo = 0, hi = n;  // first index with key >= t
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (keys[mid] < t) lo = mid + 1; else hi = mid;
    }
    const uint32_t first = lo;
    hi = n;                   // first index with key > t
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (keys[mid] <= t) lo = mid + 1; else hi = mid;
    }
    ranges[t] = lo > first ? make_int2((int)(base + first), (int)(base + lo)) : make_int2(0, 0);
}

// ---------------------------------------------------------------------------------------------
// Two-slab binning. In a dense scene most tiles are saturated (every pixel below the transmittance threshold) after
// the nearest splats, yet the single-pass pipeline emits and sorts the instances of all splats. Here the depth-ordered
// splats are cut in two slabs: the instances of the near slab are emitted, sorted and blended first; the blend marks
// the tiles in which every pixel is done, and the far slab emits instances only for the other tiles. The count of
// such tiles inside a splat's rectangle is four reads of a summed-area table, so splats over saturated regions cost
// a few loads and no instance. Nothing that could change a pixel is skipped: the output is bit-identical.
// ---------------------------------------------------------------------------------------------
// segments [s0,s1) of EM_SEG depth-ordered splats that belong to `slab` (0 = near, 1 = far); frac256/256 of the
// splats (rounded down to whole segments) form the near slab
__device__ __forceinline__ void slab_segments(uint32_t n, uint32_t frac256, int slab, uint32_t& s0, uint32_t& s1) {
    const uint32_t nseg = (n + EM_SEG - 1) / EM_SEG;
    uint32_t split = (uint32_t)(((unsigned long long)n * frac256) >> 8) / EM_SEG;
    if (split > nseg) split = nseg;
    s0 = slab == 0 ? 0u : split;
    s1 = slab == 0 ? split : nseg;
}

// Colours of the splats of one slab that have tile instances (slot_cnt != 0 after the filter): the SH rows (192 bytes
// per Gaussian, by far the largest part of what the projection reads) are fetched for those alone. In a dense scene
// most visible splats lie behind finished tiles and never get here.
__global__ void __launch_bounds__(128) rgs_colour_slab_kernel(const __grid_constant__ RgsCamera cam,
                                                              const __grid_constant__ RgsSegs4 segs,
                                                              const uint32_t* __restrict__ order,
                                                              const uint32_t* __restrict__ slot_cnt,
                                                              const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                              uint32_t frac256, int slab, RgsSplat* __restrict__ splats,
                                                              const int32_t* __restrict__ vis_ids, uint32_t* __restrict__ aux) {
    // A warp looks at 32 depth-ordered positions at a time. The SH rows of the splats among them that have instances are
    // fetched by the whole warp, one row after the other: lanes 0..11 copy the twelve 128-bit words of a row (one
    // coalesced 192-byte request per row; asynchronous copies, so all rows of the batch are in flight together) into
    // the owner lane's padded row in shared memory; every owner then evaluates its colour from there with the
    // arithmetic of the projection.
    __shared__ __align__(16) float s_sh[4][32][PC_ROW];
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    uint32_t s0, s1;
    slab_segments(n, frac256, slab, s0, s1);
    const uint32_t begin = s0 * EM_SEG, end = s1 * EM_SEG < n ? s1 * EM_SEG : n;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i0 = begin + warp * 32; i0 < end; i0 += nwarps * 32) {
        const uint32_t i = i0 + lane;
        bool act = false;
        uint32_t slot = 0;
        const float* sh_row = nullptr;
        float p[3] = {0.f, 0.f, 0.f};
        if (i < end) {
            slot = order[i];
            if (slot_cnt[slot] != 0) {
                int64_t id = vis_ids[slot];
                int sidx = 0;
                while (sidx < segs.n - 1 && id >= segs.s[sidx].count) { id -= segs.s[sidx].count; ++sidx; }
                const RgsSegment& seg = segs.s[sidx];
                if (id >= 0 && id < seg.count) {
                    act = true;
                    sh_row = seg.sh + 48 * id;
                    p[0] = seg.xyz[3 * id]; p[1] = seg.xyz[3 * id + 1]; p[2] = seg.xyz[3 * id + 2];
                }
            }
        }
        uint32_t m = __ballot_sync(0xffffffffu, act);
        if (m == 0) continue;
        const unsigned long long mine = (unsigned long long)(uintptr_t)sh_row;
        while (m) {
            const int a = __ffs(m) - 1;
            m &= m - 1;
            const float4* src = reinterpret_cast<const float4*>((uintptr_t)__shfl_sync(0xffffffffu, mine, a));
            if (lane < 12) rgs_cp_async16(&s_sh[wid][a][4 * lane], src + lane);
        }
        rgs_cp_async_wait_all();
        __syncwarp();
        if (act) {
            float r, g, b;
            unsigned clamped;
            rgs_splat_colour(cam, p, &s_sh[wid][lane][0], r, g, b, clamped);
            float* rec = reinterpret_cast<float*>(splats + slot);
            rec[6] = r; rec[7] = g; rec[8] = b;
            aux[slot] = (aux[slot] & ~7u) | clamped;
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(256) rgs_slab_count_kernel(const uint32_t* __restrict__ order,
                                                             const uint32_t* __restrict__ slot_cnt,
                                                             const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                             uint32_t frac256, int slab, uint32_t* __restrict__ seg_sums) {
    __shared__ uint32_t red[8];
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    uint32_t s0, s1;
    slab_segments(n, frac256, slab, s0, s1);
    for (uint32_t s = s0 + blockIdx.x; s < s1; s += gridDim.x) {
        uint32_t sum = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t i = s * EM_SEG + k * 256 + threadIdx.x;
            if (i < n) sum += slot_cnt[order[i]];
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t t = 0;
            for (int w = 0; w < 8; ++w) t += red[w];
            seg_sums[s] = t;
        }
        __syncthreads();
    }
}

// one CTA: exclusive scan of seg_sums[s0..s1) in place (relative to the slab's first instance); the slab's total goes
// to counters[which], exceeding region_cap raises the overflow flag
__global__ void __launch_bounds__(1024) rgs_slab_scan_kernel(uint32_t* __restrict__ seg_sums, uint32_t* __restrict__ counters,
                                                             uint32_t cap_vis, uint32_t frac256, int slab, int which,
                                                             uint32_t region_cap) {
    __shared__ uint32_t warp_tot[32];
    __shared__ unsigned long long carry_s;
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    uint32_t s0, s1;
    slab_segments(n, frac256, slab, s0, s1);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t start = s0; start < s1; start += 1024) {
        const uint32_t i = start + threadIdx.x;
        const uint32_t v = i < s1 ? seg_sums[i] : 0u;
        uint32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
        const unsigned long long excl = carry_s + wbase + incl - v;
        if (i < s1) seg_sums[i] = excl > 0xffffffffull ? 0xffffffffu : (uint32_t)excl;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const unsigned long long tot = carry_s;
        counters[which] = tot > 0xffffffffull ? 0xffffffffu : (uint32_t)tot;
        if (tot > (unsigned long long)region_cap) atomicExch(&counters[RGS_CNT_OVERFLOW], 1u);
    }
}

// Emission of one slab. tile_keys / vals point at the slab's region; with tile_done only tiles that are not marked
// are written (slot_cnt holds exactly that count for the slab's splats).
__global__ void __launch_bounds__(256) rgs_slab_emit_kernel(const __grid_constant__ RgsCamera cam,
                                                            const uint32_t* __restrict__ order,
                                                            const uint2* __restrict__ slot_rect,
                                                            const uint32_t* __restrict__ slot_cnt,
                                                            const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                            uint32_t frac256, int slab, const uint32_t* __restrict__ seg_excl,
                                                            uint32_t* __restrict__ tile_keys, uint32_t* __restrict__ vals,
                                                            uint32_t region_cap, const uint8_t* __restrict__ tile_done) {
    __shared__ uint32_t warp_tot[8], warp_nz[8];
    __shared__ uint32_t s_slot[EM_SEG], s_base[EM_SEG];
    __shared__ uint2 s_rect[EM_SEG];
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);  // 0 after an overflow: nothing is written
    uint32_t s0, s1;
    slab_segments(n, frac256, slab, s0, s1);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int tiles_x = cam.tiles_x;
    for (uint32_t s = s0 + blockIdx.x; s < s1; s += gridDim.x) {
        uint32_t slot[4], cnt[4];
        uint2 rect[4];
        uint32_t mine = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t i = s * EM_SEG + threadIdx.x * 4 + k;
            if (i < n) { slot[k] = order[i]; rect[k] = slot_rect[slot[k]]; cnt[k] = slot_cnt[slot[k]]; }
            else { slot[k] = 0; rect[k] = make_uint2(0, 0); cnt[k] = 0; }
            mine += cnt[k];
        }
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        uint32_t wbase = 0;
        for (int w = 0; w < wid; ++w) wbase += warp_tot[w];
        uint32_t base = seg_excl[s] + wbase + incl - mine;
        // Only splats that emit something are parked, compacted (their output ranges are fixed by `base`, so the order
        // in which warps take them does not matter): behind finished tiles most splats of the far slab emit nothing, and
        // walking them one by one was the serial part of this kernel.
        uint32_t nz = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) nz += cnt[k] ? 1u : 0u;
        uint32_t nz_incl = nz;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, nz_incl, d);
            if (lane >= d) nz_incl += t;
        }
        if (lane == 31) warp_nz[wid] = nz_incl;
        __syncthreads();
        uint32_t nz_base = 0, nz_total = 0;
        for (int w = 0; w < 8; ++w) { if (w < wid) nz_base += warp_nz[w]; nz_total += warp_nz[w]; }
        uint32_t pos = nz_base + nz_incl - nz;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (cnt[k]) { s_slot[pos] = slot[k]; s_base[pos] = base; s_rect[pos] = rect[k]; ++pos; }
            base += cnt[k];
        }
        __syncthreads();
        for (uint32_t e = wid; e < nz_total; e += 8) {
            const uint2 r = s_rect[e];
            const uint32_t c = rect_count(r);
            if (c == 0) continue;
            const int x0 = r.x & 0xffff, y0 = r.x >> 16, w = (int)(r.y & 0xffff) - x0;
            const uint32_t sl = s_slot[e];
            uint32_t o = s_base[e];
            if (!tile_done) {
                for (uint32_t t = lane; t < c; t += 32) {
                    const uint32_t ty = t / (uint32_t)w, tx = t - ty * (uint32_t)w;
                    if (o + t < region_cap) { tile_keys[o + t] = (uint32_t)((y0 + (int)ty) * tiles_x + x0 + (int)tx); vals[o + t] = sl; }
                }
                continue;
            }
            for (uint32_t t0 = 0; t0 < c; t0 += 32) {
                const uint32_t t = t0 + lane;
                bool hit = false;
                uint32_t key = 0;
                if (t < c) {
                    const uint32_t ty = t / (uint32_t)w, tx = t - ty * (uint32_t)w;
                    key = (uint32_t)((y0 + (int)ty) * tiles_x + x0 + (int)tx);
                    hit = tile_done[key] == 0;
                }
                const uint32_t m = __ballot_sync(0xffffffffu, hit);
                if (hit) {
                    const uint32_t dst = o + __popc(m & ((1u << lane) - 1u));
                    if (dst < region_cap) { tile_keys[dst] = key; vals[dst] = sl; }
                }
                o += __popc(m);
            }
        }
        __syncthreads();
    }
}

// Summed-area table of the tiles that are NOT done: sat[(y+1)*(tiles_x+1) + (x+1)] = number of such tiles in
// [0,x] x [0,y]. One CTA: rows first, then columns.
__global__ void __launch_bounds__(1024) rgs_slab_sat_kernel(const uint8_t* __restrict__ tile_done, int tiles_x, int tiles_y,
                                                            uint32_t* __restrict__ sat) {
    const int pitch = tiles_x + 1;
    for (int x = threadIdx.x; x <= tiles_x; x += blockDim.x) sat[x] = 0u;
    for (int y = threadIdx.x; y < tiles_y; y += blockDim.x) {
        uint32_t run = 0;
        sat[(y + 1) * pitch] = 0u;
        for (int x = 0; x < tiles_x; ++x) {
            run += tile_done[y * tiles_x + x] ? 0u : 1u;
            sat[(y + 1) * pitch + x + 1] = run;
        }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < tiles_x; x += blockDim.x) {
        uint32_t run = 0;
        for (int y = 0; y < tiles_y; ++y) {
            run += sat[(y + 1) * pitch + x + 1];
            sat[(y + 1) * pitch + x + 1] = run;
        }
    }
}

// slot_cnt of every splat of the slab = number of not-done tiles in its rectangle
__global__ void __launch_bounds__(256) rgs_slab_filtered_count_kernel(const uint32_t* __restrict__ order,
                                                                      const uint2* __restrict__ slot_rect,
                                                                      const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                                      uint32_t frac256, int slab, const uint32_t* __restrict__ sat,
                                                                      int tiles_x, uint32_t* __restrict__ slot_cnt) {
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    uint32_t s0, s1;
    slab_segments(n, frac256, slab, s0, s1);
    const int pitch = tiles_x + 1;
    const uint32_t end = s1 * EM_SEG < n ? s1 * EM_SEG : n;
    for (uint32_t i = s0 * EM_SEG + blockIdx.x * blockDim.x + threadIdx.x; i < end; i += gridDim.x * blockDim.x) {
        const uint32_t slot = order[i];
        const uint2 r = slot_rect[slot];
        const int x0 = r.x & 0xffff, y0 = r.x >> 16, x1 = r.y & 0xffff, y1 = r.y >> 16;
        uint32_t c = 0;
        if (x1 > x0 && y1 > y0) c = sat[y1 * pitch + x1] - sat[y0 * pitch + x1] - sat[y1 * pitch + x0] + sat[y0 * pitch + x0];
        slot_cnt[slot] = c;
    }
}

// ---------------------------------------------------------------------------------------------
// Grouping by tile without a second sort ("segmented counting").
//
// The depth-ordered splat list is cut into one contiguous piece per warp, balanced by instance count.  A warp
// keeps one counter per tile in shared memory and walks its piece in depth order; all 32 lanes work on the tiles
// of ONE splat at a time, so that no two lanes touch the same counter and the order of a tile's instances is the
// depth order by construction.  Pass 1 counts (row w of the table = tile histogram of piece w), a column scan
// turns the table into the number of earlier instances per (piece, tile), a scan of the tile totals yields the
// tile ranges, and pass 2 repeats the walk with the counters preloaded with the final write positions and stores
// each instance's slot straight to its place.  Against "emit (tile, slot) pairs, then a stable radix sort by tile"
// this writes 4 bytes per instance once instead of moving 8 bytes per instance through 2 sort passes, but the walk
// is a serial chain per warp (see sc_enabled for the measurement that keeps it optional).
// ---------------------------------------------------------------------------------------------
#define SC_MAX_TILES 14336  // 56 KB of counters per warp

__device__ __forceinline__ uint32_t sc_bound(const uint32_t* __restrict__ seg_excl, uint32_t nseg, uint32_t total,
                                             uint32_t w, uint32_t W) {
    if (w >= W) return nseg;
    const uint32_t x = (uint32_t)(((unsigned long long)w * total) / W);
    uint32_t lo = 0, hi = nseg;  // first segment whose exclusive prefix is >= x
    while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (seg_excl[mid] < x) lo = mid + 1; else hi = mid;
    }
    return lo;
}

template <bool EMIT>
__global__ void __launch_bounds__(32) rgs_sc_walk_kernel(const __grid_constant__ RgsCamera cam,
                                                         const uint32_t* __restrict__ order,
                                                         const uint2* __restrict__ slot_rect,
                                                         const uint32_t* __restrict__ slot_cnt,
                                                         const RgsSplat* __restrict__ splats,
                                                         const uint32_t* __restrict__ counters, uint32_t cap_vis,
                                                         const uint32_t* __restrict__ seg_excl, uint32_t* __restrict__ table,
                                                         const uint32_t* __restrict__ tile_start,
                                                         uint32_t* __restrict__ vals, uint32_t cap_inst, uint32_t num_tiles) {
    extern __shared__ uint32_t sc_cnt[];
    const int lane = threadIdx.x;
    const uint32_t w = blockIdx.x, W = gridDim.x;
    const uint32_t n = bs_count(counters, RGS_CNT_VIS, cap_vis);
    const uint32_t nseg = (n + EM_SEG - 1) / EM_SEG;
    uint32_t* row = table + (size_t)w * num_tiles;
    for (uint32_t t = lane; t < num_tiles; t += 32) sc_cnt[t] = EMIT ? tile_start[t] + row[t] : 0u;
    __syncwarp();
    const uint32_t total = counters[RGS_CNT_INST];
    const uint32_t s0 = sc_bound(seg_excl, nseg, total, w, W), s1 = sc_bound(seg_excl, nseg, total, w + 1, W);
    const uint32_t i0 = s0 * EM_SEG;
    uint32_t i1 = s1 * EM_SEG;
    if (i1 > n) i1 = n;
    const int tiles_x = cam.tiles_x;
    const bool exact = cam.tight_rect >= 2;
    uint32_t nslot = 0;
    uint2 nrect = make_uint2(0, 0);
    if (i0 + lane < i1) {
        nslot = order[i0 + lane];
        nrect = slot_cnt[nslot] ? slot_rect[nslot] : make_uint2(0, 0);
    }
    for (uint32_t base = i0; base < i1; base += 32) {
        const uint32_t cslot = nslot;
        const uint2 crect = nrect;
        nrect = make_uint2(0, 0);
        if (base + 32 + lane < i1) {  // fetch the next 32 splats while this batch is walked
            nslot = order[base + 32 + lane];
            nrect = slot_cnt[nslot] ? slot_rect[nslot] : make_uint2(0, 0);
        }
        const int m = (int)(i1 - base < 32u ? i1 - base : 32u);
        for (int j = 0; j < m; ++j) {
            const uint32_t rx = __shfl_sync(0xffffffffu, crect.x, j), ry = __shfl_sync(0xffffffffu, crect.y, j);
            const int x0 = rx & 0xffff, y0 = rx >> 16;
            const uint32_t wd = (ry & 0xffffu) - (uint32_t)x0, c = wd * ((ry >> 16) - (uint32_t)y0);
            if (c == 0) continue;
            const uint32_t sl = __shfl_sync(0xffffffffu, cslot, j);
            const float inv_w = 1.0f / (float)wd;
            float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f);
            float2 q1 = make_float2(0.f, 0.f);
            float bound = 0.f;
            if (exact) {  // same test, same inputs as the count made by the projection kernel
                q0 = reinterpret_cast<const float4*>(splats + sl)[0];
                q1 = reinterpret_cast<const float2*>(splats + sl)[2];
                bound = rgs_alpha_bound(q1.y);
            }
            for (uint32_t t = lane; t < c; t += 32) {
                const uint32_t ty = (uint32_t)(((float)t + 0.5f) * inv_w), tx = t - ty * wd;
                if (exact && !rgs_tile_hit(q0.x, q0.y, q0.z, q0.w, q1.x, bound, x0 + (int)tx, y0 + (int)ty, cam.W, cam.H))
                    continue;
                const uint32_t tile = (uint32_t)((y0 + (int)ty) * tiles_x + x0 + (int)tx);
                if (tile >= num_tiles) continue;  // cannot happen for rectangles inside the tile grid
                const uint32_t pos = sc_cnt[tile];
                sc_cnt[tile] = pos + 1u;
                if (EMIT && pos < cap_inst) vals[pos] = sl;
            }
            __syncwarp();
        }
    }
    if (!EMIT) {
        __syncwarp();
        for (uint32_t t = lane; t < num_tiles; t += 32) row[t] = sc_cnt[t];
    }
}

// table[w][t] -> number of instances of tile t in pieces before w; tile_total[t] = instances of tile t
__global__ void __launch_bounds__(128) rgs_sc_colscan_kernel(uint32_t* __restrict__ table, uint32_t W, uint32_t T,
                                                             uint32_t* __restrict__ tile_total) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    uint32_t run = 0;
    for (uint32_t w0 = 0; w0 < W; w0 += 8) {
        uint32_t v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = w0 + k < W ? table[(size_t)(w0 + k) * T + t] : 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (w0 + k < W) table[(size_t)(w0 + k) * T + t] = run;
            run += v[k];
        }
    }
    tile_total[t] = run;
}

// one CTA: tile_total -> tile_start (exclusive scan, in place) and ranges[t] = [start, start + total), clipped to cap_inst
__global__ void __launch_bounds__(1024) rgs_sc_tilescan_kernel(uint32_t* __restrict__ tile_total, uint32_t T, uint32_t cap_inst,
                                                               int2* __restrict__ ranges) {
    __shared__ uint32_t warp_tot[32];
    __shared__ uint32_t carry;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (uint32_t start = 0; start < T; start += 1024) {
        const uint32_t i = start + threadIdx.x;
        const uint32_t v = i < T ? tile_total[i] : 0u;
        uint32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += y;
        }
        if (lane == 31) warp_tot[wid] = incl;
        __syncthreads();
        uint32_t wbase = 0;
        for (int k = 0; k < wid; ++k) wbase += warp_tot[k];
        const uint32_t excl = carry + wbase + incl - v;
        if (i < T) {
            tile_total[i] = excl;
            const uint32_t a = excl < cap_inst ? excl : cap_inst, b = excl + v < cap_inst ? excl + v : cap_inst;
            ranges[i] = make_int2((int)a, (int)b);
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry = excl + v;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
// table sizes assume the smallest chunk any variant uses
static inline uint32_t chunks_of(int64_t n) {
    const int64_t chunk = BS_THREADS * BS_MIN_ITEMS;
    int64_t c = (n + chunk - 1) / chunk;
    return (uint32_t)(c > 0 ? c : 1);
}

// scratch words in front of the area of the single-sweep sort (which holds a second look-back table, the digit
// totals of every pass and the tickets)
// The counter table of the segmented counting holds (warps x tiles) words; warps per SM x tiles x 4 bytes never
// exceeds the shared memory of an SM, which bounds the table for any image size.
#define SC_TABLE_WORDS (RGS_SMS * 227 * 256)
static inline int64_t scratch_base_words(int64_t cap_vis, int64_t cap_inst) {
    const int64_t cap = cap_vis > cap_inst ? cap_vis : cap_inst;
    return 256 * (int64_t)chunks_of(cap) + 256 + (cap_vis + EM_SEG - 1) / EM_SEG + 16 + SC_TABLE_WORDS + SC_MAX_TILES;
}

// items per thread of the sort kernels: 16 (4096-pair chunks) or 8 (2048-pair chunks, half the registers);
// RGS_SORT_ITEMS selects the variant.
static int sort_items() {
    static int v = 0;
    if (!v) {
        const char* e = getenv("RGS_SORT_ITEMS");
        v = (e && atoi(e) == 8) ? 8 : 16;
    }
    return v;
}

template <int ITEMS>
static void bs_pass(const uint32_t* kin, const uint32_t* vin, uint32_t* kout, uint32_t* vout, const uint32_t* cnt, int which,
                    uint32_t cap, int shift, uint32_t* hist, uint32_t* totals, uint32_t nchunks_cap, int iota, cudaStream_t st) {
    const uint32_t chunk = BS_THREADS * ITEMS;
    const uint32_t nch = (cap + chunk - 1) / chunk;
    const unsigned grid = nch < 1u ? 1u : (nch < (unsigned)(RGS_SMS * 8) ? nch : (unsigned)(RGS_SMS * 8));
    // which == CNT_INST is the tile sort: its upper digit repeats inside a warp, everything else is close to random
    const int aggregate = ((which == RGS_CNT_INST || which == RGS_CNT_INST2) && shift >= 8) ? 1 : 0;
    rgs_bs_hist_kernel<ITEMS><<<grid, BS_THREADS, 0, st>>>(kin, cnt, which, cap, shift, hist, nchunks_cap, aggregate);
    rgs_bs_scan_kernel<<<256, 256, 0, st>>>(hist, totals, cnt, which, cap, nchunks_cap, chunk);
    rgs_bs_scatter_kernel<ITEMS><<<grid, BS_THREADS, 0, st>>>(kin, vin, kout, vout, cnt, which, cap, shift, hist, totals,
                                                              nchunks_cap, iota);
}

// 1: single-sweep sort (digit counts up front, decoupled look-back in the scatter; default), 0: histogram, scan and
// scatter launches per pass (RGS_SORT=3k).
static int g_sort_sweep = -1;
static int sort_sweep() {
    if (g_sort_sweep < 0) {
        const char* e = getenv("RGS_SORT");
        g_sort_sweep = (e && !strcmp(e, "3k")) ? 0 : 1;
    }
    return g_sort_sweep;
}

template <int ITEMS>
static void bs_sweep_passes(const uint32_t* keys_first, uint32_t* ka, uint32_t* va, uint32_t* kb, uint32_t* vb, uint32_t* cnt,
                            int which, uint32_t cap, int npass, uint32_t* lb_a, uint32_t* lb_b, uint32_t* small,
                            int iota_first, cudaStream_t st, uint32_t** k_out, uint32_t** v_out) {
    const uint32_t chunk = BS_THREADS * ITEMS;
    const uint32_t nch = (cap + chunk - 1) / chunk;
    const unsigned grid = nch < 1u ? 1u : (nch < (unsigned)(RGS_SMS * 8) ? nch : (unsigned)(RGS_SMS * 8));
    uint32_t* totals = small;
    uint32_t* tickets = small + BS_SWEEP_MAX_PASSES * 256;
    cudaMemsetAsync(small, 0, BS_SWEEP_SMALL_WORDS * sizeof(uint32_t), st);
    // digits that repeat inside a warp: the upper digit of the tile keys, the exponent byte of the depth keys
    const bool tile_sort = which == RGS_CNT_INST || which == RGS_CNT_INST2;
    const int agg_mask = tile_sort ? 0xe : 0x8;
    rgs_bs_digits_kernel<ITEMS><<<grid, BS_THREADS, 0, st>>>(keys_first, cnt, which, cap, npass, agg_mask, totals, lb_a);
    const uint32_t* kin = keys_first;
    uint32_t* vin = va;
    uint32_t *kout = kb, *vout = vb;
    for (int p = 0; p < npass; ++p) {
        const int iota = (p == 0 && iota_first) ? 1 : 0;
        rgs_bs_sweep_kernel<ITEMS><<<grid, BS_THREADS, 0, st>>>(kin, vin, kout, vout, cnt, which, cap, 8 * p, totals + 256 * p,
                                                                (p & 1) ? lb_b : lb_a, (p & 1) ? lb_a : lb_b, tickets + p, iota);
        kin = kout; vin = vout;
        if (kout == kb) { kout = ka; vout = va; } else { kout = kb; vout = vb; }
    }
    *k_out = const_cast<uint32_t*>(kin);
    *v_out = vin;
}

// sweep: the area of the single-sweep sort inside the scratch (second look-back table + digit totals + tickets), or
// null to force the three-kernel passes.
static void bs_sort(const uint32_t* keys_first, uint32_t* ka, uint32_t* va, uint32_t* kb, uint32_t* vb, uint32_t* cnt,
                    int which, uint32_t cap, int npass, uint32_t* hist, uint32_t* totals, int iota_first, cudaStream_t st,
                    uint32_t** k_out, uint32_t** v_out, uint32_t* sweep = nullptr) {
    const uint32_t nchunks_cap = chunks_of(cap);
    const int items = sort_items();
    if (sweep && sort_sweep() && npass <= BS_SWEEP_MAX_PASSES && cap < (1u << 30)) {
        // hist is the first look-back table (256 words per chunk, as many as the histogram of the other variant)
        uint32_t* lb_b = sweep;
        uint32_t* small = sweep + 256 * (size_t)nchunks_cap;
        if (items == 16) bs_sweep_passes<16>(keys_first, ka, va, kb, vb, cnt, which, cap, npass, hist, lb_b, small, iota_first, st, k_out, v_out);
        else bs_sweep_passes<8>(keys_first, ka, va, kb, vb, cnt, which, cap, npass, hist, lb_b, small, iota_first, st, k_out, v_out);
        return;
    }
    const uint32_t* kin = keys_first;
    uint32_t* vin = va;
    uint32_t *kout = kb, *vout = vb;
    for (int p = 0; p < npass; ++p) {
        const int iota = (p == 0 && iota_first) ? 1 : 0;
        if (items == 16) bs_pass<16>(kin, vin, kout, vout, cnt, which, cap, 8 * p, hist, totals, nchunks_cap, iota, st);
        else bs_pass<8>(kin, vin, kout, vout, cnt, which, cap, 8 * p, hist, totals, nchunks_cap, iota, st);
        // ping-pong: after the first pass the input buffers are (ka, va) / (kb, vb) alternately
        kin = kout; vin = vout;
        if (kout == kb) { kout = ka; vout = va; } else { kout = kb; vout = vb; }
    }
    *k_out = const_cast<uint32_t*>(kin);
    *v_out = vin;
}

extern "C" {

int rgs_cuda_project_slots(const RgsCamera* cam, const RgsSegment* seg, int64_t id_base, RgsSplat* splats,
                           int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth, uint32_t* slot_rect,
                           uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads, void* stream) {
    if (seg->count <= 0) return 0;
    if (cap_vis > 0x7ffffff0ll || cam->tiles_x > 65535 || cam->tiles_y > 65535) return 10;
    if ((uintptr_t)seg->sh & 15u) return 14;  // SH rows are read as 128-bit words
    const unsigned blocks = (unsigned)((seg->count + 255) / 256);
    rgs_project_slots_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
        *cam, *seg, id_base, splats, vis_ids, aux, (uint32_t)cap_vis, slot_depth, reinterpret_cast<uint2*>(slot_rect),
        slot_cnt, reinterpret_cast<uint32_t*>(counters), splat_grads);
    return (int)cudaGetLastError();
}

// Two-phase variant of rgs_cuda_project_slots over up to 4 segments: cull all, then project the survivors.
// `cand` holds cap_cand uint32 candidate ids (scratch owned by the caller).
static int project_slots2_impl(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, uint32_t* cand, int64_t cap_cand,
                               RgsSplat* splats, int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth,
                               uint32_t* slot_rect, uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads,
                               int lazy, void* stream) {
    if (nseg < 1 || nseg > 4) return 11;
    for (int k = 0; k < (int)nseg; ++k)  // SH rows are fetched as 16-byte aligned bulk copies
        if (segs[k].count > 0 && ((uintptr_t)segs[k].sh & 15u)) return 14;
    if (cap_vis > 0x7ffffff0ll || cap_cand > 0x7ffffff0ll || cam->tiles_x > 65535 || cam->tiles_y > 65535) return 10;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(counters);
    RgsSegs4 s4;
    s4.n = (int)nseg;
    int64_t base = 0;
    for (int k = 0; k < (int)nseg; ++k) {
        s4.s[k] = segs[k];
        if (segs[k].count > 0) {
            const unsigned blocks = (unsigned)((segs[k].count + CULL_ROWS - 1) / CULL_ROWS);
            if ((((uintptr_t)segs[k].xyz | (uintptr_t)segs[k].scale) & 15u) == 0)
                rgs_cull_kernel<true><<<blocks, 256, 0, st>>>(*cam, segs[k].xyz, segs[k].scale, segs[k].count, base, cand,
                                                              (uint32_t)cap_cand, cnt);
            else
                rgs_cull_kernel<false><<<blocks, 256, 0, st>>>(*cam, segs[k].xyz, segs[k].scale, segs[k].count, base, cand,
                                                               (uint32_t)cap_cand, cnt);
        }
        base += segs[k].count;
    }
    const int64_t want = (cap_cand + PC_THREADS - 1) / PC_THREADS;
    const unsigned grid = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 8 ? RGS_SMS * 8 : want));
    rgs_project_cand_kernel<<<grid, PC_THREADS, 0, st>>>(*cam, s4, cand, (uint32_t)cap_cand, splats, vis_ids, aux, (uint32_t)cap_vis,
                                                  slot_depth, reinterpret_cast<uint2*>(slot_rect), slot_cnt, cnt, splat_grads,
                                                  lazy);
    return (int)cudaGetLastError();
}

int rgs_cuda_project_slots2(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, uint32_t* cand, int64_t cap_cand,
                            RgsSplat* splats, int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth,
                            uint32_t* slot_rect, uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads,
                            void* stream) {
    return project_slots2_impl(cam, segs, nseg, cand, cap_cand, splats, vis_ids, aux, cap_vis, slot_depth, slot_rect, slot_cnt,
                               counters, splat_grads, 0, stream);
}

// Geometry only (colours stay zero): rgs_cuda_colour_slab fills them in for the splats that get tile instances.
int rgs_cuda_project_slots2_geom(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, uint32_t* cand, int64_t cap_cand,
                                 RgsSplat* splats, int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth,
                                 uint32_t* slot_rect, uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads,
                                 void* stream) {
    return project_slots2_impl(cam, segs, nseg, cand, cap_cand, splats, vis_ids, aux, cap_vis, slot_depth, slot_rect, slot_cnt,
                               counters, splat_grads, 1, stream);
}

// Colours of the splats of slab `slab` (the split of rgs_cuda_bin_slab) whose slot_cnt is not zero; call between the
// slab's binning and its blend. `order`: the depth order left by the binning of slab 0.
int rgs_cuda_colour_slab(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, const uint32_t* order,
                         const uint32_t* slot_cnt, const int32_t* counters, int64_t cap_vis, int64_t frac256, int64_t slab,
                         RgsSplat* splats, const int32_t* vis_ids, uint32_t* aux, void* stream) {
    if (nseg < 1 || nseg > 4 || slab < 0 || slab > 1) return 11;
    for (int k = 0; k < (int)nseg; ++k)
        if (segs[k].count > 0 && ((uintptr_t)segs[k].sh & 15u)) return 14;
    RgsSegs4 s4;
    s4.n = (int)nseg;
    for (int k = 0; k < (int)nseg; ++k) s4.s[k] = segs[k];
    const int64_t want = (cap_vis + 127) / 128;
    const unsigned grid = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 16 ? RGS_SMS * 16 : want));
    rgs_colour_slab_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(*cam, s4, order, slot_cnt,
                                                                  reinterpret_cast<const uint32_t*>(counters), (uint32_t)cap_vis,
                                                                  (uint32_t)frac256, (int)slab, splats, vis_ids, aux);
    return (int)cudaGetLastError();
}

// 1: group by tile with the segmented counting (RGS_TILE_GROUPING=count), 0: with the radix sort (default).
// Measured at 62.9 M Gaussians, 1600x1036 (85 M instances per view): 17 ms per view against 3.6 ms for pair
// emission + 2 radix passes + range detection. One warp per piece walks its splats strictly in order, so only
// 8 warps per SM run, each a chain of dependent shuffle / shared-memory instructions; the variant is kept for
// small images and as a cross-check of the sort (tests compare both).
static int sc_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RGS_TILE_GROUPING");
        v = (e && !strcmp(e, "count")) ? 1 : 0;
    }
    return v;
}

// words of uint32 scratch for capacities (cap_vis, cap_inst)
int64_t rgs_cuda_bin_scratch_words(int64_t cap_vis, int64_t cap_inst) {
    const int64_t cap = cap_vis > cap_inst ? cap_vis : cap_inst;
    return scratch_base_words(cap_vis, cap_inst) + 256 * (int64_t)chunks_of(cap) + BS_SWEEP_SMALL_WORDS;
}

// 1 selects the single-sweep radix sort, 0 the three-kernel passes; returns the setting that was in force.
int rgs_cuda_sort_sweep(int on) {
    const int old = sort_sweep();
    g_sort_sweep = on ? 1 : 0;
    return old;
}

// Depth-order the visible slots, emit instances in that order, group them by tile.
//   slot_depth/slot_rect: per slot, from rgs_cuda_project_slots
//   vis_a/vis_b (u32[cap_vis] x4: key/value ping-pong)  inst_keys/inst_vals/inst_keys_tmp/inst_vals_tmp (u32[cap_inst])
// Result: inst_vals holds the slots grouped by tile in depth order, ranges[tile] = [start,end).
int rgs_cuda_bin_instances(const RgsCamera* cam, const RgsSplat* splats, const uint32_t* slot_depth, const uint32_t* slot_rect,
                           const uint32_t* slot_cnt, int64_t cap_vis, uint32_t* vis_ka,
                           uint32_t* vis_va, uint32_t* vis_kb, uint32_t* vis_vb, uint32_t* inst_keys, uint32_t* inst_vals,
                           uint32_t* inst_keys_tmp, uint32_t* inst_vals_tmp, int64_t cap_inst, int32_t* counters,
                           int64_t tiles_x, int64_t num_tiles, int32_t* ranges, uint32_t* scratch, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (cap_inst > 0xfffffe00ll) return 10;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(counters);
    const int64_t cap = cap_vis > cap_inst ? cap_vis : cap_inst;
    uint32_t* hist = scratch;
    uint32_t* totals = scratch + 256 * (size_t)chunks_of(cap);
    uint32_t* seg_sums = totals + 256;
    uint32_t* sweep = scratch + scratch_base_words(cap_vis, cap_inst);
    // 1. depth sort of the slots (values start as 0..n-1 == the slots themselves)
    uint32_t *dk, *order;
    bs_sort(slot_depth, vis_ka, vis_va, vis_kb, vis_vb, cnt, RGS_CNT_VIS, (uint32_t)cap_vis, 4, hist, totals, 1, st, &dk,
            &order, sweep);
    // 2. emission in depth order
    const uint32_t nseg_cap = (uint32_t)((cap_vis + EM_SEG - 1) / EM_SEG);
    const unsigned egrid = nseg_cap < (unsigned)(RGS_SMS * 8) ? (nseg_cap ? nseg_cap : 1u) : (unsigned)(RGS_SMS * 8);
    rgs_emit_count_kernel<<<egrid, 256, 0, st>>>(order, slot_cnt, cnt, (uint32_t)cap_vis, seg_sums);
    rgs_emit_scan_kernel<<<1, 1024, 0, st>>>(seg_sums, cnt, (uint32_t)cap_vis, (uint32_t)cap_inst);
    if (sc_enabled() && num_tiles <= SC_MAX_TILES) {
        // 3'. no pair emission, no second sort: count per (piece, tile), scan, store every slot at its final place
        uint32_t* table = seg_sums + (cap_vis + EM_SEG - 1) / EM_SEG + 16;
        uint32_t* tile_start = table + SC_TABLE_WORDS;
        const size_t smem = (size_t)num_tiles * 4;
        int per_sm = (int)((227 * 1024) / (smem + 1024));
        per_sm = per_sm > 8 ? 8 : (per_sm < 1 ? 1 : per_sm);
        const unsigned W = (unsigned)RGS_SMS * (unsigned)per_sm;
        if ((int64_t)W * num_tiles > SC_TABLE_WORDS) return 13;
        static bool attr_set = false;
        if (!attr_set) {
            RGS_CUDA_CHECK(cudaFuncSetAttribute(rgs_sc_walk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                SC_MAX_TILES * 4));
            RGS_CUDA_CHECK(cudaFuncSetAttribute(rgs_sc_walk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                SC_MAX_TILES * 4));
            attr_set = true;
        }
        const uint2* rects = reinterpret_cast<const uint2*>(slot_rect);
        rgs_sc_walk_kernel<false><<<W, 32, smem, st>>>(*cam, order, rects, slot_cnt, splats, cnt, (uint32_t)cap_vis, seg_sums,
                                                       table, tile_start, inst_vals, (uint32_t)cap_inst, (uint32_t)num_tiles);
        rgs_sc_colscan_kernel<<<(unsigned)((num_tiles + 127) / 128), 128, 0, st>>>(table, W, (uint32_t)num_tiles, tile_start);
        rgs_sc_tilescan_kernel<<<1, 1024, 0, st>>>(tile_start, (uint32_t)num_tiles, (uint32_t)cap_inst,
                                                   reinterpret_cast<int2*>(ranges));
        rgs_sc_walk_kernel<true><<<W, 32, smem, st>>>(*cam, order, rects, slot_cnt, splats, cnt, (uint32_t)cap_vis, seg_sums,
                                                      table, tile_start, inst_vals, (uint32_t)cap_inst, (uint32_t)num_tiles);
        return (int)cudaGetLastError();
    }
    rgs_emit_kernel<<<egrid, 256, 0, st>>>(*cam, order, reinterpret_cast<const uint2*>(slot_rect), slot_cnt, splats, cnt,
                                           (uint32_t)cap_vis, seg_sums, inst_keys, inst_vals, (uint32_t)cap_inst);
    (void)tiles_x;
    // 3. stable sort by tile id
    int tile_bits = 0;
    while ((1ll << tile_bits) < num_tiles) ++tile_bits;
    const int npass = tile_bits <= 8 ? 1 : (tile_bits + 7) / 8;
    uint32_t *tk, *tv;
    bs_sort(inst_keys, inst_keys, inst_vals, inst_keys_tmp, inst_vals_tmp, cnt, RGS_CNT_INST, (uint32_t)cap_inst, npass, hist,
            totals, 0, st, &tk, &tv, sweep);
    const bool in_tmp = (tv != inst_vals);
    if (!in_tmp) {  // nothing to copy back: find the ranges without reading every key
        rgs_bs_tile_ranges_search_kernel<<<(unsigned)((num_tiles + 127) / 128), 128, 0, st>>>(
            tk, cnt, (uint32_t)cap_inst, reinterpret_cast<int2*>(ranges), (uint32_t)num_tiles, RGS_CNT_INST, 0u);
        return (int)cudaGetLastError();
    }
    RGS_CUDA_CHECK(cudaMemsetAsync(ranges, 0, (size_t)num_tiles * 8, st));
    rgs_bs_tile_ranges_kernel<<<(unsigned)(RGS_SMS * 8), 256, 0, st>>>(tk, cnt, (uint32_t)cap_inst, reinterpret_cast<int2*>(ranges),
                                                       (uint32_t)num_tiles, in_tmp ? tv : nullptr, in_tmp ? inst_vals : nullptr);
    return (int)cudaGetLastError();
}

// Two-slab binning, one call per slab (see the comment above rgs_slab_count_kernel).
//   slab 0: depth sort of all visible slots, then emission + tile sort of the near slab (frac256/256 of the splats)
//           into the first region_cap elements of the instance buffers; count -> counters[RGS_CNT_INST]. With
//           tile_done (+ sat) only tiles that are not marked get instances: tiles hidden behind nearer sub-models.
//   slab 1: tile_done (one byte per tile, written by the blend of slab 0) -> summed-area table -> filtered counts,
//           emission + tile sort of the far slab into the region starting at region_off; count -> counters[RGS_CNT_INST2];
//           ranges hold absolute indices into inst_vals.
// sat: (tiles_x + 1) * (tiles_y + 1) words. Only tile grids of at most 2^24 tiles and tight_rect < 2.
int rgs_cuda_bin_slab(const RgsCamera* cam, const uint32_t* slot_depth, const uint32_t* slot_rect, uint32_t* slot_cnt,
                      int64_t cap_vis, uint32_t* vis_ka, uint32_t* vis_va, uint32_t* vis_kb, uint32_t* vis_vb,
                      uint32_t* inst_keys, uint32_t* inst_vals, uint32_t* inst_keys_tmp, uint32_t* inst_vals_tmp,
                      int64_t region_off, int64_t region_cap, int32_t* counters, int64_t num_tiles, int32_t* ranges,
                      uint32_t* scratch, int64_t scratch_cap_inst, int64_t slab, int64_t frac256, const uint8_t* tile_done,
                      uint32_t* sat, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (num_tiles > (1 << 24) || cam->tight_rect >= 2 || slab < 0 || slab > 1) return 15;
    if (region_off + region_cap > 0xfffffe00ll || frac256 < 0 || frac256 > 256) return 10;
    if (region_off < 0 || region_cap <= 0 || region_off + region_cap > scratch_cap_inst) return 10;  // outside the buffers
    uint32_t* cnt = reinterpret_cast<uint32_t*>(counters);
    const int64_t cap = cap_vis > scratch_cap_inst ? cap_vis : scratch_cap_inst;
    uint32_t* hist = scratch;
    uint32_t* totals = scratch + 256 * (size_t)chunks_of(cap);
    uint32_t* seg_sums = totals + 256;
    uint32_t* sweep = scratch + scratch_base_words(cap_vis, scratch_cap_inst);
    uint32_t* order = vis_va;  // where four ping-pong passes leave the sorted values
    if (slab == 0) {
        uint32_t *dk, *ord;
        bs_sort(slot_depth, vis_ka, vis_va, vis_kb, vis_vb, cnt, RGS_CNT_VIS, (uint32_t)cap_vis, 4, hist, totals, 1, st, &dk, &ord,
                sweep);
        if (ord != order) return 16;
    }
    const int which = slab == 0 ? RGS_CNT_INST : RGS_CNT_INST2;
    const uint2* rects = reinterpret_cast<const uint2*>(slot_rect);
    const uint32_t nseg_cap = (uint32_t)((cap_vis + EM_SEG - 1) / EM_SEG);
    const unsigned egrid = nseg_cap < (unsigned)(RGS_SMS * 8) ? (nseg_cap ? nseg_cap : 1u) : (unsigned)(RGS_SMS * 8);
    if (slab == 1 && (!tile_done || !sat)) return 15;
    if (tile_done) {  // the far slab always filters; the near slab when tiles are known to be hidden by nearer sub-models
        if (!sat) return 15;
        rgs_slab_sat_kernel<<<1, 1024, 0, st>>>(tile_done, cam->tiles_x, cam->tiles_y, sat);
        rgs_slab_filtered_count_kernel<<<(unsigned)(RGS_SMS * 8), 256, 0, st>>>(order, rects, cnt, (uint32_t)cap_vis, (uint32_t)frac256,
                                                               (int)slab, sat, cam->tiles_x, slot_cnt);
    }
    rgs_slab_count_kernel<<<egrid, 256, 0, st>>>(order, slot_cnt, cnt, (uint32_t)cap_vis, (uint32_t)frac256, (int)slab, seg_sums);
    rgs_slab_scan_kernel<<<1, 1024, 0, st>>>(seg_sums, cnt, (uint32_t)cap_vis, (uint32_t)frac256, (int)slab, which,
                                             (uint32_t)region_cap);
    uint32_t* rk = inst_keys + region_off;
    uint32_t* rv = inst_vals + region_off;
    rgs_slab_emit_kernel<<<egrid, 256, 0, st>>>(*cam, order, rects, slot_cnt, cnt, (uint32_t)cap_vis, (uint32_t)frac256,
                                                (int)slab, seg_sums, rk, rv, (uint32_t)region_cap, tile_done);
    int tile_bits = 0;
    while ((1ll << tile_bits) < num_tiles) ++tile_bits;
    const int npass = tile_bits <= 8 ? 1 : (tile_bits + 7) / 8;
    uint32_t *tk, *tv;
    bs_sort(rk, rk, rv, inst_keys_tmp + region_off, inst_vals_tmp + region_off, cnt, which, (uint32_t)region_cap, npass, hist,
            totals, 0, st, &tk, &tv, sweep);
    if (tv != rv) {  // a single pass leaves the result in the second buffer
        RGS_CUDA_CHECK(cudaMemcpyAsync(rv, tv, (size_t)region_cap * 4, cudaMemcpyDeviceToDevice, st));
    }
    rgs_bs_tile_ranges_search_kernel<<<(unsigned)((num_tiles + 127) / 128), 128, 0, st>>>(
        tk, cnt, (uint32_t)region_cap, reinterpret_cast<int2*>(ranges), (uint32_t)num_tiles, which, (uint32_t)region_off);
    return (int)cudaGetLastError();
}

}  // extern "C"
