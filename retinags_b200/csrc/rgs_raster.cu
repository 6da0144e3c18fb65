// sm_100a rasteriser kernels: projection + SH + instance emission, tile blend forward/backward,
// per-Gaussian geometry backward.
//
// Design notes (what differs from the reference's
// rasterization_kernels/diff-gaussian-rasterization-half-gaussian/cuda_rasterizer_hgs/{forward,backward,
// rasterizer_impl}.cu):
//  * projection, tile counting, the prefix sum over tile counts and duplicate-with-keys are ONE
//    kernel: a block aggregates its instance count, reserves a range of the key buffer with one
//    atomic and emits directly. No per-Gaussian count/offset arrays, no separate scan, and the
//    instance total stays on the device (the reference copies it to the host,
//    rasterizer_impl.cu:286-287).
//  * visible splats are compacted into 48-byte records; everything downstream is sized by the
//    number of visible splats, not by the number of Gaussians.
//  * the blend kernels stage the depth-sorted splat records of a tile into shared memory with
//    bulk asynchronous copies (cp.async.bulk, completion on an mbarrier), double buffered.
//  * the blend backward reduces the nine per-splat gradients over the warp and issues one
//    vector reduction per warp instead of nine atomics per pixel (backward.cu:576-619).
//  * every wait on an mbarrier is bounded; on expiry the block records a status word and leaves.
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"

// ---------------------------------------------------------------------------------------------
// project + emit
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rgs_project_emit_kernel(
    const __grid_constant__ RgsCamera cam, const RgsSegment seg, const int64_t id_base, RgsSplat* __restrict__ splats,
    int32_t* __restrict__ vis_ids, uint32_t* __restrict__ aux, const uint32_t cap_vis, uint64_t* __restrict__ keys,
    uint32_t* __restrict__ vals, const uint32_t cap_inst, uint32_t* __restrict__ counters,
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
    uint32_t cnt = ok ? (uint32_t)((rc.x1 - rc.x0) * (rc.y1 - rc.y0)) : 0u;
    // block-wide exclusive scans of (visible, instances)
    __shared__ uint32_t warp_cnt[8], warp_vis[8];
    __shared__ uint32_t base_cnt, base_vis;
    __shared__ int drop;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint32_t incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    const uint32_t vmask = __ballot_sync(0xffffffffu, ok);
    if (lane == 31) { warp_cnt[wid] = incl; warp_vis[wid] = __popc(vmask); }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t tc = 0, tv = 0;
        for (int w = 0; w < 8; ++w) { uint32_t c = warp_cnt[w]; warp_cnt[w] = tc; tc += c;
                                      uint32_t v = warp_vis[w]; warp_vis[w] = tv; tv += v; }
        uint32_t bc = 0, bv = 0;
        int d = 0;
        if (tv) {
            bc = atomicAdd(&counters[RGS_CNT_INST], tc);
            bv = atomicAdd(&counters[RGS_CNT_VIS], tv);
            // unsigned wrap of the instance counter also counts as overflow
            if (bc + tc > cap_inst || bc + tc < bc || bv + tv > cap_vis) { atomicExch(&counters[RGS_CNT_OVERFLOW], 1u); d = 1; }
        }
        base_cnt = bc; base_vis = bv; drop = d;
    }
    __syncthreads();
    if (!ok || drop) return;
    const uint32_t slot = base_vis + warp_vis[wid] + __popc(vmask & ((1u << lane) - 1u));
    uint32_t off = base_cnt + warp_cnt[wid] + (incl - cnt);
    float4* dst = reinterpret_cast<float4*>(splats + slot);
    dst[0] = make_float4(sp.px, sp.py, sp.ca, sp.cb);
    dst[1] = make_float4(sp.cc, sp.opacity, sp.r, sp.g);
    dst[2] = make_float4(sp.b, sp.w, sp.depth, sp.pmin);
    vis_ids[slot] = (int32_t)(id_base + i);
    aux[slot] = ((uint32_t)radius << 3) | clamped;
    if (splat_grads) {  // the backward accumulates into this record: clear it here, no separate memset
        float4* gz = reinterpret_cast<float4*>(splat_grads + slot);
        gz[0] = make_float4(0.f, 0.f, 0.f, 0.f); gz[1] = gz[0]; gz[2] = gz[0];
    }
    const uint64_t dbits = (uint64_t)__float_as_uint(sp.depth);
    for (int y = rc.y0; y < rc.y1; ++y)
        for (int x = rc.x0; x < rc.x1; ++x) {
            keys[off] = ((uint64_t)(uint32_t)(y * cam.tiles_x + x) << 32) | dbits;
            vals[off] = slot;
            ++off;
        }
}

// ---------------------------------------------------------------------------------------------
// blend forward
// ---------------------------------------------------------------------------------------------
#define BLEND_BATCH 256
#define RGS_MAX_PUSH 32
#define RGS_WAIT_LIMIT (1u << 22)

struct BlendSmem {
    RgsSplat buf[2][BLEND_BATCH];
    unsigned long long bar[2];
};

// Issue the gather of one batch: every thread copies the 48-byte record of one sorted instance.
#define RGS_STATUS_BAD_INDEX 16u  // a slot or range read from the binning buffers was out of bounds (flagged, clamped)

// A slot index from the sorted instance list, checked against the number of visible splats: a bad index is reported
// through the status word and replaced by slot 0, so that no copy ever leaves the splat buffer.
__device__ __forceinline__ uint32_t checked_slot(uint32_t slot, uint32_t n_vis, uint32_t* counters) {
    if (slot < n_vis) return slot;
    atomicOr(&counters[RGS_CNT_STATUS], RGS_STATUS_BAD_INDEX);
    return 0u;
}

// Tile range clipped to [0, n_inst]; an inverted or out-of-range record is reported and treated as empty.
__device__ __forceinline__ int2 checked_range(int2 r, uint32_t* counters, int which = RGS_CNT_INST, uint32_t base = 0u) {
    if (counters[RGS_CNT_OVERFLOW]) return make_int2(0, 0);
    if (r.x == 0 && r.y == 0) return r;  // empty
    const uint32_t end = base + counters[which];
    if (r.x < 0 || r.y < r.x || (uint32_t)r.x < base || (uint32_t)r.y > end) {
        atomicOr(&counters[RGS_CNT_STATUS], RGS_STATUS_BAD_INDEX);
        return make_int2(0, 0);
    }
    return r;
}

// Two-slab rendering (see rgs_binning.cu): how a blend launch relates to the slabs.
#define RGS_SLAB_SINGLE 0  // one list per tile, the whole render
#define RGS_SLAB_NEAR 1    // first of two launches: leaves the pixel state in the output buffers, marks finished tiles
#define RGS_SLAB_FAR 2     // second launch: resumes from that state with the far slab's list
struct RgsSlabArgs {
    const int2* ranges_b;   // per-tile ranges of the far slab (absolute indices into vals), null without slabs
    uint8_t* tile_done;     // one byte per tile: every pixel of the tile is finished (written by both slab launches)
    uint32_t base_b;        // first element of the far slab's region in vals
    int mode;
    const uint8_t* occl;    // near launch, optional: tiles hidden behind nearer sub-models (they hold no instances)
};

__device__ __forceinline__ void blend_issue(BlendSmem& sm, int stage, const RgsSplat* __restrict__ splats,
                                            const uint32_t* __restrict__ vals, int first, int count, bool reverse,
                                            int range_end, uint32_t n_vis, uint32_t* counters) {
    const int t = threadIdx.x;
    if (t == 0) rgs_mbar_expect_tx(&sm.bar[stage], (uint32_t)count * (uint32_t)sizeof(RgsSplat));
    if (t < count) {
        const int idx = reverse ? (range_end - 1 - first - t) : (first + t);
        const uint32_t slot = checked_slot(vals[idx], n_vis, counters);
        rgs_bulk_g2s(&sm.buf[stage][t], splats + slot, (uint32_t)sizeof(RgsSplat), &sm.bar[stage]);
    }
}

// Destinations of the fused push: for every owner rank the rows [row0,row1) it needs of this partial and
// the (possibly peer-mapped) base of its slot, which holds exactly those rows.
struct RgsPushPlan {
    int n;
    int row0[RGS_MAX_PUSH];
    int row1[RGS_MAX_PUSH];
    float4* dst[RGS_MAX_PUSH];
};

__global__ void __launch_bounds__(256) rgs_blend_fwd_kernel(
    const __grid_constant__ RgsCamera cam, const int2* __restrict__ ranges, const uint32_t* __restrict__ vals,
    const RgsSplat* __restrict__ splats, float4* __restrict__ out, float* __restrict__ depth,
    int32_t* __restrict__ n_contrib, uint32_t* __restrict__ counters, const __grid_constant__ RgsPushPlan push,
    const __grid_constant__ RgsSlabArgs slab) {
    __shared__ __align__(128) BlendSmem sm;
    const int tid = threadIdx.x;
    // a warp owns a compact 8x4 block of the tile (2 x 4 blocks per tile): the smaller the extent of the warp's
    // pixels, the more splats the warp-level test rejects
    const int bx = (tid >> 5) & 1, by = tid >> 6;
    const int lx = bx * 8 + (tid & 7), ly = by * 4 + ((tid >> 3) & 3);
    const int px = blockIdx.x * RGS_TILE + lx, py = blockIdx.y * RGS_TILE + ly;
    const bool inside = px < cam.W && py < cam.H;
    const int tile = blockIdx.y * cam.tiles_x + blockIdx.x;
    const int2 range_a = checked_range(ranges[tile], counters);
    const int2 range = slab.mode == RGS_SLAB_FAR ? checked_range(slab.ranges_b[tile], counters, RGS_CNT_INST2, slab.base_b)
                                                 : range_a;
    // position of this launch's first instance in the tile's whole (near + far) list
    const int first_contrib = slab.mode == RGS_SLAB_FAR ? range_a.y - range_a.x : 0;
    const uint32_t n_vis = counters[RGS_CNT_VIS];
    const int total = range.y - range.x;
    const int rounds = (total + BLEND_BATCH - 1) / BLEND_BATCH;
    if (tid == 0) { rgs_mbar_init(&sm.bar[0], 1); rgs_mbar_init(&sm.bar[1], 1); rgs_fence_mbar_init(); }
    __syncthreads();

    const float pixx = (float)px, pixy = (float)py;
    const int lane = tid & 31;
    // pixel-centre rectangle of this warp's 8x4 block, clipped to the image
    const float strip_x0 = (float)(blockIdx.x * RGS_TILE + bx * 8), strip_y0 = (float)(blockIdx.y * RGS_TILE + by * 4);
    const float strip_x1 = fminf(strip_x0 + 7.0f, (float)(cam.W - 1)), strip_y1 = fminf(strip_y0 + 3.0f, (float)(cam.H - 1));
    RgsPixelRay ray;
    rgs_pixel_ray(cam, pixx, pixy, ray);
    RgsPixelState st;
    rgs_pixel_init(st);
    st.done = !inside;
    if (slab.mode == RGS_SLAB_FAR && inside) {  // resume where the near slab stopped
        const int64_t pid = (int64_t)py * cam.W + px;
        const float4 o = out[pid];
        st.C[0] = o.x; st.C[1] = o.y; st.C[2] = o.z; st.T = o.w;
        if (depth) st.D = depth[pid];
        const uint32_t nc = (uint32_t)n_contrib[pid];
        st.last = (int)(nc & 0x7fffffffu);
        st.done = (int)(nc >> 31);
    }

    if (rounds > 0) blend_issue(sm, 0, splats, vals, range.x, min(BLEND_BATCH, total), false, range.y, n_vis, counters);
    int pending = rounds > 0 ? 0 : -1;  // stage with a copy in flight that has not been waited for
    bool failed = false;
    for (int b = 0; b < rounds; ++b) {
        const int stage = b & 1;
        const int cnt = min(BLEND_BATCH, total - b * BLEND_BATCH);
        if (b + 1 < rounds) {
            rgs_fence_proxy_async();
            blend_issue(sm, stage ^ 1, splats, vals, range.x + (b + 1) * BLEND_BATCH,
                        min(BLEND_BATCH, total - (b + 1) * BLEND_BATCH), false, range.y, n_vis, counters);
        }
        if (!rgs_mbar_wait(&sm.bar[stage], (b >> 1) & 1, RGS_WAIT_LIMIT)) failed = true;
        pending = (b + 1 < rounds) ? (stage ^ 1) : -1;
        if (!failed) {
            // Warp-level culling: the 32 lanes test 32 splats of the batch against the warp's 8x4 pixel block (exact
            // minimum of the quadratic form over the strip, the rule of rgs_tile_hit), then all lanes walk only the
            // splats that can reach the strip, in order. A skipped splat fails the per-pixel test at every pixel of the
            // strip, so no output bit changes.
            for (int g0 = 0; g0 < cnt; g0 += 32) {
                if (__all_sync(0xffffffffu, st.done)) break;
                bool reach = false;
                if (g0 + lane < cnt) {
                    const RgsSplat& sp = sm.buf[stage][g0 + lane];
                    reach = rgs_rect_hit(sp.px, sp.py, sp.ca, sp.cb, sp.cc, -2.0f * sp.pmin, strip_x0, strip_y0, strip_x1,
                                         strip_y1);
                }
                uint32_t m = __ballot_sync(0xffffffffu, reach);
                while (m) {
                    const int j = g0 + __ffs(m) - 1;
                    m &= m - 1;
                    if (!st.done) {
                        st.contributor = first_contrib + b * BLEND_BATCH + j;
                        rgs_blend_fwd_step(cam, ray, pixx, pixy, sm.buf[stage][j], st);
                    }
                }
            }
        }
        // also the barrier that frees this stage for the copy issued two rounds later
        const int ndone = __syncthreads_count(st.done || failed);
        if (ndone == 256) {
            if (pending >= 0) rgs_mbar_wait(&sm.bar[pending], ((b + 1) >> 1) & 1, RGS_WAIT_LIMIT);
            break;
        }
    }
    if (failed && tid == 0) atomicOr(&counters[RGS_CNT_STATUS], 1u);
    if (slab.mode == RGS_SLAB_NEAR) {
        // a tile whose every pixel is finished needs no instance of the far slab; neither does a tile that nearer
        // sub-models have finished already
        const int all_done = __syncthreads_and(st.done);
        if (tid == 0) slab.tile_done[tile] = (all_done || (slab.occl && slab.occl[tile])) ? 1 : 0;
    } else if (slab.mode == RGS_SLAB_FAR && slab.tile_done) {
        // final state of the tile: what sub-models behind this one may skip
        const int all_done = __syncthreads_and(st.done);
        if (tid == 0 && all_done) slab.tile_done[tile] = 1;
    }
    if (inside) {
        const int64_t pid = (int64_t)py * cam.W + px;
        // what the near slab leaves is resumed by the far slab; a final value carries the finished mark for the compositor
        const float4 val = make_float4(st.C[0], st.C[1], st.C[2],
                                       slab.mode == RGS_SLAB_NEAR ? st.T : rgs_mark_finished(st.T, st.done));
        out[pid] = val;
        if (depth) depth[pid] = st.D;
        // between the two launches the finished flag travels in the top bit
        n_contrib[pid] = slab.mode == RGS_SLAB_NEAR ? (int32_t)((uint32_t)st.last | ((uint32_t)(st.done ? 1 : 0) << 31)) : st.last;
        // epilogue push: the finished pixel goes straight into the slot of every rank that composites
        // this row (plain stores; the destination may be another GPU's memory mapped over NVLink)
        for (int o = 0; o < push.n; ++o)
            if (py >= push.row0[o] && py < push.row1[o])
                push.dst[o][(int64_t)(py - push.row0[o]) * cam.W + px] = val;
    }
}

// ---------------------------------------------------------------------------------------------
// blend backward
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// FIXED: the cross-warp / cross-tile accumulation goes through 64-bit fixed-point integers (scale 2^40) instead of
// float atomics. Integer addition is associative, so the result no longer depends on the order in which tiles and
// warps arrive: two runs give identical bits, which separates a race from rounding when gradients disagree.
#define RGS_FIXED_SCALE 1099511627776.0  // 2^40: resolution 9e-13, range +-8.4e6
// DEPTH: the depth output carries a gradient (grad_depth, one float per pixel); a tenth value per splat is reduced.
template <bool FIXED, bool DEPTH = false>
__global__ void __launch_bounds__(256) rgs_blend_bwd_kernel(
    const __grid_constant__ RgsCamera cam, const int2* __restrict__ ranges, const uint32_t* __restrict__ vals,
    const RgsSplat* __restrict__ splats, const float4* __restrict__ out, const int32_t* __restrict__ n_contrib,
    const float4* __restrict__ grad_out, RgsSplatGrad* __restrict__ splat_grads, uint32_t* __restrict__ counters,
    unsigned long long* __restrict__ fixed_acc, const __grid_constant__ RgsSlabArgs slab,
    const float* __restrict__ grad_depth = nullptr) {
    __shared__ __align__(128) BlendSmem sm;
    __shared__ uint32_t sm_slot[2][BLEND_BATCH];
    const int tid = threadIdx.x, lane = tid & 31;
    const int bx = (tid >> 5) & 1, by = tid >> 6;  // 8x4 block per warp, as in the forward
    const int lx = bx * 8 + (tid & 7), ly = by * 4 + ((tid >> 3) & 3);
    const int px = blockIdx.x * RGS_TILE + lx, py = blockIdx.y * RGS_TILE + ly;
    const bool inside = px < cam.W && py < cam.H;
    const int tile = blockIdx.y * cam.tiles_x + blockIdx.x;
    // the tile's list is the near slab's range followed by the far slab's (empty without slabs)
    const int2 range = checked_range(ranges[tile], counters);
    const int2 range_b = slab.ranges_b ? checked_range(slab.ranges_b[tile], counters, RGS_CNT_INST2, slab.base_b)
                                       : make_int2(0, 0);
    const int len_a = range.y - range.x, len_b = range_b.y - range_b.x;
    const uint32_t n_vis = counters[RGS_CNT_VIS];
    const int64_t pid = (int64_t)py * cam.W + px;
    // a pixel whose incoming gradient is exactly zero (outside the loss rows, or behind saturated nearer sub-models)
    // adds nothing to any splat: it replays nothing, and a tile of such pixels ends here
    const float4 g_pix = inside ? grad_out[pid] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float gd_pix = (DEPTH && inside) ? grad_depth[pid] : 0.f;
    const bool g_live = g_pix.x != 0.f || g_pix.y != 0.f || g_pix.z != 0.f || g_pix.w != 0.f || gd_pix != 0.f;
    const int last = (inside && g_live) ? n_contrib[pid] : 0;
    // only the first max(last) instances of the tile contributed to any pixel
    __shared__ int sm_max_last;
    if (tid == 0) { sm_max_last = 0; rgs_mbar_init(&sm.bar[0], 1); rgs_mbar_init(&sm.bar[1], 1); rgs_fence_mbar_init(); }
    __syncthreads();
    {
        int m = last;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, d));
        if (lane == 0) atomicMax(&sm_max_last, m);
    }
    __syncthreads();
    const int total = min(sm_max_last, len_a + len_b);  // replay positions [0, total) of the list back to front
    const int rounds = (total + BLEND_BATCH - 1) / BLEND_BATCH;

    const float pixx = (float)px, pixy = (float)py;
    RgsPixelRay ray;
    rgs_pixel_ray(cam, pixx, pixy, ray);
    RgsPixelBwd st;
    {
        float4 o = inside ? out[pid] : make_float4(0.f, 0.f, 0.f, 1.f);
        float gC[3] = {g_pix.x, g_pix.y, g_pix.z};
        rgs_pixel_bwd_init(st, o.w, gC, g_pix.w);
    }
    RgsPixelBwdDepth dep = {0.f, 0.f, gd_pix};
    auto issue = [&](int b) {
        const int stage = b & 1;
        const int cnt = min(BLEND_BATCH, total - b * BLEND_BATCH);
        if (tid == 0) rgs_mbar_expect_tx(&sm.bar[stage], (uint32_t)cnt * (uint32_t)sizeof(RgsSplat));
        if (tid < cnt) {
            const int v = total - 1 - b * BLEND_BATCH - tid;  // position in the concatenated list
            const int idx = v < len_a ? range.x + v : range_b.x + (v - len_a);
            const uint32_t slot = checked_slot(vals[idx], n_vis, counters);
            sm_slot[stage][tid] = slot;
            rgs_bulk_g2s(&sm.buf[stage][tid], splats + slot, (uint32_t)sizeof(RgsSplat), &sm.bar[stage]);
        }
    };
    if (rounds > 0) issue(0);
    bool failed = false;
    int warp_last = last;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) warp_last = max(warp_last, __shfl_xor_sync(0xffffffffu, warp_last, d));
    const float strip_x0 = (float)(blockIdx.x * RGS_TILE + bx * 8), strip_y0 = (float)(blockIdx.y * RGS_TILE + by * 4);
    const float strip_x1 = fminf(strip_x0 + 7.0f, (float)(cam.W - 1)), strip_y1 = fminf(strip_y0 + 3.0f, (float)(cam.H - 1));
    for (int b = 0; b < rounds; ++b) {
        const int stage = b & 1;
        const int cnt = min(BLEND_BATCH, total - b * BLEND_BATCH);
        if (b + 1 < rounds) { rgs_fence_proxy_async(); issue(b + 1); }
        if (!rgs_mbar_wait(&sm.bar[stage], (b >> 1) & 1, RGS_WAIT_LIMIT)) failed = true;
        __syncthreads();  // sm_slot of this stage is visible to all
        if (!failed) {
          for (int g0 = 0; g0 < cnt; g0 += 32) {
            // warp-level culling as in the forward; splats beyond the last contributor of every pixel of the strip are
            // skipped as well
            bool reach = false;
            if (g0 + lane < cnt && total - (b * BLEND_BATCH + g0 + lane) <= warp_last) {
                const RgsSplat& sp = sm.buf[stage][g0 + lane];
                reach = rgs_rect_hit(sp.px, sp.py, sp.ca, sp.cb, sp.cc, -2.0f * sp.pmin, strip_x0, strip_y0, strip_x1, strip_y1);
            }
            uint32_t reach_mask = __ballot_sync(0xffffffffu, reach);
            while (reach_mask) {
                const int j = g0 + __ffs(reach_mask) - 1;
                reach_mask &= reach_mask - 1;
                const int contributor = total - (b * BLEND_BATCH + j);  // 1-based index of this instance in the tile list
                RgsSplatGrad g;
                bool hit = false;
                if (contributor <= last) hit = rgs_blend_bwd_step(cam, ray, pixx, pixy, sm.buf[stage][j], st, g, DEPTH ? &dep : nullptr);
                if (!__any_sync(0xffffffffu, hit)) continue;
                // Reduce 8 of the 9 values with a transposing butterfly: at every step a lane keeps half of its values
                // and hands the other half to its partner, so the 8 sums cost 4+2+1+1+1 = 9 shuffles instead of 40;
                // lane 4k ends up with the total of value k. The ninth value takes the plain 5-step reduction.
                float v[8] = {g.dpx, g.dpy, g.dca, g.dcb, g.dcc, g.dopacity, g.dr, g.dg};
                float v8 = hit ? g.db : 0.f;
                if (!hit) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = 0.f;
                }
                float w4[4], w2[2], w1;
                {
                    const bool up = lane & 16;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float send = up ? v[k] : v[k + 4], keep = up ? v[k + 4] : v[k];
                        w4[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                    }
                }
                {
                    const bool up = lane & 8;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const float send = up ? w4[k] : w4[k + 2], keep = up ? w4[k + 2] : w4[k];
                        w2[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                }
                {
                    const bool up = lane & 4;
                    const float send = up ? w2[0] : w2[1], keep = up ? w2[1] : w2[0];
                    w1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                }
                w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
                w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
                v8 = warp_sum(v8);
                float v9 = 0.f;
                if (DEPTH) v9 = warp_sum(hit ? g.ddepth : 0.f);
                // value index held by this lane: bit 16 -> +4, bit 8 -> +2, bit 4 -> +1
                const int which = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                if (FIXED) {
                    unsigned long long* dst = fixed_acc + (size_t)sm_slot[stage][j] * 9;
                    if ((lane & 3) == 0) atomicAdd(dst + which, (unsigned long long)__double2ll_rn((double)w1 * RGS_FIXED_SCALE));
                    if (lane == 0) atomicAdd(dst + 8, (unsigned long long)__double2ll_rn((double)v8 * RGS_FIXED_SCALE));
                } else {
                    float* dst = reinterpret_cast<float*>(splat_grads + sm_slot[stage][j]);
                    if ((lane & 3) == 0) atomicAdd(dst + which, w1);
                    if (lane == 0) atomicAdd(dst + 8, v8);
                    if (DEPTH && lane == 1) atomicAdd(dst + 9, v9);
                }
            }
          }
        }
        __syncthreads();  // frees this stage for the copy issued two rounds later
    }
    if (failed && tid == 0) atomicOr(&counters[RGS_CNT_STATUS], 2u);
}

__global__ void __launch_bounds__(256) rgs_fixed_fold_kernel(long long* __restrict__ fixed_acc, int64_t cap_vis,
                                                             const uint32_t* __restrict__ counters,
                                                             RgsSplatGrad* __restrict__ splat_grads) {
    int64_t n = counters[RGS_CNT_OVERFLOW] ? 0 : (int64_t)counters[RGS_CNT_VIS];
    if (n > cap_vis) n = cap_vis;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n * 9; e += (int64_t)gridDim.x * blockDim.x) {
        const long long v = fixed_acc[e];
        if (v == 0) continue;
        fixed_acc[e] = 0;
        const int64_t slot = e / 9;
        reinterpret_cast<float*>(splat_grads + slot)[e - slot * 9] += (float)((double)v / RGS_FIXED_SCALE);
    }
}

// ---------------------------------------------------------------------------------------------
// geometry backward: one thread per visible splat
// ---------------------------------------------------------------------------------------------
struct RgsSegments { RgsSegment s[4]; int n; };

__global__ void __launch_bounds__(128, 8) rgs_geom_bwd_kernel(
    const __grid_constant__ RgsCamera cam, const __grid_constant__ RgsSegments segs,
    const uint32_t* __restrict__ counters, const int32_t* __restrict__ vis_ids, const uint32_t* __restrict__ aux,
    const RgsSplatGrad* __restrict__ splat_grads) {
    if (counters[RGS_CNT_OVERFLOW]) return;
    const uint32_t n_vis = counters[RGS_CNT_VIS];
    for (uint32_t slot = blockIdx.x * blockDim.x + threadIdx.x; slot < n_vis; slot += gridDim.x * blockDim.x) {
        int64_t i = vis_ids[slot];
        int sidx = 0;
        while (sidx < segs.n - 1 && i >= segs.s[sidx].count) { i -= segs.s[sidx].count; ++sidx; }
        const RgsSegment& sg = segs.s[sidx];
        if (i < 0 || i >= sg.count) {  // a corrupt id would address another buffer: report and skip
            atomicOr(const_cast<uint32_t*>(&counters[RGS_CNT_STATUS]), RGS_STATUS_BAD_INDEX);
            continue;
        }
        const uint32_t a = aux[slot];
        const float4* gsrc = reinterpret_cast<const float4*>(splat_grads + slot);
        float4 g0 = gsrc[0], g1 = gsrc[1], g2 = gsrc[2];
        RgsSplatGrad g;
        g.dpx = g0.x; g.dpy = g0.y; g.dca = g0.z; g.dcb = g0.w;
        g.dcc = g1.x; g.dopacity = g1.y; g.dr = g1.z; g.dg = g1.w;
        g.db = g2.x; g.ddepth = g2.y; g.pad0 = 0.f; g.pad1 = 0.f;
        // A visible splat that no pixel blended (it lies behind saturated pixels) has exactly zero image-space
        // gradients, hence exactly zero parameter gradients: only its visibility statistics change, and its
        // gradient row stays untouched (which the optimiser exploits as well).
        if (g0.x == 0.f && g0.y == 0.f && g0.z == 0.f && g0.w == 0.f && g1.x == 0.f && g1.y == 0.f && g1.z == 0.f &&
            g1.w == 0.f && g2.x == 0.f && g2.y == 0.f) {
            if (sg.g_mean2d) { sg.g_mean2d[2 * i] = 0.f; sg.g_mean2d[2 * i + 1] = 0.f; }
            if (sg.stat_denom) sg.stat_denom[i] += 1.0f;
            if (sg.stat_maxrad) sg.stat_maxrad[i] = fmaxf(sg.stat_maxrad[i], (float)(a >> 3));
            continue;
        }
        float p[3] = {sg.xyz[3 * i], sg.xyz[3 * i + 1], sg.xyz[3 * i + 2]};
        float s[3] = {sg.scale[3 * i], sg.scale[3 * i + 1], sg.scale[3 * i + 2]};
        float4 q4 = reinterpret_cast<const float4*>(sg.rot)[i];
        float q[4] = {q4.x, q4.y, q4.z, q4.w};
        float gx[3] = {0.f, 0.f, 0.f}, gs[3] = {0.f, 0.f, 0.f}, gq[4] = {0.f, 0.f, 0.f, 0.f}, go[1] = {0.f};
        // SH gradients are outer products basis[k] * gc[c]: formed on the fly when written (no 48-float array)
        float basis[16], gc[3];
        const float nrm = rgs_project_bwd(cam, p, s, q, sg.opacity[i], sg.sh + 48 * i, a & 7u, g, gx, nullptr, gs, gq, go,
                                          basis, gc);
        // first writer of this row in this step stores, later ones (other views of the batch) add
        bool first = false;
        if (sg.touched) { first = sg.touched[i] == 0; if (first) sg.touched[i] = 1; }
        if (sg.g_xyz) {
            if (first) { sg.g_xyz[3 * i] = gx[0]; sg.g_xyz[3 * i + 1] = gx[1]; sg.g_xyz[3 * i + 2] = gx[2]; }
            else { sg.g_xyz[3 * i] += gx[0]; sg.g_xyz[3 * i + 1] += gx[1]; sg.g_xyz[3 * i + 2] += gx[2]; }
        }
        if (sg.g_scale) {
            if (first) { sg.g_scale[3 * i] = gs[0]; sg.g_scale[3 * i + 1] = gs[1]; sg.g_scale[3 * i + 2] = gs[2]; }
            else { sg.g_scale[3 * i] += gs[0]; sg.g_scale[3 * i + 1] += gs[1]; sg.g_scale[3 * i + 2] += gs[2]; }
        }
        if (sg.g_rot) {
            float4* d = reinterpret_cast<float4*>(sg.g_rot) + i;
            float4 o = first ? make_float4(0.f, 0.f, 0.f, 0.f) : *d;
            o.x += gq[0]; o.y += gq[1]; o.z += gq[2]; o.w += gq[3];
            *d = o;
        }
        if (sg.g_opacity) { if (first) sg.g_opacity[i] = go[0]; else sg.g_opacity[i] += go[0]; }
        if (sg.g_sh) {
            const int nc4 = ((cam.sh_degree + 1) * (cam.sh_degree + 1) * 3 + 3) / 4;
            float4* d = reinterpret_cast<float4*>(sg.g_sh + 48 * i);
#pragma unroll
            for (int k = 0; k < 12; ++k) {
                if (k < nc4) {
                    float4 o = first ? make_float4(0.f, 0.f, 0.f, 0.f) : d[k];
                    // element e = 3*coef + channel
                    o.x += basis[(4 * k) / 3] * gc[(4 * k) % 3];
                    o.y += basis[(4 * k + 1) / 3] * gc[(4 * k + 1) % 3];
                    o.z += basis[(4 * k + 2) / 3] * gc[(4 * k + 2) % 3];
                    o.w += basis[(4 * k + 3) / 3] * gc[(4 * k + 3) % 3];
                    d[k] = o;
                }
            }
        }
        if (sg.g_mean2d) { sg.g_mean2d[2 * i] = g.dpx * 0.5f * cam.W; sg.g_mean2d[2 * i + 1] = g.dpy * 0.5f * cam.H; }
        if (sg.stat_grad) sg.stat_grad[i] += nrm;
        if (sg.stat_denom) sg.stat_denom[i] += 1.0f;
        if (sg.stat_maxrad) sg.stat_maxrad[i] = fmaxf(sg.stat_maxrad[i], (float)(a >> 3));
    }
}

__global__ void rgs_scatter_radii_kernel(const uint32_t* __restrict__ counters, const int32_t* __restrict__ vis_ids,
                                         const uint32_t* __restrict__ aux, int64_t id_base, int64_t count,
                                         int32_t* __restrict__ radii) {
    if (counters[RGS_CNT_OVERFLOW]) return;
    const uint32_t n_vis = counters[RGS_CNT_VIS];
    for (uint32_t s = blockIdx.x * blockDim.x + threadIdx.x; s < n_vis; s += gridDim.x * blockDim.x) {
        int64_t i = (int64_t)vis_ids[s] - id_base;
        if (i >= 0 && i < count) radii[i] = (int32_t)(aux[s] >> 3);
    }
}

// ---------------------------------------------------------------------------------------------
// host entry points
// ---------------------------------------------------------------------------------------------
extern "C" {

int rgs_cuda_project_emit(const RgsCamera* cam, const RgsSegment* seg, int64_t id_base, RgsSplat* splats,
                          int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint64_t* keys, uint32_t* vals,
                          int64_t cap_inst, int32_t* counters, RgsSplatGrad* splat_grads, void* stream) {
    if (seg->count <= 0) return 0;
    if (cap_inst > 0xfffffff0ll || cap_vis > 0x7ffffff0ll) return 10;
    if ((uintptr_t)seg->sh & 15u) return 14;  // SH rows are read as 128-bit words
    const unsigned blocks = (unsigned)((seg->count + 255) / 256);
    rgs_project_emit_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
        *cam, *seg, id_base, splats, vis_ids, aux, (uint32_t)cap_vis, keys, vals, (uint32_t)cap_inst,
        reinterpret_cast<uint32_t*>(counters), splat_grads);
    return (int)cudaGetLastError();
}

int rgs_cuda_blend_fwd(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                       float* out, float* depth, int32_t* n_contrib, int32_t* counters, void* stream) {
    dim3 grid(cam->tiles_x, cam->tiles_y);
    RgsPushPlan push;
    push.n = 0;
    rgs_blend_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges), vals, splats, reinterpret_cast<float4*>(out), depth, n_contrib,
        reinterpret_cast<uint32_t*>(counters), push, RgsSlabArgs{nullptr, nullptr, 0u, RGS_SLAB_SINGLE, nullptr});
    return (int)cudaGetLastError();
}

// Blend forward with the fused push: besides the local (H,W,4) image, rows [row0[o],row1[o]) are stored
// into dst[o] for o < n_dst (slot bases, local or peer-mapped).
int rgs_cuda_blend_fwd_push(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                            float* out, float* depth, int32_t* n_contrib, int32_t* counters, int64_t n_dst,
                            const int32_t* row0, const int32_t* row1, float* const* dst, void* stream) {
    if (n_dst < 0 || n_dst > RGS_MAX_PUSH) return 15;
    dim3 grid(cam->tiles_x, cam->tiles_y);
    RgsPushPlan push;
    push.n = (int)n_dst;
    for (int o = 0; o < n_dst; ++o) { push.row0[o] = row0[o]; push.row1[o] = row1[o]; push.dst[o] = reinterpret_cast<float4*>(dst[o]); }
    rgs_blend_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges), vals, splats, reinterpret_cast<float4*>(out), depth, n_contrib,
        reinterpret_cast<uint32_t*>(counters), push, RgsSlabArgs{nullptr, nullptr, 0u, RGS_SLAB_SINGLE, nullptr});
    return (int)cudaGetLastError();
}

// One launch of the two-slab forward. mode 1 (near slab): ranges_a is walked, tile_done is written, no push.
// mode 2 (far slab): resumes from out / depth / n_contrib, walks ranges_b (indices from base_b on), pushes.
// occl (near launch, optional): one byte per tile, tiles finished by nearer sub-models; they are marked done as well.
int rgs_cuda_blend_fwd_slab(const RgsCamera* cam, const int32_t* ranges_a, const int32_t* ranges_b, const uint32_t* vals,
                            const RgsSplat* splats, float* out, float* depth, int32_t* n_contrib, int32_t* counters,
                            uint8_t* tile_done, int64_t base_b, int64_t mode, int64_t n_dst, const int32_t* row0,
                            const int32_t* row1, float* const* dst, const uint8_t* occl, void* stream) {
    if (n_dst < 0 || n_dst > RGS_MAX_PUSH || (mode != RGS_SLAB_NEAR && mode != RGS_SLAB_FAR)) return 15;
    dim3 grid(cam->tiles_x, cam->tiles_y);
    RgsPushPlan push;
    push.n = mode == RGS_SLAB_FAR ? (int)n_dst : 0;
    for (int o = 0; o < push.n; ++o) { push.row0[o] = row0[o]; push.row1[o] = row1[o]; push.dst[o] = reinterpret_cast<float4*>(dst[o]); }
    rgs_blend_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges_a), vals, splats, reinterpret_cast<float4*>(out), depth, n_contrib,
        reinterpret_cast<uint32_t*>(counters), push,
        RgsSlabArgs{reinterpret_cast<const int2*>(ranges_b), tile_done, (uint32_t)base_b, (int)mode,
                    mode == RGS_SLAB_NEAR ? occl : nullptr});
    return (int)cudaGetLastError();
}

int rgs_cuda_blend_bwd(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                       const float* out, const int32_t* n_contrib, const float* grad_out, RgsSplatGrad* splat_grads,
                       int32_t* counters, void* stream) {
    dim3 grid(cam->tiles_x, cam->tiles_y);
    rgs_blend_bwd_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges), vals, splats, reinterpret_cast<const float4*>(out), n_contrib,
        reinterpret_cast<const float4*>(grad_out), splat_grads, reinterpret_cast<uint32_t*>(counters), nullptr,
        RgsSlabArgs{nullptr, nullptr, 0u, RGS_SLAB_SINGLE, nullptr});
    return (int)cudaGetLastError();
}

// Backward with a gradient on the depth output as well (grad_depth: H*W floats): the path of the autograd interface.
int rgs_cuda_blend_bwd_depth(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                             const float* out, const int32_t* n_contrib, const float* grad_out, const float* grad_depth,
                             RgsSplatGrad* splat_grads, int32_t* counters, void* stream) {
    dim3 grid(cam->tiles_x, cam->tiles_y);
    if (!grad_depth) return rgs_cuda_blend_bwd(cam, ranges, vals, splats, out, n_contrib, grad_out, splat_grads, counters, stream);
    rgs_blend_bwd_kernel<false, true><<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges), vals, splats, reinterpret_cast<const float4*>(out), n_contrib,
        reinterpret_cast<const float4*>(grad_out), splat_grads, reinterpret_cast<uint32_t*>(counters), nullptr,
        RgsSlabArgs{nullptr, nullptr, 0u, RGS_SLAB_SINGLE, nullptr}, grad_depth);
    return (int)cudaGetLastError();
}

// Backward of a two-slab render: the list of a tile is ranges_a followed by ranges_b. fixed_acc (nullable) selects the
// order-independent accumulation (see rgs_cuda_blend_bwd_fixed).
int rgs_cuda_blend_bwd_slab(const RgsCamera* cam, const int32_t* ranges_a, const int32_t* ranges_b, int64_t base_b,
                            const uint32_t* vals, const RgsSplat* splats, const float* out, const int32_t* n_contrib,
                            const float* grad_out, RgsSplatGrad* splat_grads, int32_t* counters, int64_t* fixed_acc,
                            int64_t cap_vis, const float* grad_depth, void* stream) {
    dim3 grid(cam->tiles_x, cam->tiles_y);
    const RgsSlabArgs slab{reinterpret_cast<const int2*>(ranges_b), nullptr, (uint32_t)base_b, RGS_SLAB_SINGLE, nullptr};
    if (grad_depth) {  // gradient on the depth output as well (float accumulation only)
        if (fixed_acc) return 15;
        rgs_blend_bwd_kernel<false, true><<<grid, 256, 0, (cudaStream_t)stream>>>(
            *cam, reinterpret_cast<const int2*>(ranges_a), vals, splats, reinterpret_cast<const float4*>(out), n_contrib,
            reinterpret_cast<const float4*>(grad_out), splat_grads, reinterpret_cast<uint32_t*>(counters), nullptr, slab,
            grad_depth);
        return (int)cudaGetLastError();
    }
    if (!fixed_acc) {
        rgs_blend_bwd_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(
            *cam, reinterpret_cast<const int2*>(ranges_a), vals, splats, reinterpret_cast<const float4*>(out), n_contrib,
            reinterpret_cast<const float4*>(grad_out), splat_grads, reinterpret_cast<uint32_t*>(counters), nullptr, slab);
        return (int)cudaGetLastError();
    }
    rgs_blend_bwd_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges_a), vals, splats, reinterpret_cast<const float4*>(out), n_contrib,
        reinterpret_cast<const float4*>(grad_out), splat_grads, reinterpret_cast<uint32_t*>(counters),
        reinterpret_cast<unsigned long long*>(fixed_acc), slab);
    const int64_t want = (cap_vis * 9 + 255) / 256;
    const unsigned blocks = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 32 ? RGS_SMS * 32 : want));
    rgs_fixed_fold_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<long long*>(fixed_acc), cap_vis,
                                                                   reinterpret_cast<const uint32_t*>(counters), splat_grads);
    return (int)cudaGetLastError();
}

// Debug variant with order-independent accumulation. fixed_acc: 9 int64 words per slot (cap_vis slots), all zero on
// entry; they are folded into splat_grads (added to what it holds) and zeroed again before the call returns control
// to the stream.
int rgs_cuda_blend_bwd_fixed(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                             const float* out, const int32_t* n_contrib, const float* grad_out, RgsSplatGrad* splat_grads,
                             int32_t* counters, int64_t* fixed_acc, int64_t cap_vis, void* stream) {
    dim3 grid(cam->tiles_x, cam->tiles_y);
    rgs_blend_bwd_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(
        *cam, reinterpret_cast<const int2*>(ranges), vals, splats, reinterpret_cast<const float4*>(out), n_contrib,
        reinterpret_cast<const float4*>(grad_out), splat_grads, reinterpret_cast<uint32_t*>(counters),
        reinterpret_cast<unsigned long long*>(fixed_acc), RgsSlabArgs{nullptr, nullptr, 0u, RGS_SLAB_SINGLE, nullptr});
    const int64_t want = (cap_vis * 9 + 255) / 256;
    const unsigned blocks = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 32 ? RGS_SMS * 32 : want));
    rgs_fixed_fold_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<long long*>(fixed_acc), cap_vis,
                                                                   reinterpret_cast<const uint32_t*>(counters), splat_grads);
    return (int)cudaGetLastError();
}

int rgs_cuda_geom_bwd(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, const int32_t* counters,
                      const RgsSplat* splats, const int32_t* vis_ids, const uint32_t* aux,
                      const RgsSplatGrad* splat_grads, int64_t cap_vis, void* stream) {
    (void)splats;
    if (nseg < 1 || nseg > 4) return 11;
    RgsSegments s;
    s.n = (int)nseg;
    for (int k = 0; k < (int)nseg; ++k) s.s[k] = segs[k];
    const int64_t want = (cap_vis + 127) / 128;
    const unsigned blocks = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 16 ? RGS_SMS * 16 : want));
    rgs_geom_bwd_kernel<<<blocks, 128, 0, (cudaStream_t)stream>>>(*cam, s, reinterpret_cast<const uint32_t*>(counters),
                                                                 vis_ids, aux, splat_grads);
    return (int)cudaGetLastError();
}

int rgs_cuda_scatter_radii(const int32_t* counters, const int32_t* vis_ids, const uint32_t* aux, int64_t id_base,
                           int64_t count, int32_t* radii, void* stream) {
    rgs_scatter_radii_kernel<<<(unsigned)(RGS_SMS * 4), 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint32_t*>(counters),
                                                                         vis_ids, aux, id_base, count, radii);
    return (int)cudaGetLastError();
}

}  // extern "C"
