// Native CPU backend: OpenMP loops around the math that the sm_100a kernels use (rgs_math.h).
//
// It serves three purposes: (1) the rasteriser of CPU/gloo ranks, so that every multi-rank code
// path can run on a machine without a GPU; (2) the validation vehicle for the shared math
// against a PyTorch-autograd restatement; (3) the timed CPU baseline.
// The reference has no CPU path at all (its rasteriser is CUDA-only:
// rasterization_kernels/diff-gaussian-rasterization-half-gaussian/cuda_rasterizer_hgs/).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>
#include <vector>
#include "rgs_api.h"
#include "rgs_loss_math.h"
#include "rgs_knn.h"
#include "rgs_surgery.h"
#include "rgs_border.h"

extern "C" {

int rgs_cpu_project_emit(const RgsCamera* cam, const RgsSegment* seg, int64_t id_base, RgsSplat* splats,
                         int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint64_t* keys, uint32_t* vals,
                         int64_t cap_inst, int32_t* counters, RgsSplatGrad* splat_grads, void*) {
    int64_t n_vis = counters[RGS_CNT_VIS], n_inst = counters[RGS_CNT_INST];
    for (int64_t i = 0; i < seg->count; ++i) {
        RgsSplat sp; RgsRect rc; int radius; unsigned clamped;
        if (!rgs_project(*cam, seg->xyz + 3 * i, seg->scale + 3 * i, seg->rot + 4 * i, seg->opacity[i],
                         seg->sh + 48 * i, sp, rc, radius, clamped))
            continue;
        if (n_vis >= cap_vis) { counters[RGS_CNT_OVERFLOW] = 1; continue; }
        int64_t cnt = (int64_t)(rc.x1 - rc.x0) * (rc.y1 - rc.y0);
        int64_t base = n_inst;
        n_inst += cnt;
        if (n_inst > cap_inst) { counters[RGS_CNT_OVERFLOW] = 1; continue; }
        int64_t slot = n_vis++;
        splats[slot] = sp;
        vis_ids[slot] = (int32_t)(id_base + i);
        aux[slot] = ((uint32_t)radius << 3) | clamped;
        if (splat_grads) std::memset(&splat_grads[slot], 0, sizeof(RgsSplatGrad));
        uint32_t dbits; std::memcpy(&dbits, &sp.depth, 4);
        for (int y = rc.y0; y < rc.y1; ++y)
            for (int x = rc.x0; x < rc.x1; ++x) {
                uint64_t key = (uint64_t)(y * cam->tiles_x + x);
                keys[base] = (key << 32) | dbits;
                vals[base] = (uint32_t)slot;
                ++base;
            }
    }
    counters[RGS_CNT_VIS] = (int32_t)n_vis;
    counters[RGS_CNT_INST] = (int32_t)std::min<int64_t>(n_inst, 0x7fffffff);
    return 0;
}

int64_t rgs_cpu_sort_scratch_words(int64_t) { return 1; }
int64_t rgs_cpu_bin_scratch_words(int64_t, int64_t) { return 1; }

// CPU twins of the depth-ordered binning (rgs_binning.cu)
int rgs_cpu_project_slots(const RgsCamera* cam, const RgsSegment* seg, int64_t id_base, RgsSplat* splats,
                          int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth, uint32_t* slot_rect,
                          uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads, void*) {
    int64_t n_vis = counters[RGS_CNT_VIS];
    for (int64_t i = 0; i < seg->count; ++i) {
        RgsSplat sp; RgsRect rc; int radius; unsigned clamped;
        if (!rgs_project(*cam, seg->xyz + 3 * i, seg->scale + 3 * i, seg->rot + 4 * i, seg->opacity[i],
                         seg->sh ? seg->sh + 48 * i : nullptr, sp, rc, radius, clamped))
            continue;
        if (n_vis >= cap_vis) { counters[RGS_CNT_OVERFLOW] = 1; continue; }
        int64_t slot = n_vis++;
        splats[slot] = sp;
        vis_ids[slot] = (int32_t)(id_base + i);
        aux[slot] = ((uint32_t)radius << 3) | clamped;
        std::memcpy(&slot_depth[slot], &sp.depth, 4);
        slot_rect[2 * slot] = (uint32_t)rc.x0 | ((uint32_t)rc.y0 << 16);
        slot_rect[2 * slot + 1] = (uint32_t)rc.x1 | ((uint32_t)rc.y1 << 16);
        uint32_t hits = 0;
        const float bound = rgs_alpha_bound(sp.opacity);
        for (int y = rc.y0; y < rc.y1; ++y)
            for (int x = rc.x0; x < rc.x1; ++x)
                hits += (cam->tight_rect < 2 || rgs_tile_hit(sp.px, sp.py, sp.ca, sp.cb, sp.cc, bound, x, y, cam->W, cam->H)) ? 1u : 0u;
        slot_cnt[slot] = hits;
        if (splat_grads) std::memset(&splat_grads[slot], 0, sizeof(RgsSplatGrad));
    }
    counters[RGS_CNT_VIS] = (int32_t)n_vis;
    return 0;
}

// Geometry-only variant of rgs_cpu_project_slots2: the colours are filled in later by rgs_cpu_colour_slab for the
// splats that have tile instances.
int rgs_cpu_project_slots2_geom(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, uint32_t*, int64_t,
                                RgsSplat* splats, int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth,
                                uint32_t* slot_rect, uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads,
                                void* stream) {
    int64_t base = 0;
    for (int64_t k = 0; k < nseg; ++k) {
        RgsSegment geo = segs[k];
        geo.sh = nullptr;
        rgs_cpu_project_slots(cam, &geo, base, splats, vis_ids, aux, cap_vis, slot_depth, slot_rect, slot_cnt, counters,
                              splat_grads, stream);
        base += segs[k].count;
    }
    return 0;
}

// Colours of the splats of one slab (depth-ordered positions, see rgs_cpu_bin_slab) whose instance count is not zero.
int rgs_cpu_colour_slab(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, const uint32_t* order,
                        const uint32_t* slot_cnt, const int32_t* counters, int64_t cap_vis, int64_t frac256, int64_t slab,
                        RgsSplat* splats, const int32_t* vis_ids, uint32_t* aux, void*) {
    if (counters[RGS_CNT_OVERFLOW]) return 0;
    const int64_t n = std::min<int64_t>(counters[RGS_CNT_VIS], cap_vis);
    const int64_t seg = 1024, nsegs = (n + seg - 1) / seg;
    const int64_t split = std::min<int64_t>(nsegs, ((n * frac256) >> 8) / seg);
    const int64_t i0 = (slab == 0 ? 0 : split) * seg, i1 = std::min<int64_t>(n, (slab == 0 ? split : nsegs) * seg);
    for (int64_t i = i0; i < i1; ++i) {
        const uint32_t s = order[i];
        if (slot_cnt[s] == 0) continue;
        int64_t id = vis_ids[s];
        const RgsSegment* sg = nullptr;
        for (int64_t k = 0; k < nseg; ++k) {
            if (id < segs[k].count) { sg = &segs[k]; break; }
            id -= segs[k].count;
        }
        if (!sg) continue;
        unsigned clamped = 0;
        rgs_splat_colour(*cam, sg->xyz + 3 * id, sg->sh + 48 * id, splats[s].r, splats[s].g, splats[s].b, clamped);
        aux[s] = (aux[s] & ~7u) | clamped;
    }
    return 0;
}

int rgs_cpu_project_slots2(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, uint32_t*, int64_t,
                           RgsSplat* splats, int32_t* vis_ids, uint32_t* aux, int64_t cap_vis, uint32_t* slot_depth,
                           uint32_t* slot_rect, uint32_t* slot_cnt, int32_t* counters, RgsSplatGrad* splat_grads,
                           void* stream) {
    int64_t base = 0;
    for (int64_t k = 0; k < nseg; ++k) {
        rgs_cpu_project_slots(cam, &segs[k], base, splats, vis_ids, aux, cap_vis, slot_depth, slot_rect, slot_cnt, counters,
                              splat_grads, stream);
        base += segs[k].count;
    }
    return 0;
}

int rgs_cpu_bin_instances(const RgsCamera* cam, const RgsSplat* splats, const uint32_t* slot_depth, const uint32_t* slot_rect,
                          const uint32_t* slot_cnt, int64_t cap_vis, uint32_t*, uint32_t*,
                          uint32_t*, uint32_t*, uint32_t* inst_keys, uint32_t* inst_vals, uint32_t*, uint32_t*,
                          int64_t cap_inst, int32_t* counters, int64_t tiles_x, int64_t num_tiles, int32_t* ranges,
                          uint32_t*, void*) {
    (void)cap_vis;
    std::memset(ranges, 0, num_tiles * 8);
    if (counters[RGS_CNT_OVERFLOW]) return 0;
    const int64_t n = counters[RGS_CNT_VIS];
    std::vector<uint32_t> order(n);
    std::iota(order.begin(), order.end(), 0u);
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return slot_depth[a] < slot_depth[b]; });
    std::vector<std::pair<uint32_t, uint32_t>> inst;
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t s = order[i], lo = slot_rect[2 * s], hi = slot_rect[2 * s + 1];
        if (slot_cnt[s] == 0) continue;
        const RgsSplat& sp = splats[s];
        const float bound = rgs_alpha_bound(sp.opacity);
        for (uint32_t y = lo >> 16; y < (hi >> 16); ++y)
            for (uint32_t x = lo & 0xffff; x < (hi & 0xffff); ++x)
                if (cam->tight_rect < 2 || rgs_tile_hit(sp.px, sp.py, sp.ca, sp.cb, sp.cc, bound, (int)x, (int)y, cam->W, cam->H))
                    inst.emplace_back((uint32_t)(y * tiles_x + x), s);
    }
    counters[RGS_CNT_INST] = (int32_t)std::min<size_t>(inst.size(), 0x7fffffff);
    if ((int64_t)inst.size() > cap_inst) { counters[RGS_CNT_OVERFLOW] = 1; return 0; }
    std::stable_sort(inst.begin(), inst.end(), [](const std::pair<uint32_t, uint32_t>& a, const std::pair<uint32_t, uint32_t>& b) { return a.first < b.first; });
    const int64_t m = (int64_t)inst.size();
    for (int64_t i = 0; i < m; ++i) {
        inst_keys[i] = inst[i].first; inst_vals[i] = inst[i].second;
        const uint32_t t = inst[i].first;
        if (i == 0 || inst[i - 1].first != t) ranges[2 * t] = (int32_t)i;
        if (i == m - 1 || inst[i + 1].first != t) ranges[2 * t + 1] = (int32_t)(i + 1);
    }
    return 0;
}

// Sorts the instances by (tile, depth) and writes [start,end) per tile. The sorted lists end up in
// keys/vals (the *_tmp buffers are scratch, as for the GPU sort).
int rgs_cpu_sort_ranges(uint64_t* keys, uint32_t* vals, uint64_t* keys_tmp, uint32_t* vals_tmp, int64_t cap_inst,
                        const int32_t* counters, int64_t num_tiles, int32_t* ranges, void*, void*) {
    int64_t n = std::min<int64_t>(counters[RGS_CNT_INST], cap_inst);
    if (counters[RGS_CNT_OVERFLOW]) n = 0;
    std::vector<int64_t> idx(n);
    std::iota(idx.begin(), idx.end(), 0);
    std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return keys[a] < keys[b]; });
    for (int64_t i = 0; i < n; ++i) { keys_tmp[i] = keys[idx[i]]; vals_tmp[i] = vals[idx[i]]; }
    std::memcpy(keys, keys_tmp, n * 8);
    std::memcpy(vals, vals_tmp, n * 4);
    std::memset(ranges, 0, num_tiles * 8);
    for (int64_t i = 0; i < n; ++i) {
        int64_t t = (int64_t)(keys[i] >> 32);
        if (i == 0 || (int64_t)(keys[i - 1] >> 32) != t) ranges[2 * t] = (int32_t)i;
        if (i == n - 1 || (int64_t)(keys[i + 1] >> 32) != t) ranges[2 * t + 1] = (int32_t)(i + 1);
    }
    return 0;
}

// out: (H,W,4) premultiplied RGB + transmittance; depth: optional (H,W); n_contrib: (H,W)
int rgs_cpu_blend_fwd(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                      float* out, float* depth, int32_t* n_contrib, int32_t* counters, void*) {
    (void)counters;
    const int W = cam->W, H = cam->H;
#pragma omp parallel for schedule(dynamic, 1)
    for (int tile = 0; tile < cam->tiles_x * cam->tiles_y; ++tile) {
        int tx = tile % cam->tiles_x, ty = tile / cam->tiles_x;
        int r0 = ranges[2 * tile], r1 = ranges[2 * tile + 1];
        for (int ly = 0; ly < RGS_TILE; ++ly)
            for (int lx = 0; lx < RGS_TILE; ++lx) {
                int x = tx * RGS_TILE + lx, y = ty * RGS_TILE + ly;
                if (x >= W || y >= H) continue;
                RgsPixelRay ray; rgs_pixel_ray(*cam, (float)x, (float)y, ray);
                RgsPixelState st; rgs_pixel_init(st);
                for (int i = r0; i < r1 && !st.done; ++i)
                    rgs_blend_fwd_step(*cam, ray, (float)x, (float)y, splats[vals[i]], st);
                int64_t pid = (int64_t)y * W + x;
                out[4 * pid + 0] = st.C[0]; out[4 * pid + 1] = st.C[1]; out[4 * pid + 2] = st.C[2];
                out[4 * pid + 3] = rgs_mark_finished(st.T, st.done);
                if (depth) depth[pid] = st.D;
                n_contrib[pid] = st.last;
            }
    }
    return 0;
}

// CPU twin of the fused push (used by the loopback tests): copies the rows after the render.
int rgs_cpu_blend_fwd_push(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                           float* out, float* depth, int32_t* n_contrib, int32_t* counters, int64_t n_dst,
                           const int32_t* row0, const int32_t* row1, float* const* dst, void* stream) {
    rgs_cpu_blend_fwd(cam, ranges, vals, splats, out, depth, n_contrib, counters, stream);
    for (int64_t o = 0; o < n_dst; ++o)
        if (row1[o] > row0[o])
            std::memcpy(dst[o], out + (int64_t)row0[o] * cam->W * 4, (size_t)(row1[o] - row0[o]) * cam->W * 16);
    return 0;
}

// grad_out: (H,W,4) = dL/dC (rgb), dL/dT. splat_grads[n_vis] must be zeroed by the caller.
// grad_depth (optional, H*W): gradient of the depth output
int rgs_cpu_blend_bwd_depth(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                            const float* out, const int32_t* n_contrib, const float* grad_out, const float* grad_depth,
                            RgsSplatGrad* splat_grads, int32_t* counters, void*) {
    (void)counters;
    const int W = cam->W, H = cam->H;
    // serial over tiles: the accumulation order is then fixed, which makes this path the
    // deterministic reference for the atomically accumulating GPU kernel.
    for (int tile = 0; tile < cam->tiles_x * cam->tiles_y; ++tile) {
        int tx = tile % cam->tiles_x, ty = tile / cam->tiles_x;
        int r0 = ranges[2 * tile];
        for (int ly = 0; ly < RGS_TILE; ++ly)
            for (int lx = 0; lx < RGS_TILE; ++lx) {
                int x = tx * RGS_TILE + lx, y = ty * RGS_TILE + ly;
                if (x >= W || y >= H) continue;
                int64_t pid = (int64_t)y * W + x;
                RgsPixelRay ray; rgs_pixel_ray(*cam, (float)x, (float)y, ray);
                RgsPixelBwd st;
                rgs_pixel_bwd_init(st, out[4 * pid + 3], grad_out + 4 * pid, grad_out[4 * pid + 3]);
                RgsPixelBwdDepth dep = {0.f, 0.f, grad_depth ? grad_depth[pid] : 0.f};
                for (int i = r0 + n_contrib[pid] - 1; i >= r0; --i) {
                    RgsSplatGrad g;
                    uint32_t slot = vals[i];
                    if (!rgs_blend_bwd_step(*cam, ray, (float)x, (float)y, splats[slot], st, g, grad_depth ? &dep : nullptr))
                        continue;
                    float* dst = reinterpret_cast<float*>(&splat_grads[slot]);
                    const float* src = reinterpret_cast<const float*>(&g);
                    for (int k = 0; k < 10; ++k) dst[k] += src[k];
                }
            }
    }
    return 0;
}

int rgs_cpu_blend_bwd(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                      const float* out, const int32_t* n_contrib, const float* grad_out, RgsSplatGrad* splat_grads,
                      int32_t* counters, void*) {
    return rgs_cpu_blend_bwd_depth(cam, ranges, vals, splats, out, n_contrib, grad_out, nullptr, splat_grads, counters, nullptr);
}

static inline const RgsSegment* find_segment(const RgsSegment* segs, int nseg, int64_t id, int64_t& local) {
    for (int s = 0; s < nseg; ++s) {
        if (id < segs[s].count) { local = id; return &segs[s]; }
        id -= segs[s].count;
    }
    local = 0;
    return nullptr;
}

int rgs_cpu_geom_bwd(const RgsCamera* cam, const RgsSegment* segs, int64_t nseg, const int32_t* counters,
                     const RgsSplat* splats, const int32_t* vis_ids, const uint32_t* aux,
                     const RgsSplatGrad* splat_grads, int64_t cap_vis, void*) {
    (void)splats; (void)cap_vis;
    int64_t n_vis = counters[RGS_CNT_VIS];
    for (int64_t slot = 0; slot < n_vis; ++slot) {
        int64_t i;
        const RgsSegment* sg = find_segment(segs, (int)nseg, vis_ids[slot], i);
        if (!sg) continue;
        float gx[3] = {0, 0, 0}, gsh[48], gs[3] = {0, 0, 0}, gq[4] = {0, 0, 0, 0}, go[1] = {0};
        for (int k = 0; k < 48; ++k) gsh[k] = 0.f;
        unsigned clamped = aux[slot] & 7u;
        float radius = (float)(aux[slot] >> 3);
        float nrm = rgs_project_bwd(*cam, sg->xyz + 3 * i, sg->scale + 3 * i, sg->rot + 4 * i, sg->opacity[i],
                                    sg->sh + 48 * i, clamped, splat_grads[slot], gx, gsh, gs, gq, go);
        if (sg->touched) sg->touched[i] = 1;
        if (sg->g_xyz) for (int k = 0; k < 3; ++k) sg->g_xyz[3 * i + k] += gx[k];
        if (sg->g_sh) for (int k = 0; k < 48; ++k) sg->g_sh[48 * i + k] += gsh[k];
        if (sg->g_scale) for (int k = 0; k < 3; ++k) sg->g_scale[3 * i + k] += gs[k];
        if (sg->g_rot) for (int k = 0; k < 4; ++k) sg->g_rot[4 * i + k] += gq[k];
        if (sg->g_opacity) sg->g_opacity[i] += go[0];
        if (sg->g_mean2d) {
            sg->g_mean2d[2 * i] = splat_grads[slot].dpx * 0.5f * cam->W;
            sg->g_mean2d[2 * i + 1] = splat_grads[slot].dpy * 0.5f * cam->H;
        }
        if (sg->stat_grad) sg->stat_grad[i] += nrm;
        if (sg->stat_denom) sg->stat_denom[i] += 1.0f;
        if (sg->stat_maxrad) sg->stat_maxrad[i] = std::max(sg->stat_maxrad[i], radius);
    }
    return 0;
}

// radii (P) of one segment, for API parity with the reference's `radii` output.
int rgs_cpu_scatter_radii(const int32_t* counters, const int32_t* vis_ids, const uint32_t* aux, int64_t id_base,
                          int64_t count, int32_t* radii, void*) {
    int64_t n_vis = counters[RGS_CNT_VIS];
    for (int64_t s = 0; s < n_vis; ++s) {
        int64_t i = (int64_t)vis_ids[s] - id_base;
        if (i >= 0 && i < count) radii[i] = (int32_t)(aux[s] >> 3);
    }
    return 0;
}

// Fused Adam over the grouped parameter block. The block holds five groups of `cap` rows each:
// xyz(3) sh(48) scale(3) rot(4) opacity(1); only the first `count` rows of each group are live.
// `skip` (optional counter block) with a non-zero overflow word drops the update and clears the step's gradients.
int rgs_cpu_adam(float* p, float* g, float* m, float* v, int64_t count, int64_t cap, const double* lrs,
                 double beta1, double beta2, double eps, int64_t step, int64_t zero_grad, const int32_t* skip,
                 const uint8_t* touched, uint8_t* active, void*) {
    const int widths[5] = {3, 48, 3, 4, 1};
    if (skip && skip[RGS_CNT_OVERFLOW]) {  // dropped step: no update, but the gradients that were written are cleared
        int64_t goff = 0;
        for (int grp = 0; grp < 5 && zero_grad; ++grp) {
            const int w = widths[grp];
            for (int64_t e = 0; e < count * w; ++e)
                if (!touched || touched[e / w]) g[goff + e] = 0.f;
            goff += cap * w;
        }
        return 0;
    }
    float bc1 = (float)(1.0 / (1.0 - std::pow(beta1, (double)step)));
    float bc2s = (float)(1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step)));
    int64_t off = 0;
    for (int grp = 0; grp < 5; ++grp) {
        int w = widths[grp];
#pragma omp parallel for
        for (int64_t e = 0; e < count * w; ++e) {
            int col = (int)(e % w);
            float lr;
            switch (grp) {
                case 0: lr = (float)lrs[RGS_LR_XYZ]; break;
                case 1: lr = (float)(col < 3 ? lrs[RGS_LR_FDC] : lrs[RGS_LR_FREST]); break;
                case 2: lr = (float)lrs[RGS_LR_SCALE]; break;
                case 3: lr = (float)lrs[RGS_LR_ROT]; break;
                default: lr = (float)lrs[RGS_LR_OPACITY]; break;
            }
            int64_t k = off + e;
            const bool t = touched ? touched[e / w] != 0 : true;
            if (!t && touched && active && !active[e / w]) continue;  // never touched since the moments were zeroed
            if (!t && m[k] == 0.f && v[k] == 0.f) continue;  // zero gradient, zero moments: the update is exactly zero
            rgs_adam_elem(p[k], t ? g[k] : 0.f, m[k], v[k], lr, (float)beta1, (float)beta2, (float)eps, bc1, bc2s);
            if (zero_grad && t) g[k] = 0.f;
        }
        off += cap * w;
    }
    if (touched && active)
        for (int64_t r = 0; r < count; ++r)
            if (touched[r]) active[r] = 1;
    return 0;
}

// the row-block variant of the CUDA library is a different work distribution of the same update
int rgs_cpu_adam_rows(float* p, float* g, float* m, float* v, int64_t count, int64_t cap, const double* lrs, double beta1,
                      double beta2, double eps, int64_t step, int64_t zero_grad, const int32_t* skip, const uint8_t* touched,
                      uint8_t* active, uint32_t*, uint32_t*, void*) {
    return rgs_cpu_adam(p, g, m, v, count, cap, lrs, beta1, beta2, eps, step, zero_grad, skip, touched, active, nullptr);
}

// ---------------------------------------------------------------------------------------------
// Compositing of K partial images (front to back) and the fused L1 + D-SSIM loss.
// ---------------------------------------------------------------------------------------------

// partials: K pointers to (H,W,4) buffers in front-to-back order. image: (3,H,W) planar,
// trans: (H,W) total transmittance. Rows [row0,row1) only.
int rgs_cpu_composite_fwd(const float* const* partials, int64_t K, const float* bg, int64_t H, int64_t W,
                          int64_t row0, int64_t row1, float* image, float* trans, void*) {
    (void)H;
#pragma omp parallel for
    for (int64_t y = row0; y < row1; ++y)
        for (int64_t x = 0; x < W; ++x) {
            int64_t pid = y * W + x;
            float C[3], T;
            rgs_composite_pixel_fwd(partials, (int)K, pid, bg, C, T);
            image[pid] = C[0]; image[H * W + pid] = C[1]; image[2 * H * W + pid] = C[2];
            trans[pid] = T;
        }
    return 0;
}

// g_image: (3,H,W) dL/dimage; grads: K pointers to (H,W,4) buffers receiving dL/dC_k, dL/dT_k.
int rgs_cpu_composite_bwd(const float* const* partials, float* const* grads, int64_t K, const float* bg,
                          int64_t H, int64_t W, int64_t row0, int64_t row1, const float* g_image, int64_t marked, void*) {
#pragma omp parallel for
    for (int64_t y = row0; y < row1; ++y)
        for (int64_t x = 0; x < W; ++x) {
            int64_t pid = y * W + x;
            float g[3] = {g_image[pid], g_image[H * W + pid], g_image[2 * H * W + pid]};
            rgs_composite_pixel_bwd(partials, grads, (int)K, pid, bg, g, marked ? 1 : 0);
        }
    return 0;
}

// SSIM statistics pass: for rows [row0,row1) computes the SSIM map sum, the L1 sum and the three
// derivative maps (dmu, dsig1, dsig12; each (3,H,W)) that the second pass convolves.
// sums[0] += sum |img-gt| ; sums[1] += sum ssim_map ; sums[2] += sum (img-gt)^2
int rgs_cpu_ssim_fwd(const float* img, const float* gt, int64_t H, int64_t W, int64_t row0, int64_t row1,
                     int64_t srow0, int64_t srow1, float* dmaps, double* sums, void*) {
    float gw[11];
    rgs_gauss_window(gw);
    double l1 = 0, ss = 0, l2 = 0;
#pragma omp parallel for reduction(+ : l1, ss, l2)
    for (int64_t y = row0; y < row1; ++y)
        for (int c = 0; c < 3; ++c)
            for (int64_t x = 0; x < W; ++x) {
                const float* a = img + c * H * W; const float* b = gt + c * H * W;
                float mu1 = 0, mu2 = 0, e11 = 0, e22 = 0, e12 = 0;
                for (int dy = -5; dy <= 5; ++dy) {
                    int64_t yy = y + dy; if (yy < 0 || yy >= H) continue;
                    for (int dx = -5; dx <= 5; ++dx) {
                        int64_t xx = x + dx; if (xx < 0 || xx >= W) continue;
                        float wgt = gw[dy + 5] * gw[dx + 5];
                        float p = a[yy * W + xx], q = b[yy * W + xx];
                        mu1 += wgt * p; mu2 += wgt * q; e11 += wgt * p * p; e22 += wgt * q * q; e12 += wgt * p * q;
                    }
                }
                float d[3];
                float s = rgs_ssim_pixel(mu1, mu2, e11, e22, e12, d);
                int64_t pid = c * H * W + y * W + x;
                if (dmaps) { dmaps[pid] = d[0]; dmaps[3 * H * W + pid] = d[1]; dmaps[6 * H * W + pid] = d[2]; }
                if (y >= srow0 && y < srow1) {
                    float diff = a[y * W + x] - b[y * W + x];
                    l1 += std::fabs(diff); ss += s; l2 += (double)diff * diff;
                }
            }
    sums[0] += l1; sums[1] += ss; sums[2] += l2;
    return 0;
}

// Second pass: g_image = w_l1 * sign(img-gt) + w_ssim * d(-SSIM mean)/dimg on rows [row0,row1);
// w_l1 = (1-lambda)/(3HW), w_ssim = lambda/(3HW) are passed pre-multiplied by the caller.
int rgs_cpu_ssim_bwd(const float* img, const float* gt, const float* dmaps, int64_t H, int64_t W, int64_t row0,
                     int64_t row1, int64_t vrow0, int64_t vrow1, double w_l1, double w_ssim, float* g_image, void*) {
    float gw[11];
    rgs_gauss_window(gw);
#pragma omp parallel for
    for (int64_t y = row0; y < row1; ++y)
        for (int c = 0; c < 3; ++c)
            for (int64_t x = 0; x < W; ++x) {
                const float* dm = dmaps + c * H * W;
                float s0 = 0, s1 = 0, s2 = 0;
                for (int dy = -5; dy <= 5; ++dy) {
                    int64_t yy = y + dy; if (yy < vrow0 || yy >= vrow1) continue;
                    for (int dx = -5; dx <= 5; ++dx) {
                        int64_t xx = x + dx; if (xx < 0 || xx >= W) continue;
                        float wgt = gw[dy + 5] * gw[dx + 5];
                        s0 += wgt * dm[yy * W + xx]; s1 += wgt * dm[3 * H * W + yy * W + xx];
                        s2 += wgt * dm[6 * H * W + yy * W + xx];
                    }
                }
                int64_t pid = c * H * W + y * W + x;
                float p = img[pid], q = gt[pid];
                float dssim = s0 + 2.0f * p * s1 + q * s2;  // d(sum ssim)/d img
                float diff = p - q;
                float sgn = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
                g_image[pid] = (float)w_l1 * sgn - (float)w_ssim * dssim;
            }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// CPU twins of the two-slab forward (rgs_cuda_bin_slab, rgs_cuda_blend_fwd_slab, rgs_cuda_blend_bwd_slab): the same
// contract (regions of the instance buffers, counter words, absolute ranges, state carried in out / depth /
// n_contrib with the finished flag in the top bit, tile_done bytes), written as plain loops. They let the host-side
// logic around the slabs (capacities, regrow, mode switching) run in tests without a GPU.
// ---------------------------------------------------------------------------------------------
int rgs_cpu_bin_slab(const RgsCamera* cam, const uint32_t* slot_depth, const uint32_t* slot_rect, uint32_t* slot_cnt,
                     int64_t cap_vis, uint32_t*, uint32_t* vis_va, uint32_t*, uint32_t*, uint32_t* inst_keys,
                     uint32_t* inst_vals, uint32_t*, uint32_t*, int64_t region_off, int64_t region_cap, int32_t* counters,
                     int64_t num_tiles, int32_t* ranges, uint32_t*, int64_t, int64_t slab, int64_t frac256,
                     const uint8_t* tile_done, uint32_t*, void*) {
    if (num_tiles > (1 << 24) || cam->tight_rect >= 2 || slab < 0 || slab > 1) return 15;
    if (slab == 1 && !tile_done) return 15;
    const int which = slab == 0 ? RGS_CNT_INST : RGS_CNT_INST2;
    std::memset(ranges, 0, num_tiles * 8);
    counters[which] = 0;
    if (counters[RGS_CNT_OVERFLOW]) return 0;
    const int64_t n = std::min<int64_t>(counters[RGS_CNT_VIS], cap_vis);
    uint32_t* order = vis_va;  // the sorted slot order lives where the CUDA sort leaves it
    if (slab == 0) {
        std::iota(order, order + n, 0u);
        std::stable_sort(order, order + n, [&](uint32_t a, uint32_t b) { return slot_depth[a] < slot_depth[b]; });
    }
    const int64_t seg = 1024, nseg = (n + seg - 1) / seg;
    int64_t split = std::min<int64_t>(nseg, ((n * frac256) >> 8) / seg);
    const int64_t i0 = (slab == 0 ? 0 : split) * seg, i1 = std::min<int64_t>(n, (slab == 0 ? split : nseg) * seg);
    const int tiles_x = cam->tiles_x;
    std::vector<std::pair<uint32_t, uint32_t>> inst;
    for (int64_t i = i0; i < i1; ++i) {
        const uint32_t s = order[i], lo = slot_rect[2 * s], hi = slot_rect[2 * s + 1];
        uint32_t c = 0;
        for (uint32_t y = lo >> 16; y < (hi >> 16); ++y)
            for (uint32_t x = lo & 0xffff; x < (hi & 0xffff); ++x) {
                const uint32_t t = y * (uint32_t)tiles_x + x;
                if (tile_done && tile_done[t]) continue;
                if (slab == 0 && slot_cnt[s] == 0) continue;
                inst.emplace_back(t, s);
                ++c;
            }
        if (tile_done) slot_cnt[s] = c;
    }
    counters[which] = (int32_t)std::min<size_t>(inst.size(), 0x7fffffff);
    if ((int64_t)inst.size() > region_cap) { counters[RGS_CNT_OVERFLOW] = 1; return 0; }
    std::stable_sort(inst.begin(), inst.end(),
                     [](const std::pair<uint32_t, uint32_t>& a, const std::pair<uint32_t, uint32_t>& b) { return a.first < b.first; });
    const int64_t m = (int64_t)inst.size();
    for (int64_t i = 0; i < m; ++i) {
        inst_keys[region_off + i] = inst[i].first; inst_vals[region_off + i] = inst[i].second;
        const uint32_t t = inst[i].first;
        if (i == 0 || inst[i - 1].first != t) ranges[2 * t] = (int32_t)(region_off + i);
        if (i == m - 1 || inst[i + 1].first != t) ranges[2 * t + 1] = (int32_t)(region_off + i + 1);
    }
    return 0;
}

int rgs_cpu_blend_fwd_slab(const RgsCamera* cam, const int32_t* ranges_a, const int32_t* ranges_b, const uint32_t* vals,
                           const RgsSplat* splats, float* out, float* depth, int32_t* n_contrib, int32_t* counters,
                           uint8_t* tile_done, int64_t, int64_t mode, int64_t n_dst, const int32_t* row0, const int32_t* row1,
                           float* const* dst, const uint8_t* occl, void*) {
    if (mode != 1 && mode != 2) return 15;
    const int W = cam->W, H = cam->H;
    const bool blank = counters[RGS_CNT_OVERFLOW] != 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int tile = 0; tile < cam->tiles_x * cam->tiles_y; ++tile) {
        const int tx = tile % cam->tiles_x, ty = tile / cam->tiles_x;
        const int len_a = blank ? 0 : ranges_a[2 * tile + 1] - ranges_a[2 * tile];
        const int r0 = blank ? 0 : (mode == 1 ? ranges_a[2 * tile] : ranges_b[2 * tile]);
        const int r1 = blank ? 0 : (mode == 1 ? ranges_a[2 * tile + 1] : ranges_b[2 * tile + 1]);
        bool all_done = true;
        for (int ly = 0; ly < RGS_TILE; ++ly)
            for (int lx = 0; lx < RGS_TILE; ++lx) {
                const int x = tx * RGS_TILE + lx, y = ty * RGS_TILE + ly;
                if (x >= W || y >= H) continue;
                const int64_t pid = (int64_t)y * W + x;
                RgsPixelRay ray; rgs_pixel_ray(*cam, (float)x, (float)y, ray);
                RgsPixelState st; rgs_pixel_init(st);
                if (mode == 2) {
                    st.C[0] = out[4 * pid]; st.C[1] = out[4 * pid + 1]; st.C[2] = out[4 * pid + 2]; st.T = out[4 * pid + 3];
                    if (depth) st.D = depth[pid];
                    const uint32_t nc = (uint32_t)n_contrib[pid];
                    st.last = (int)(nc & 0x7fffffffu); st.done = (int)(nc >> 31);
                }
                for (int i = r0; i < r1 && !st.done; ++i) {
                    st.contributor = (mode == 2 ? len_a : 0) + (i - r0);
                    rgs_blend_fwd_step(*cam, ray, (float)x, (float)y, splats[vals[i]], st);
                }
                out[4 * pid] = st.C[0]; out[4 * pid + 1] = st.C[1]; out[4 * pid + 2] = st.C[2];
                out[4 * pid + 3] = mode == 1 ? st.T : rgs_mark_finished(st.T, st.done);  // the near slab's value is resumed
                if (depth) depth[pid] = st.D;
                n_contrib[pid] = mode == 1 ? (int32_t)((uint32_t)st.last | ((uint32_t)(st.done ? 1 : 0) << 31)) : st.last;
                all_done = all_done && st.done;
            }
        if (mode == 1) tile_done[tile] = (all_done || (occl && occl[tile])) ? 1 : 0;
        else if (tile_done && all_done) tile_done[tile] = 1;
    }
    if (mode == 2)
        for (int64_t o = 0; o < n_dst; ++o)
            if (row1[o] > row0[o])
                std::memcpy(dst[o], out + (int64_t)row0[o] * W * 4, (size_t)(row1[o] - row0[o]) * W * 16);
    return 0;
}

// host twins of the tile-map helpers (rgs_p2p.cu)
int rgs_cpu_tile_maps_or(const uint8_t* const* srcs, int64_t n, uint8_t* dst, int64_t nbytes, int64_t overwrite, void*) {
    for (int64_t i = 0; i < nbytes; ++i) {
        uint8_t v = overwrite ? 0 : dst[i];
        for (int64_t k = 0; k < n; ++k) v |= srcs[k][i];
        dst[i] = v ? 1 : 0;
    }
    return 0;
}

int rgs_cpu_tile_map_push(const uint8_t* src, uint8_t* const* dsts, int64_t n_dst, int64_t nbytes, void*) {
    for (int64_t k = 0; k < n_dst; ++k) std::memcpy(dsts[k], src, (size_t)nbytes);
    return 0;
}

int rgs_cpu_blend_bwd_slab(const RgsCamera* cam, const int32_t* ranges_a, const int32_t* ranges_b, int64_t,
                           const uint32_t* vals, const RgsSplat* splats, const float* out, const int32_t* n_contrib,
                           const float* grad_out, RgsSplatGrad* splat_grads, int32_t* counters, int64_t*, int64_t,
                           const float* grad_depth, void*) {
    const int W = cam->W, H = cam->H;
    if (counters[RGS_CNT_OVERFLOW]) return 0;
    for (int tile = 0; tile < cam->tiles_x * cam->tiles_y; ++tile) {
        const int tx = tile % cam->tiles_x, ty = tile / cam->tiles_x;
        const int a0 = ranges_a[2 * tile], len_a = ranges_a[2 * tile + 1] - a0, b0 = ranges_b[2 * tile];
        for (int ly = 0; ly < RGS_TILE; ++ly)
            for (int lx = 0; lx < RGS_TILE; ++lx) {
                const int x = tx * RGS_TILE + lx, y = ty * RGS_TILE + ly;
                if (x >= W || y >= H) continue;
                const int64_t pid = (int64_t)y * W + x;
                RgsPixelRay ray; rgs_pixel_ray(*cam, (float)x, (float)y, ray);
                RgsPixelBwd st;
                rgs_pixel_bwd_init(st, out[4 * pid + 3], grad_out + 4 * pid, grad_out[4 * pid + 3]);
                RgsPixelBwdDepth dep = {0.f, 0.f, grad_depth ? grad_depth[pid] : 0.f};
                for (int v = n_contrib[pid] - 1; v >= 0; --v) {  // position in the list "near range, then far range"
                    const uint32_t slot = vals[v < len_a ? a0 + v : b0 + (v - len_a)];
                    RgsSplatGrad g;
                    if (!rgs_blend_bwd_step(*cam, ray, (float)x, (float)y, splats[slot], st, g, grad_depth ? &dep : nullptr))
                        continue;
                    float* d = reinterpret_cast<float*>(&splat_grads[slot]);
                    const float* src = reinterpret_cast<const float*>(&g);
                    for (int k = 0; k < 10; ++k) d[k] += src[k];
                }
            }
    }
    return 0;
}

// The CPU backward visits pixels in a fixed order and is deterministic as it is: the fixed-point variant is the same call.
int rgs_cpu_blend_bwd_fixed(const RgsCamera* cam, const int32_t* ranges, const uint32_t* vals, const RgsSplat* splats,
                            const float* out, const int32_t* n_contrib, const float* grad_out, RgsSplatGrad* splat_grads,
                            int32_t* counters, int64_t*, int64_t, void*) {
    return rgs_cpu_blend_bwd(cam, ranges, vals, splats, out, n_contrib, grad_out, splat_grads, counters, nullptr);
}

// CPU twins of the fused training path of rgs_loss.cu: the same four steps, run back to back.
int rgs_cpu_composite_ssim_fwd(const float* const* partials, int64_t K, const float* bg, const float* gt, int64_t H,
                               int64_t W, int64_t crow0, int64_t crow1, int64_t srow0, int64_t srow1, float* image,
                               float* trans, float* dmaps, double* sums, void*) {
    if (crow1 <= crow0) return 0;
    const int64_t e0 = std::max<int64_t>(0, crow0 - 5), e1 = std::min<int64_t>(H, crow1 + 5);
    int rc = rgs_cpu_composite_fwd(partials, K, bg, H, W, e0, e1, image, trans, nullptr);
    if (rc) return rc;
    return rgs_cpu_ssim_fwd(image, gt, H, W, crow0, crow1, srow0, srow1, dmaps, sums, nullptr);
}

int rgs_cpu_ssim_composite_bwd(const float* const* partials, float* const* grads, int64_t K, const float* bg,
                               const float* img, const float* gt, const float* dmaps, int64_t H, int64_t W, int64_t row0,
                               int64_t row1, int64_t vrow0, int64_t vrow1, double w_l1, double w_ssim, float* g_image,
                               int64_t marked, void*) {
    if (row1 <= row0) return 0;
    int rc = rgs_cpu_ssim_bwd(img, gt, dmaps, H, W, row0, row1, vrow0, vrow1, w_l1, w_ssim, g_image, nullptr);
    if (rc) return rc;
    return rgs_cpu_composite_bwd(partials, grads, K, bg, H, W, row0, row1, g_image, marked, nullptr);
}

// CPU twin of rgs_border_mask_kernel
int rgs_cpu_border_mask(const float* xyz, const float* scale, int64_t n, const float* boxes, int64_t M, int64_t self,
                        double margin, int64_t* masks, void*) {
    if (M < 1 || M > RGS_MAX_BORDER_MODELS || self < 0 || self >= M) return 17;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) masks[i] = rgs_border_mask(xyz + 3 * i, scale + 3 * i, boxes, (int)M, (int)self, (float)margin);
    return 0;
}

// CPU twins of rgs_aux.cu
int rgs_cpu_knn3(const RgsKnnGrid* g, const float* pts, const int32_t* cell_start, int64_t n, float* out, void*) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t i = 0; i < n; ++i) out[i] = rgs_knn3(*g, pts, cell_start, n, i);
    return 0;
}

int rgs_cpu_histogram(const float* xyz, const float* weight, int64_t n, const double* lo, const double* voxel,
                      const int64_t* dims, float* grid, void*) {
    for (int64_t i = 0; i < n; ++i) {
        int64_t c[3];
        for (int a = 0; a < 3; ++a) {
            int64_t v = (int64_t)std::floor((xyz[3 * i + a] - (float)lo[a]) / (float)voxel[a]);
            c[a] = std::min<int64_t>(std::max<int64_t>(v, 0), dims[a] - 1);
        }
        grid[(c[0] * dims[1] + c[1]) * dims[2] + c[2]] += weight ? weight[i] : 1.0f;
    }
    return 0;
}

int rgs_cpu_mark_visible(const float* xyz, int64_t n, const RgsCamera* cam, uint8_t* out, void*) {
    for (int64_t i = 0; i < n; ++i) {
        float t[3];
        rgs_view_point(cam->view, xyz + 3 * i, t);
        out[i] = t[2] > RGS_NEAR_Z ? 1 : 0;
    }
    return 0;
}

// CPU twins of rgs_surgery.cu (same entry points, same output order, same split samples)
int rgs_cpu_densify_classify(const float* params, int64_t cap, int64_t n, const float* accum, const float* denom,
                             const float* maxrad, const RgsDensifyCfg* cfg, uint8_t* codes, int32_t* block_counts,
                             int64_t* totals, void*) {
    for (int c = 0; c < 4; ++c) totals[c] = 0;
    if (n <= 0) return 0;
    const RgsConstBlock p = rgs_const_block_of(params, cap);
    const int64_t nblocks = (n + RGS_SURGERY_BLOCK - 1) / RGS_SURGERY_BLOCK;
    for (int64_t b = 0; b < nblocks; ++b) {
        int cnt[4] = {0, 0, 0, 0};
        const int64_t end = std::min<int64_t>(n, (b + 1) * RGS_SURGERY_BLOCK);
        for (int64_t i = b * RGS_SURGERY_BLOCK; i < end; ++i) {
            const uint32_t code = rgs_densify_code(*cfg, p.scale + 3 * i, p.opacity[i], accum[i], denom[i], maxrad[i]);
            codes[i] = (uint8_t)code;
            for (int c = 0; c < 4; ++c) cnt[c] += (code >> c) & 1u;
        }
        for (int c = 0; c < 4; ++c) {
            block_counts[c * nblocks + b] = (int32_t)totals[c];
            totals[c] += cnt[c];
        }
    }
    return 0;
}

int rgs_cpu_densify_gather(const float* params, const float* m, const float* v, int64_t cap, int64_t n,
                           const uint8_t* codes, const int32_t* block_offsets, const int64_t* totals, float* dparams,
                           float* dm, float* dv, int64_t dcap, uint64_t seed, int* status, void*) {
    if (n <= 0) return 0;
    const int64_t base_of[4] = {0, totals[0], totals[0] + totals[1], totals[0] + totals[1] + totals[2]};
    if (base_of[3] + totals[3] > dcap) { *status = 1; return 0; }
    const RgsConstBlock sp = rgs_const_block_of(params, cap), sm = rgs_const_block_of(m, cap), sv = rgs_const_block_of(v, cap);
    const RgsBlock dp = rgs_block_of(dparams, dcap), dmm = rgs_block_of(dm, dcap), dvv = rgs_block_of(dv, dcap);
    const int64_t nblocks = (n + RGS_SURGERY_BLOCK - 1) / RGS_SURGERY_BLOCK;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; ++b) {
        int64_t run[4];
        for (int c = 0; c < 4; ++c) run[c] = base_of[c] + block_offsets[c * nblocks + b];
        const int64_t end = std::min<int64_t>(n, (b + 1) * RGS_SURGERY_BLOCK);
        for (int64_t i = b * RGS_SURGERY_BLOCK; i < end; ++i)
            for (int c = 0; c < 4; ++c)
                if ((codes[i] >> c) & 1u) rgs_surgery_emit(sp, sm, sv, i, dp, dmm, dvv, run[c]++, c, seed);
    }
    return 0;
}

int rgs_cpu_records_pack(const float* params, const float* m, const float* v, int64_t cap, const int64_t* index,
                         int64_t row0, int64_t n, float* out, void*) {
    const float* src[3] = {params, m, v};
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const int64_t i = index ? index[r] : row0 + r;
        for (int c = 0; c < 177; ++c) out[r * 177 + c] = src[c / 59][rgs_record_offset(cap, i, c % 59)];
    }
    return 0;
}

int rgs_cpu_records_unpack(const float* rec, int64_t n, float* params, float* m, float* v, int64_t cap, int64_t start,
                           void*) {
    float* dst[3] = {params, m, v};
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r)
        for (int c = 0; c < 177; ++c) dst[c / 59][rgs_record_offset(cap, start + r, c % 59)] = rec[r * 177 + c];
    return 0;
}

}  // extern "C"
