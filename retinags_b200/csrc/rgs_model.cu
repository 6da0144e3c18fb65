// sm_100a kernels over the Gaussian parameter store: fused Adam over the grouped 59-float block.
//
// Replaces the per-tensor torch.optim.Adam loops the reference runs for each sub-model and each of
// its seven parameter groups (parallel_utils/basic_parallel_trainer/trainer4tree_partition.py:663-666,
// scene/gaussian_nn_module.py:429-452): one launch updates xyz / SH / scale / rotation / opacity
// with their own learning rates, clears the gradient and honours the overflow guard.
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"

struct RgsLrTable { float lr[6]; };

__device__ __forceinline__ float adam_lr(const RgsLrTable& t, int grp, int col) {
    switch (grp) {
        case 0: return t.lr[RGS_LR_XYZ];
        case 1: return col < 3 ? t.lr[RGS_LR_FDC] : t.lr[RGS_LR_FREST];
        case 2: return t.lr[RGS_LR_SCALE];
        case 3: return t.lr[RGS_LR_ROT];
        default: return t.lr[RGS_LR_OPACITY];
    }
}

// Update of one float4 (or the ragged tail) of a column group of compile-time width W, so that the row / column
// arithmetic is multiplications by constants instead of 64-bit divisions.
template <int W, int GRP>
__device__ __forceinline__ void adam_vec(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                         float* __restrict__ v, int64_t e0, int64_t live, int64_t goff,
                                         const RgsLrTable& lrs, float beta1, float beta2, float eps, float bc1, float bc2s,
                                         int zero_grad, const uint8_t* __restrict__ touched,
                                         const uint8_t* __restrict__ active) {
    const int64_t base = goff + e0;
    if (e0 + 3 < live) {
        // rows whose `touched` byte is 0 hold zero gradients: skip the gradient read and clear, and when the
        // moments are zero as well the whole update is exactly zero and nothing is written
        bool any = true;
        if (touched) {
            const int64_t r0 = e0 / W, r3 = (e0 + 3) / W;
            any = touched[r0] != 0;
            if (W < 4) { any = any || touched[(e0 + 1) / W] || touched[(e0 + 2) / W]; }
            if (r3 != r0) any = any || touched[r3];
            // rows without the `active` mark have never received a gradient since their moments were zeroed: the
            // moments are zero, the update is exactly zero, and not even the moments need to be read
            if (!any && active) {
                bool live_m = active[r0] != 0;
                if (W < 4) { live_m = live_m || active[(e0 + 1) / W] || active[(e0 + 2) / W]; }
                if (r3 != r0) live_m = live_m || active[r3];
                if (!live_m) return;
            }
        }
        float4 M = *reinterpret_cast<float4*>(m + base), V = *reinterpret_cast<float4*>(v + base);
        float4 G = make_float4(0.f, 0.f, 0.f, 0.f);
        if (any) G = *reinterpret_cast<float4*>(g + base);
        else if (M.x == 0.f && M.y == 0.f && M.z == 0.f && M.w == 0.f && V.x == 0.f && V.y == 0.f && V.z == 0.f && V.w == 0.f)
            return;
        float4 P = *reinterpret_cast<float4*>(p + base);
        const int c0 = (int)(e0 % W);
        rgs_adam_elem(P.x, G.x, M.x, V.x, adam_lr(lrs, GRP, c0 % W), beta1, beta2, eps, bc1, bc2s);
        rgs_adam_elem(P.y, G.y, M.y, V.y, adam_lr(lrs, GRP, (c0 + 1) % W), beta1, beta2, eps, bc1, bc2s);
        rgs_adam_elem(P.z, G.z, M.z, V.z, adam_lr(lrs, GRP, (c0 + 2) % W), beta1, beta2, eps, bc1, bc2s);
        rgs_adam_elem(P.w, G.w, M.w, V.w, adam_lr(lrs, GRP, (c0 + 3) % W), beta1, beta2, eps, bc1, bc2s);
        *reinterpret_cast<float4*>(p + base) = P;
        *reinterpret_cast<float4*>(m + base) = M;
        *reinterpret_cast<float4*>(v + base) = V;
        if (zero_grad && any) *reinterpret_cast<float4*>(g + base) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        for (int k = 0; k < 4 && e0 + k < live; ++k) {
            const int col = (int)((e0 + k) % W);
            const bool t = touched ? touched[(e0 + k) / W] != 0 : true;
            if (!t && touched && active && !active[(e0 + k) / W]) continue;
            if (!t && m[base + k] == 0.f && v[base + k] == 0.f) continue;
            rgs_adam_elem(p[base + k], t ? g[base + k] : 0.f, m[base + k], v[base + k], adam_lr(lrs, GRP, col), beta1, beta2,
                          eps, bc1, bc2s);
            if (zero_grad && t) g[base + k] = 0.f;
        }
    }
}

// One 128-bit unit that lies inside a single row (SH and rotation groups, 13 of the 15 units of a row): the row and the
// column are known to the caller, so that the flag test of a dead row costs two byte loads and no index arithmetic.
template <int GRP>
__device__ __forceinline__ void adam_row_vec(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                             float* __restrict__ v, int64_t base, int64_t row, int col0,
                                             const RgsLrTable& lrs, float beta1, float beta2, float eps, float bc1, float bc2s,
                                             int zero_grad, const uint8_t* __restrict__ touched,
                                             const uint8_t* __restrict__ active) {
    bool any = true;
    if (touched) {
        any = touched[row] != 0;
        if (!any && active && !active[row]) return;
    }
    float4 M = *reinterpret_cast<float4*>(m + base), V = *reinterpret_cast<float4*>(v + base);
    float4 G = make_float4(0.f, 0.f, 0.f, 0.f);
    if (any) G = *reinterpret_cast<float4*>(g + base);
    else if (M.x == 0.f && M.y == 0.f && M.z == 0.f && M.w == 0.f && V.x == 0.f && V.y == 0.f && V.z == 0.f && V.w == 0.f)
        return;
    float4 P = *reinterpret_cast<float4*>(p + base);
    rgs_adam_elem(P.x, G.x, M.x, V.x, adam_lr(lrs, GRP, col0), beta1, beta2, eps, bc1, bc2s);
    rgs_adam_elem(P.y, G.y, M.y, V.y, adam_lr(lrs, GRP, col0 + 1), beta1, beta2, eps, bc1, bc2s);
    rgs_adam_elem(P.z, G.z, M.z, V.z, adam_lr(lrs, GRP, col0 + 2), beta1, beta2, eps, bc1, bc2s);
    rgs_adam_elem(P.w, G.w, M.w, V.w, adam_lr(lrs, GRP, col0 + 3), beta1, beta2, eps, bc1, bc2s);
    *reinterpret_cast<float4*>(p + base) = P;
    *reinterpret_cast<float4*>(m + base) = M;
    *reinterpret_cast<float4*>(v + base) = V;
    if (zero_grad && any) *reinterpret_cast<float4*>(g + base) = make_float4(0.f, 0.f, 0.f, 0.f);
}

// A step whose forward overflowed its instance buffers rendered garbage: its update is dropped on every rank. The
// gradients that were written must still be cleared, or the invariant "rows without the touched mark hold zero
// gradients" would break when the host clears the marks.
__device__ __forceinline__ void adam_drop_gradients(float* __restrict__ g, int64_t count, int64_t cap,
                                                    const uint8_t* __restrict__ touched) {
    const int64_t off[5] = {0, cap * 3, cap * 51, cap * 54, cap * 58};
    const int wid[5] = {3, 48, 3, 4, 1};
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < count; r += (int64_t)gridDim.x * blockDim.x) {
        if (touched && !touched[r]) continue;
        for (int grp = 0; grp < 5; ++grp)
            for (int c = 0; c < wid[grp]; ++c) g[off[grp] + r * wid[grp] + c] = 0.f;
    }
}

__global__ void __launch_bounds__(256) rgs_adam_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                                       float* __restrict__ v, int64_t count, int64_t cap,
                                                       const __grid_constant__ RgsLrTable lrs, float beta1, float beta2,
                                                       float eps, float bc1, float bc2s, int zero_grad,
                                                       const uint32_t* __restrict__ skip,
                                                       const uint8_t* __restrict__ touched,
                                                       uint8_t* __restrict__ active) {
    if (skip && skip[RGS_CNT_OVERFLOW]) {
        if (zero_grad) adam_drop_gradients(g, count, cap, touched);
        return;
    }
    // vector ranges of the five groups: xyz(3) sh(48) scale(3) rot(4) opacity(1)
    const int64_t n0 = (count * 3 + 3) / 4, n1 = count * 12, n2 = n0, n3 = count, n4 = (count + 3) / 4;
    const int64_t v1 = n0, v2 = v1 + n1, v3 = v2 + n2, v4 = v3 + n3, tv = v4 + n4;
    const int64_t o1 = cap * 3, o2 = o1 + cap * 48, o3 = o2 + cap * 3, o4 = o3 + cap * 4;
    const bool small = count < 300000000ll;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < tv; t += (int64_t)gridDim.x * blockDim.x) {
        if (t < v1) adam_vec<3, 0>(p, g, m, v, t * 4, count * 3, 0, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad, touched, active);
        else if (t < v2) {
            if (small) {  // 32-bit unit index: row = u / 12 is one multiply
                const uint32_t u = (uint32_t)(t - v1), row = u / 12u, j = u - row * 12u;
                adam_row_vec<1>(p, g, m, v, o1 + (int64_t)row * 48 + j * 4, row, (int)(j * 4), lrs, beta1, beta2, eps, bc1, bc2s,
                                zero_grad, touched, active);
            } else {
                adam_vec<48, 1>(p, g, m, v, (t - v1) * 4, count * 48, o1, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad, touched, active);
            }
        }
        else if (t < v3) adam_vec<3, 2>(p, g, m, v, (t - v2) * 4, count * 3, o2, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad, touched, active);
        else if (t < v4) adam_row_vec<3>(p, g, m, v, o3 + (t - v3) * 4, t - v3, 0, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad, touched, active);
        else {
            adam_vec<1, 4>(p, g, m, v, (t - v4) * 4, count, o4, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad, touched, active);
            // the opacity group visits every row exactly once: it carries the marks forward. No thread of this launch
            // depends on a mark set here, because a touched row is processed whatever its mark says.
            if (touched && active)
                for (int64_t r = (t - v4) * 4; r < (t - v4) * 4 + 4 && r < count; ++r)
                    if (touched[r]) active[r] = 1;
        }
    }
}

// Row-block variant: a warp looks at the marks of a stretch of consecutive rows first (see the kernel) and
// then works only on the rows that are live, two rows per pass (15 units of a row on 15 lanes of a half-warp:
// 12 float4 of SH, the rotation, position, scale + opacity). A block of rows without a live row costs a few
// instructions instead of fifteen unit tests per row, which is what bounds rgs_adam_kernel when few rows are live
// (62.9 M rows, 0.2 % live: 3.9 ms of flag tests). Same arithmetic per element, same results.
__device__ __forceinline__ void adam_scalar(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                            float* __restrict__ v, int64_t idx, bool touched_row, float lr, float beta1,
                                            float beta2, float eps, float bc1, float bc2s, int zero_grad) {
    float M = m[idx], V = v[idx];
    if (!touched_row && M == 0.f && V == 0.f) return;
    float P = p[idx];
    rgs_adam_elem(P, touched_row ? g[idx] : 0.f, M, V, lr, beta1, beta2, eps, bc1, bc2s);
    p[idx] = P; m[idx] = M; v[idx] = V;
    if (zero_grad && touched_row) g[idx] = 0.f;
}

template <int GRP>
__device__ __forceinline__ void adam_quad(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                          float* __restrict__ v, int64_t base, int col0, bool touched_row,
                                          const RgsLrTable& lrs, float beta1, float beta2, float eps, float bc1, float bc2s,
                                          int zero_grad) {
    float4 M = *reinterpret_cast<float4*>(m + base), V = *reinterpret_cast<float4*>(v + base);
    float4 G = make_float4(0.f, 0.f, 0.f, 0.f);
    if (touched_row) G = *reinterpret_cast<float4*>(g + base);
    else if (M.x == 0.f && M.y == 0.f && M.z == 0.f && M.w == 0.f && V.x == 0.f && V.y == 0.f && V.z == 0.f && V.w == 0.f)
        return;
    float4 P = *reinterpret_cast<float4*>(p + base);
    rgs_adam_elem(P.x, G.x, M.x, V.x, adam_lr(lrs, GRP, col0), beta1, beta2, eps, bc1, bc2s);
    rgs_adam_elem(P.y, G.y, M.y, V.y, adam_lr(lrs, GRP, col0 + 1), beta1, beta2, eps, bc1, bc2s);
    rgs_adam_elem(P.z, G.z, M.z, V.z, adam_lr(lrs, GRP, col0 + 2), beta1, beta2, eps, bc1, bc2s);
    rgs_adam_elem(P.w, G.w, M.w, V.w, adam_lr(lrs, GRP, col0 + 3), beta1, beta2, eps, bc1, bc2s);
    *reinterpret_cast<float4*>(p + base) = P;
    *reinterpret_cast<float4*>(m + base) = M;
    *reinterpret_cast<float4*>(v + base) = V;
    if (zero_grad && touched_row) *reinterpret_cast<float4*>(g + base) = make_float4(0.f, 0.f, 0.f, 0.f);
}

// Row-block Adam in two launches. (1) rgs_adam_live_kernel scans the marks -- a warp looks at 512 consecutive rows per
// iteration, every lane fetching the 16 mark bytes of its rows with one 128-bit load per array -- carries the `active`
// marks forward and appends the live rows (touched this step, or holding moments) to a list, one atomic per warp.
// (2) rgs_adam_rows_kernel updates the listed rows, one half-warp per row (the 15 units of a row on 15 lanes: 12 float4
// of SH, the rotation, position, scale + opacity). Dead rows cost two wide loads per 16 rows, and the live rows are
// spread evenly over the machine wherever they lie: after the rows were sorted along a space-filling curve the live
// ones (the visible, blended Gaussians) sit in dense runs, which a kernel that walked fixed row blocks serialised.
__global__ void __launch_bounds__(256) rgs_adam_live_kernel(int64_t count, int64_t cap, const uint8_t* __restrict__ touched,
                                                            uint8_t* __restrict__ active, uint32_t* __restrict__ live_list,
                                                            uint32_t* __restrict__ live_count,
                                                            const uint32_t* __restrict__ skip) {
    if (skip && skip[RGS_CNT_OVERFLOW]) return;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t nsuper = (count + 511) / 512;
    for (int64_t sb = warp; sb < nsuper; sb += nwarps) {
        const int64_t r0 = sb * 512 + (int64_t)lane * 16;
        uint32_t tbits = 0, lbits = 0;  // bit k: row r0 + k was touched this step / has to be updated
        if (r0 < count) {
            uint32_t tw[4] = {0, 0, 0, 0}, aw[4] = {0, 0, 0, 0};
            const bool wide = r0 + 16 <= cap;
            if (wide) {
                if (touched) { const uint4 q = *reinterpret_cast<const uint4*>(touched + r0); tw[0] = q.x; tw[1] = q.y; tw[2] = q.z; tw[3] = q.w; }
                if (active) { const uint4 q = *reinterpret_cast<const uint4*>(active + r0); aw[0] = q.x; aw[1] = q.y; aw[2] = q.z; aw[3] = q.w; }
            } else {
                for (int k = 0; k < 16 && r0 + k < cap; ++k) {
                    if (touched) tw[k >> 2] |= (uint32_t)touched[r0 + k] << (8 * (k & 3));
                    if (active) aw[k >> 2] |= (uint32_t)active[r0 + k] << (8 * (k & 3));
                }
            }
            bool mark = false;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                if (r0 + k >= count) break;
                const bool t = touched ? ((tw[k >> 2] >> (8 * (k & 3))) & 0xffu) != 0 : true;
                const bool a = ((aw[k >> 2] >> (8 * (k & 3))) & 0xffu) != 0;
                if (t) tbits |= 1u << k;
                if (t || !touched || !active || a) lbits |= 1u << k;   // without marks every row counts as live
                if (t && touched && active && !a) { aw[k >> 2] |= 1u << (8 * (k & 3)); mark = true; }
            }
            if (mark) {  // rows that received their first gradient carry moments from now on
                if (wide) *reinterpret_cast<uint4*>(active + r0) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
                else for (int k = 0; k < 16 && r0 + k < cap; ++k) active[r0 + k] = (uint8_t)((aw[k >> 2] >> (8 * (k & 3))) & 0xffu);
            }
        }
        // warp-wide exclusive scan of the live counts, one reservation per warp
        const uint32_t mine = __popc(lbits);
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += y;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (total == 0) continue;
        uint32_t base = 0;
        if (lane == 31) base = atomicAdd(live_count, total);
        base = __shfl_sync(0xffffffffu, base, 31);
        uint32_t pos = base + incl - mine;
        uint32_t lb = lbits;
        while (lb) {
            const int k = __ffs(lb) - 1;
            lb &= lb - 1;
            live_list[pos++] = (uint32_t)(r0 + k) | (((tbits >> k) & 1u) << 31);
        }
    }
}

__global__ void __launch_bounds__(256) rgs_adam_rows_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                                            float* __restrict__ v, int64_t count, int64_t cap,
                                                            const __grid_constant__ RgsLrTable lrs, float beta1, float beta2,
                                                            float eps, float bc1, float bc2s, int zero_grad,
                                                            const uint32_t* __restrict__ skip,
                                                            const uint8_t* __restrict__ touched,
                                                            const uint32_t* __restrict__ live_list,
                                                            const uint32_t* __restrict__ live_count) {
    if (skip && skip[RGS_CNT_OVERFLOW]) {
        if (zero_grad) adam_drop_gradients(g, count, cap, touched);
        return;
    }
    const int64_t o1 = cap * 3, o2 = o1 + cap * 48, o3 = o2 + cap * 3, o4 = o3 + cap * 4;
    const uint32_t n = *live_count;
    const int u = threadIdx.x & 15;
    const uint32_t hw = (uint32_t)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4);
    const uint32_t nhw = (uint32_t)(((int64_t)gridDim.x * blockDim.x) >> 4);
    if (u >= 15) return;
    for (uint32_t i = hw; i < n; i += nhw) {
        const uint32_t e = live_list[i];
        const int64_t row = (int64_t)(e & 0x7fffffffu);
        const bool tr = (e >> 31) != 0;
        if (u < 12) {
            adam_quad<1>(p, g, m, v, o1 + row * 48 + u * 4, u * 4, tr, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad);
        } else if (u == 12) {
            adam_quad<3>(p, g, m, v, o3 + row * 4, 0, tr, lrs, beta1, beta2, eps, bc1, bc2s, zero_grad);
        } else if (u == 13) {
            for (int c = 0; c < 3; ++c)
                adam_scalar(p, g, m, v, row * 3 + c, tr, lrs.lr[RGS_LR_XYZ], beta1, beta2, eps, bc1, bc2s, zero_grad);
        } else {
            for (int c = 0; c < 3; ++c)
                adam_scalar(p, g, m, v, o2 + row * 3 + c, tr, lrs.lr[RGS_LR_SCALE], beta1, beta2, eps, bc1, bc2s, zero_grad);
            adam_scalar(p, g, m, v, o4 + row, tr, lrs.lr[RGS_LR_OPACITY], beta1, beta2, eps, bc1, bc2s, zero_grad);
        }
    }
}

extern "C" {

int rgs_cuda_adam(float* p, float* g, float* m, float* v, int64_t count, int64_t cap, const double* lrs, double beta1,
                  double beta2, double eps, int64_t step, int64_t zero_grad, const int32_t* skip, const uint8_t* touched,
                  uint8_t* active, void* stream) {
    if (count <= 0) return 0;
    if (cap % 4 != 0) return 13;
    RgsLrTable t;
    for (int k = 0; k < 6; ++k) t.lr[k] = (float)lrs[k];
    const float bc1 = (float)(1.0 / (1.0 - pow(beta1, (double)step)));       // reciprocal bias corrections
    const float bc2s = (float)(1.0 / sqrt(1.0 - pow(beta2, (double)step)));
    const int64_t tv = (count * 59 + 3) / 4 + 5;
    const int64_t want = (tv + 255) / 256;
    const unsigned blocks = (unsigned)(want > RGS_SMS * 64 ? RGS_SMS * 64 : want);
    rgs_adam_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, count, cap, t, (float)beta1, (float)beta2,
                                                             (float)eps, bc1, bc2s, (int)zero_grad,
                                                             reinterpret_cast<const uint32_t*>(skip), touched, active);
    return (int)cudaGetLastError();
}

// Same contract as rgs_cuda_adam, row-block kernels (see above). live_list: `cap` words of scratch, live_count: one word;
// both owned by the caller, contents irrelevant on entry. Rows are limited to 2^31 per store.
int rgs_cuda_adam_rows(float* p, float* g, float* m, float* v, int64_t count, int64_t cap, const double* lrs, double beta1,
                       double beta2, double eps, int64_t step, int64_t zero_grad, const int32_t* skip, const uint8_t* touched,
                       uint8_t* active, uint32_t* live_list, uint32_t* live_count, void* stream) {
    if (count <= 0) return 0;
    if (cap % 4 != 0 || cap > 0x7fffffffll || !live_list || !live_count) return 13;
    cudaStream_t st = (cudaStream_t)stream;
    RgsLrTable t;
    for (int k = 0; k < 6; ++k) t.lr[k] = (float)lrs[k];
    const float bc1 = (float)(1.0 / (1.0 - pow(beta1, (double)step)));
    const float bc2s = (float)(1.0 / sqrt(1.0 - pow(beta2, (double)step)));
    RGS_CUDA_CHECK(cudaMemsetAsync(live_count, 0, 4, st));
    int64_t want = ((count + 511) / 512 + 7) / 8;  // 8 warps per block, 512 rows per warp and iteration
    unsigned blocks = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 64 ? RGS_SMS * 64 : want));
    rgs_adam_live_kernel<<<blocks, 256, 0, st>>>(count, cap, touched, active, live_list, live_count,
                                                 reinterpret_cast<const uint32_t*>(skip));
    want = (count + 15) / 16;  // 16 rows per block and pass; the kernel strides over the list
    blocks = (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 32 ? RGS_SMS * 32 : want));
    rgs_adam_rows_kernel<<<blocks, 256, 0, st>>>(p, g, m, v, count, cap, t, (float)beta1, (float)beta2, (float)eps, bc1, bc2s,
                                                 (int)zero_grad, reinterpret_cast<const uint32_t*>(skip), touched, live_list,
                                                 live_count);
    return (int)cudaGetLastError();
}

}  // extern "C"
