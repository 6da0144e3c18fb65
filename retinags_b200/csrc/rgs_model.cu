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

__global__ void __launch_bounds__(256) rgs_adam_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                                       float* __restrict__ v, int64_t count, int64_t cap,
                                                       const __grid_constant__ RgsLrTable lrs, float beta1, float beta2,
                                                       float eps, float bc1, float bc2s, int zero_grad,
                                                       const uint32_t* __restrict__ skip,
                                                       const uint8_t* __restrict__ touched) {
    if (skip && skip[RGS_CNT_OVERFLOW]) return;
    const int widths[5] = {3, 48, 3, 4, 1};
    int64_t nvec[5], voff[5], goff[5];
    int64_t tv = 0, to = 0;
#pragma unroll
    for (int k = 0; k < 5; ++k) {
        nvec[k] = (count * widths[k] + 3) / 4;
        voff[k] = tv; goff[k] = to;
        tv += nvec[k]; to += cap * widths[k];
    }
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < tv; t += (int64_t)gridDim.x * blockDim.x) {
        int grp = 0;
#pragma unroll
        for (int k = 1; k < 5; ++k) if (t >= voff[k]) grp = k;
        const int w = widths[grp];
        const int64_t e0 = (t - voff[grp]) * 4, live = count * w;
        const int64_t base = goff[grp] + e0;
        if (e0 + 3 < live) {
            // rows whose `touched` byte is 0 hold zero gradients: skip the gradient read and clear, and when the
            // moments are zero as well the whole update is exactly zero and nothing is written
            bool any = true;
            if (touched) {
                any = touched[e0 / w] | touched[(e0 + 1) / w] | touched[(e0 + 2) / w] | touched[(e0 + 3) / w];
            }
            float4 M = *reinterpret_cast<float4*>(m + base), V = *reinterpret_cast<float4*>(v + base);
            float4 G = make_float4(0.f, 0.f, 0.f, 0.f);
            if (any) G = *reinterpret_cast<float4*>(g + base);
            else if (M.x == 0.f && M.y == 0.f && M.z == 0.f && M.w == 0.f && V.x == 0.f && V.y == 0.f && V.z == 0.f && V.w == 0.f)
                continue;
            float4 P = *reinterpret_cast<float4*>(p + base);
            const int c0 = (int)(e0 % w);
            rgs_adam_elem(P.x, G.x, M.x, V.x, adam_lr(lrs, grp, c0 % w), beta1, beta2, eps, bc1, bc2s);
            rgs_adam_elem(P.y, G.y, M.y, V.y, adam_lr(lrs, grp, (c0 + 1) % w), beta1, beta2, eps, bc1, bc2s);
            rgs_adam_elem(P.z, G.z, M.z, V.z, adam_lr(lrs, grp, (c0 + 2) % w), beta1, beta2, eps, bc1, bc2s);
            rgs_adam_elem(P.w, G.w, M.w, V.w, adam_lr(lrs, grp, (c0 + 3) % w), beta1, beta2, eps, bc1, bc2s);
            *reinterpret_cast<float4*>(p + base) = P;
            *reinterpret_cast<float4*>(m + base) = M;
            *reinterpret_cast<float4*>(v + base) = V;
            if (zero_grad && any) *reinterpret_cast<float4*>(g + base) = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int k = 0; k < 4 && e0 + k < live; ++k) {
                const int col = (int)((e0 + k) % w);
                const bool t = touched ? touched[(e0 + k) / w] != 0 : true;
                if (!t && m[base + k] == 0.f && v[base + k] == 0.f) continue;
                rgs_adam_elem(p[base + k], t ? g[base + k] : 0.f, m[base + k], v[base + k], adam_lr(lrs, grp, col), beta1,
                              beta2, eps, bc1, bc2s);
                if (zero_grad && t) g[base + k] = 0.f;
            }
        }
    }
}

extern "C" {

int rgs_cuda_adam(float* p, float* g, float* m, float* v, int64_t count, int64_t cap, const double* lrs, double beta1,
                  double beta2, double eps, int64_t step, int64_t zero_grad, const int32_t* skip, const uint8_t* touched,
                  void* stream) {
    if (count <= 0) return 0;
    if (cap % 4 != 0) return 13;
    RgsLrTable t;
    for (int k = 0; k < 6; ++k) t.lr[k] = (float)lrs[k];
    const float bc1 = (float)(1.0 - pow(beta1, (double)step));
    const float bc2s = (float)sqrt(1.0 - pow(beta2, (double)step));
    const int64_t tv = (count * 59 + 3) / 4 + 5;
    const int64_t want = (tv + 255) / 256;
    const unsigned blocks = (unsigned)(want > 148 * 64 ? 148 * 64 : want);
    rgs_adam_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, count, cap, t, (float)beta1, (float)beta2,
                                                             (float)eps, bc1, bc2s, (int)zero_grad,
                                                             reinterpret_cast<const uint32_t*>(skip), touched);
    return (int)cudaGetLastError();
}

}  // extern "C"
