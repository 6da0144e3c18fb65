// Per-pixel math of the compositing operator and of the L1 + D-SSIM loss, shared by the sm_100a
// kernels and the native CPU backend.
//
// Parity targets in the reference (MooreThreads/RetinaGS):
//   parallel_utils/basic_parallel_trainer/result_aggregator.py:244-259  (front-to-back "blender")
//   utils/loss_utils.py:17-63  (L1; SSIM with an 11x11 sigma=1.5 window, zero padding, C1=.01^2, C2=.03^2)
// The reference gets the backward of both from autograd; here it is written out.
#pragma once
#include "rgs_math.h"

#define RGS_MAX_PARTIALS 64
#define RGS_SSIM_C1 0.0001f
#define RGS_SSIM_C2 0.0009f

RGS_HD void rgs_gauss_window(float* g) {
    float s = 0.f;
    for (int i = 0; i < 11; ++i) { float d = (float)(i - 5); g[i] = expf(-(d * d) / (2.0f * 1.5f * 1.5f)); s += g[i]; }
    for (int i = 0; i < 11; ++i) g[i] /= s;
}

// SSIM of one window given the five weighted moments. d[0..2] receive the coefficients with which
// the window's weights enter d(ssim)/d(img1): d ssim / d x_p = w_p (d0 + 2 x_p d1 + y_p d2).
RGS_HD float rgs_ssim_pixel(float mu1, float mu2, float e11, float e22, float e12, float* d) {
    float mu1s = mu1 * mu1, mu2s = mu2 * mu2, mu12 = mu1 * mu2;
    float s1 = e11 - mu1s, s2 = e22 - mu2s, s12 = e12 - mu12;
    float A1 = 2.f * mu12 + RGS_SSIM_C1, A2 = 2.f * s12 + RGS_SSIM_C2;
    float B1 = mu1s + mu2s + RGS_SSIM_C1, B2 = s1 + s2 + RGS_SSIM_C2;
    float inv = 1.0f / (B1 * B2);
    float ssim = A1 * A2 * inv;
    float d_mu1 = 2.f * mu2 * A2 * inv - 2.f * mu1 * ssim / B1;
    float d_s1 = -ssim / B2;
    float d_s12 = 2.f * A1 * inv;
    d[0] = d_mu1 - 2.f * mu1 * d_s1 - mu2 * d_s12;
    d[1] = d_s1;
    d[2] = d_s12;
    return ssim;
}

// Front-to-back "over" of K partials (premultiplied RGB + transmittance) at one pixel.
RGS_HD void rgs_composite_pixel_fwd(const float* const* partials, int K, int64_t pid, const float* bg, float* C,
                                    float& T) {
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, t = 1.f;
    for (int k = 0; k < K; ++k) {
        const float* q = partials[k] + 4 * pid;
        acc0 += t * q[0]; acc1 += t * q[1]; acc2 += t * q[2];
        t *= q[3];
    }
    C[0] = acc0 + bg[0] * t; C[1] = acc1 + bg[1] * t; C[2] = acc2 + bg[2] * t;
    T = t;
}

// Backward: dL/dC_k = T_<k g ;  dL/dT_k = T_<k * (S_k . g) with S_k the colour behind partial k
// (S_{K-1} = bg, S_{k-1} = C_k + T_k S_k).
// A partial behind less than RGS_COMPOSITE_T_STOP of transmittance, or (with `marked`) behind a pixel that a nearer
// partial finished, receives exactly zero instead of a gradient scaled by that small factor: the rule by which a single
// render stops at a saturated pixel, applied across sub-models. The blend backward skips pixels (and whole tiles)
// whose gradient is zero, and their Gaussians get no Adam moments.
#define RGS_COMPOSITE_T_STOP 0.0001f
RGS_HD float rgs_composite_grad_weight(float t_before) { return t_before < RGS_COMPOSITE_T_STOP ? 0.f : t_before; }

// marked: the partials come from the blend kernels, whose transmittance carries the finished mark of
// rgs_mark_finished; partials behind a finished pixel then receive zero as well.
RGS_HD void rgs_composite_pixel_bwd(const float* const* partials, float* const* grads, int K, int64_t pid,
                                    const float* bg, const float* g, int marked = 0) {
    float tpre[RGS_MAX_PARTIALS];
    float t = 1.f;
    int blocked = 0;
    for (int k = 0; k < K; ++k) {
        const float tk = partials[k][4 * pid + 3];
        tpre[k] = blocked ? 0.f : t;
        blocked |= marked & rgs_is_finished(tk);
        t *= tk;
    }
    float s = bg[0] * g[0] + bg[1] * g[1] + bg[2] * g[2];
    for (int k = K - 1; k >= 0; --k) {
        const float* q = partials[k] + 4 * pid;
        float* o = grads[k] + 4 * pid;
        float tp = rgs_composite_grad_weight(tpre[k]);
        o[0] = tp * g[0]; o[1] = tp * g[1]; o[2] = tp * g[2];
        o[3] = tp * s;
        s = q[0] * g[0] + q[1] * g[1] + q[2] * g[2] + q[3] * s;
    }
}
