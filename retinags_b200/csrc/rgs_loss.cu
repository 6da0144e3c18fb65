// sm_100a kernels for ordered compositing of partial images and the fused L1 + D-SSIM loss with
// its hand-written backward (fp32 SIMT path; the tensor-core SSIM filter lives in rgs_ssim_tc.cu).
//
// Replaces, in the reference: the ATen chain of parallel_utils/basic_parallel_trainer/
// result_aggregator.py:244-259 (cat / cumprod / weighted sums + autograd) and the five depthwise
// cuDNN convolutions of utils/loss_utils.py:43-63 (+ five more in autograd's backward).
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"
#include "rgs_loss_math.h"

struct RgsPartialPtrs { const float* p[RGS_MAX_PARTIALS]; };
struct RgsGradPtrs { float* p[RGS_MAX_PARTIALS]; };

__global__ void __launch_bounds__(256) rgs_composite_fwd_kernel(const __grid_constant__ RgsPartialPtrs parts, int K,
                                                                float bg0, float bg1, float bg2, int64_t H, int64_t W,
                                                                int64_t row0, int64_t row1, float* __restrict__ image,
                                                                float* __restrict__ trans) {
    const int64_t n = (row1 - row0) * W;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pid = row0 * W + i;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, t = 1.f;
        for (int k = 0; k < K; ++k) {
            const float4 q = reinterpret_cast<const float4*>(parts.p[k])[pid];
            a0 += t * q.x; a1 += t * q.y; a2 += t * q.z;
            t *= q.w;
        }
        image[pid] = a0 + bg0 * t;
        image[H * W + pid] = a1 + bg1 * t;
        image[2 * H * W + pid] = a2 + bg2 * t;
        trans[pid] = t;
    }
}

// d(loss)/d(partial_k) of one pixel for all K partials. KMAX = 8: fully unrolled, the prefix transmittances and the
// partials stay in registers (the usual case: at most 8 sub-models overlap a pixel's row band); KMAX = RGS_MAX_PARTIALS:
// plain loops over a local array for anything larger.
template <int KMAX>
__device__ __forceinline__ void composite_pixel_grads(const RgsPartialPtrs& parts, const RgsGradPtrs& grads, int K, size_t pid,
                                                      float g0, float g1, float g2, float bg0, float bg1, float bg2,
                                                      int marked) {
    float tpre[KMAX];
    float t = 1.f;
    int blocked = 0;
    if (KMAX <= 8) {
        float4 q[KMAX];
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            if (k < K) {
                q[k] = reinterpret_cast<const float4*>(parts.p[k])[pid];
                tpre[k] = blocked ? 0.f : t;
                blocked |= marked & rgs_is_finished(q[k].w);
                t *= q[k].w;
            }
        }
        float s = bg0 * g0 + bg1 * g1 + bg2 * g2;
#pragma unroll
        for (int k = KMAX - 1; k >= 0; --k) {
            if (k < K) {
                const float tp = rgs_composite_grad_weight(tpre[k]);
                reinterpret_cast<float4*>(grads.p[k])[pid] = make_float4(tp * g0, tp * g1, tp * g2, tp * s);
                s = q[k].x * g0 + q[k].y * g1 + q[k].z * g2 + q[k].w * s;
            }
        }
    } else {
        for (int k = 0; k < K; ++k) {
            const float tk = parts.p[k][4 * pid + 3];
            tpre[k] = blocked ? 0.f : t;
            blocked |= marked & rgs_is_finished(tk);
            t *= tk;
        }
        float s = bg0 * g0 + bg1 * g1 + bg2 * g2;
        for (int k = K - 1; k >= 0; --k) {
            const float4 q = reinterpret_cast<const float4*>(parts.p[k])[pid];
            const float tp = rgs_composite_grad_weight(tpre[k]);
            reinterpret_cast<float4*>(grads.p[k])[pid] = make_float4(tp * g0, tp * g1, tp * g2, tp * s);
            s = q.x * g0 + q.y * g1 + q.z * g2 + q.w * s;
        }
    }
}

template <int KMAX>
__global__ void __launch_bounds__(256) rgs_composite_bwd_kernel(const __grid_constant__ RgsPartialPtrs parts,
                                                                const __grid_constant__ RgsGradPtrs grads, int K,
                                                                float bg0, float bg1, float bg2, int64_t H, int64_t W,
                                                                int64_t row0, int64_t row1,
                                                                const float* __restrict__ g_image, int marked) {
    const int64_t n = (row1 - row0) * W;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pid = row0 * W + i;
        const float g0 = g_image[pid], g1 = g_image[H * W + pid], g2 = g_image[2 * H * W + pid];
        composite_pixel_grads<KMAX>(parts, grads, K, (size_t)pid, g0, g1, g2, bg0, bg1, bg2, marked);
    }
}

// ---------------------------------------------------------------------------------------------
// SSIM: 32x32 output tile per block and channel, separable 11-tap filter through shared memory
// ---------------------------------------------------------------------------------------------
#define ST 32
#define SH_ 42  // ST + 10

__device__ __forceinline__ void ssim_window(float* g) { rgs_gauss_window(g); }

__global__ void __launch_bounds__(256) rgs_ssim_fwd_kernel(const float* __restrict__ img, const float* __restrict__ gt,
                                                           int H, int W, int crow0, int crow1, int srow0, int srow1,
                                                           float* __restrict__ dmaps, double* __restrict__ sums) {
    __shared__ float in1[SH_][SH_ + 1], in2[SH_][SH_ + 1];
    __shared__ float hb[5][SH_][ST];
    __shared__ float red[3][8];
    float gw[11];
    ssim_window(gw);
    const int c = blockIdx.z;
    const int x0 = blockIdx.x * ST, y0 = crow0 + blockIdx.y * ST;
    const float* a = img + (size_t)c * H * W;
    const float* b = gt + (size_t)c * H * W;
    for (int idx = threadIdx.x; idx < SH_ * SH_; idx += 256) {
        const int r = idx / SH_, q = idx % SH_;
        const int y = y0 + r - 5, x = x0 + q - 5;
        const bool in = y >= 0 && y < H && x >= 0 && x < W;
        in1[r][q] = in ? a[(size_t)y * W + x] : 0.f;
        in2[r][q] = in ? b[(size_t)y * W + x] : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < SH_ * ST; idx += 256) {
        const int r = idx / ST, q = idx % ST;
        float m1 = 0, m2 = 0, e11 = 0, e22 = 0, e12 = 0;
#pragma unroll
        for (int k = 0; k < 11; ++k) {
            const float p = in1[r][q + k], v = in2[r][q + k], w = gw[k];
            m1 += w * p; m2 += w * v; e11 += w * p * p; e22 += w * v * v; e12 += w * p * v;
        }
        hb[0][r][q] = m1; hb[1][r][q] = m2; hb[2][r][q] = e11; hb[3][r][q] = e22; hb[4][r][q] = e12;
    }
    __syncthreads();
    float l1 = 0.f, ss = 0.f, l2 = 0.f;
    const int q = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = (threadIdx.x >> 5) + 8 * i;
        const int y = y0 + r, x = x0 + q;
        if (y < crow1 && y < H && x < W) {
            float m[5] = {0, 0, 0, 0, 0};
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const float w = gw[k];
#pragma unroll
                for (int j = 0; j < 5; ++j) m[j] += w * hb[j][r + k][q];
            }
            float d[3];
            const float s = rgs_ssim_pixel(m[0], m[1], m[2], m[3], m[4], d);
            const size_t pid = (size_t)c * H * W + (size_t)y * W + x;
            const size_t plane = (size_t)3 * H * W;
            dmaps[pid] = d[0]; dmaps[plane + pid] = d[1]; dmaps[2 * plane + pid] = d[2];
            if (y >= srow0 && y < srow1) {
                const float diff = in1[r + 5][q + 5] - in2[r + 5][q + 5];
                l1 += fabsf(diff); ss += s; l2 += diff * diff;
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        l1 += __shfl_xor_sync(0xffffffffu, l1, d);
        ss += __shfl_xor_sync(0xffffffffu, ss, d);
        l2 += __shfl_xor_sync(0xffffffffu, l2, d);
    }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = l1; red[1][threadIdx.x >> 5] = ss; red[2][threadIdx.x >> 5] = l2; }
    __syncthreads();
    if (threadIdx.x < 3) {
        double t = 0;
        for (int w = 0; w < 8; ++w) t += (double)red[threadIdx.x][w];
        atomicAdd(&sums[threadIdx.x], t);
    }
}

__global__ void __launch_bounds__(256) rgs_ssim_bwd_kernel(const float* __restrict__ img, const float* __restrict__ gt,
                                                           const float* __restrict__ dmaps, int H, int W, int row0,
                                                           int row1, int vrow0, int vrow1, float w_l1, float w_ssim,
                                                           float* __restrict__ g_image) {
    __shared__ float in[3][SH_][SH_ + 1];
    __shared__ float hb[3][SH_][ST];
    float gw[11];
    ssim_window(gw);
    const int c = blockIdx.z;
    const int x0 = blockIdx.x * ST, y0 = row0 + blockIdx.y * ST;
    const size_t plane = (size_t)3 * H * W;
    const float* dm = dmaps + (size_t)c * H * W;
    for (int idx = threadIdx.x; idx < SH_ * SH_; idx += 256) {
        const int r = idx / SH_, q = idx % SH_;
        const int y = y0 + r - 5, x = x0 + q - 5;
        // derivative maps exist only on rows [vrow0, vrow1); outside the image they are zero padding
        const bool ok = y >= vrow0 && y < vrow1 && x >= 0 && x < W;
        const size_t o = (size_t)y * W + x;
        in[0][r][q] = ok ? dm[o] : 0.f;
        in[1][r][q] = ok ? dm[plane + o] : 0.f;
        in[2][r][q] = ok ? dm[2 * plane + o] : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < SH_ * ST; idx += 256) {
        const int r = idx / ST, q = idx % ST;
        float s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
        for (int k = 0; k < 11; ++k) {
            const float w = gw[k];
            s0 += w * in[0][r][q + k]; s1 += w * in[1][r][q + k]; s2 += w * in[2][r][q + k];
        }
        hb[0][r][q] = s0; hb[1][r][q] = s1; hb[2][r][q] = s2;
    }
    __syncthreads();
    const int q = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = (threadIdx.x >> 5) + 8 * i;
        const int y = y0 + r, x = x0 + q;
        if (y < row1 && y < H && x < W) {
            float s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const float w = gw[k];
                s0 += w * hb[0][r + k][q]; s1 += w * hb[1][r + k][q]; s2 += w * hb[2][r + k][q];
            }
            const size_t pid = (size_t)c * H * W + (size_t)y * W + x;
            const float p = img[pid], v = gt[pid];
            const float dssim = s0 + 2.0f * p * s1 + v * s2;
            const float diff = p - v;
            const float sgn = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
            g_image[pid] = w_l1 * sgn - w_ssim * dssim;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Fused training path: two kernels instead of four.
//   rgs_composite_ssim_fwd_kernel   folds the K partial slots of a 42x42 pixel patch (front to back) while it fills
//                                   the shared-memory tile of the SSIM filter: the composited image is never read
//                                   back from global memory; it is written once (tile interior) for the backward.
//   rgs_ssim_composite_bwd_kernel   filters the derivative maps, forms d(loss)/d(image) in registers and writes
//                                   d(loss)/d(partial_k) for every partial straight away (into peer-mapped gradient
//                                   images when the partial came from another rank).
// The arithmetic per pixel is the one of the four separate kernels above, in the same order.
// ---------------------------------------------------------------------------------------------
struct FusedFwdSmem {
    float img[3][SH_][SH_ + 1];
    float gt[SH_][SH_ + 1];
    float hb[5][SH_][ST];
    float red[3][8];
};

// A 2 x 2 cluster of blocks covers a 64 x 64 patch. The 5-pixel rims that neighbouring tiles need of each other are
// composited once, by the block whose tile holds them, and the other blocks of the cluster read them out of that
// block's shared memory (distributed shared memory): 37 x 37 instead of 42 x 42 composites per block, each of which
// costs K 16-byte loads. CL = 1 is the kernel without clusters (every block composites its whole 42 x 42 window).
template <int CL>
__global__ void __launch_bounds__(256) rgs_composite_ssim_fwd_kernel(
    const __grid_constant__ RgsPartialPtrs parts, int K, float bg0, float bg1, float bg2, const float* __restrict__ gt,
    int H, int W, int crow0, int crow1, int srow0, int srow1, float* __restrict__ image, float* __restrict__ trans,
    float* __restrict__ dmaps, double* __restrict__ sums) {
    extern __shared__ __align__(16) unsigned char fused_raw[];
    FusedFwdSmem& sm = *reinterpret_cast<FusedFwdSmem*>(fused_raw);
    float gw[11];
    ssim_window(gw);
    const int x0 = blockIdx.x * ST, y0 = crow0 + blockIdx.y * ST;
    const size_t HW = (size_t)H * W;
    // position of this block in its cluster; a window column q (row r) belongs to the neighbour when it lies in the
    // neighbour's tile: q >= 37 for the left block of a pair, q < 5 for the right one
    const int cx = CL > 1 ? (int)(blockIdx.x & 1) : 0, cy = CL > 1 ? (int)(blockIdx.y & 1) : 0;
    for (int idx = threadIdx.x; idx < SH_ * SH_; idx += 256) {
        const int r = idx / SH_, q = idx % SH_;
        if (CL > 1) {
            const bool mine_x = cx == 0 ? q < 5 + ST : q >= 5, mine_y = cy == 0 ? r < 5 + ST : r >= 5;
            if (!(mine_x && mine_y)) continue;
        }
        const int y = y0 + r - 5, x = x0 + q - 5;
        float c0 = 0.f, c1 = 0.f, c2 = 0.f;
        // rows beyond crow1 + 5 feed no output of this launch, and the partial slots need not hold them
        if (y >= 0 && y < H && x >= 0 && x < W && y >= crow0 - 5 && y < crow1 + 5) {
            const size_t pid = (size_t)y * W + x;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, t = 1.f;
            for (int k = 0; k < K; ++k) {
                const float4 v = reinterpret_cast<const float4*>(parts.p[k])[pid];
                a0 += t * v.x; a1 += t * v.y; a2 += t * v.z;
                t *= v.w;
            }
            c0 = a0 + bg0 * t; c1 = a1 + bg1 * t; c2 = a2 + bg2 * t;
            if (r >= 5 && r < 5 + ST && q >= 5 && q < 5 + ST && y < crow1) {
                image[pid] = c0; image[HW + pid] = c1; image[2 * HW + pid] = c2;
                trans[pid] = t;
            }
        }
        sm.img[0][r][q] = c0; sm.img[1][r][q] = c1; sm.img[2][r][q] = c2;
    }
    if (CL > 1) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();  // every block of the cluster has composited the part of the patch it owns
        for (int idx = threadIdx.x; idx < SH_ * SH_; idx += 256) {
            const int r = idx / SH_, q = idx % SH_;
            const int ox = cx == 0 ? (q >= 5 + ST ? 1 : 0) : (q < 5 ? 0 : 1);
            const int oy = cy == 0 ? (r >= 5 + ST ? 1 : 0) : (r < 5 ? 0 : 1);
            if (ox == cx && oy == cy) continue;
            // the same pixel in the owner's window: one tile further left / up per step of the cluster index
            const int rq = q + ST * (cx - ox), rr = r + ST * (cy - oy);
            const FusedFwdSmem* peer = cluster.map_shared_rank(&sm, (unsigned)(ox + 2 * oy));
            sm.img[0][r][q] = peer->img[0][rr][rq];
            sm.img[1][r][q] = peer->img[1][rr][rq];
            sm.img[2][r][q] = peer->img[2][rr][rq];
        }
        cluster.sync();  // nobody reads a neighbour's shared memory after this, so any block may finish first
    }
    float l1 = 0.f, ss = 0.f, l2 = 0.f;
    const int q = threadIdx.x & 31;
    for (int c = 0; c < 3; ++c) {
        const float* b = gt + (size_t)c * HW;
        for (int idx = threadIdx.x; idx < SH_ * SH_; idx += 256) {
            const int r = idx / SH_, qq = idx % SH_;
            const int y = y0 + r - 5, x = x0 + qq - 5;
            sm.gt[r][qq] = (y >= 0 && y < H && x >= 0 && x < W) ? b[(size_t)y * W + x] : 0.f;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < SH_ * ST; idx += 256) {
            const int r = idx / ST, qq = idx % ST;
            float m1 = 0, m2 = 0, e11 = 0, e22 = 0, e12 = 0;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const float p = sm.img[c][r][qq + k], v = sm.gt[r][qq + k], w = gw[k];
                m1 += w * p; m2 += w * v; e11 += w * p * p; e22 += w * v * v; e12 += w * p * v;
            }
            sm.hb[0][r][qq] = m1; sm.hb[1][r][qq] = m2; sm.hb[2][r][qq] = e11; sm.hb[3][r][qq] = e22; sm.hb[4][r][qq] = e12;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = (threadIdx.x >> 5) + 8 * i;
            const int y = y0 + r, x = x0 + q;
            if (y < crow1 && y < H && x < W) {
                float m[5] = {0, 0, 0, 0, 0};
#pragma unroll
                for (int k = 0; k < 11; ++k) {
                    const float w = gw[k];
#pragma unroll
                    for (int j = 0; j < 5; ++j) m[j] += w * sm.hb[j][r + k][q];
                }
                float d[3];
                const float sv = rgs_ssim_pixel(m[0], m[1], m[2], m[3], m[4], d);
                const size_t pid = (size_t)c * HW + (size_t)y * W + x;
                const size_t plane = (size_t)3 * HW;
                dmaps[pid] = d[0]; dmaps[plane + pid] = d[1]; dmaps[2 * plane + pid] = d[2];
                if (y >= srow0 && y < srow1) {
                    const float diff = sm.img[c][r + 5][q + 5] - sm.gt[r + 5][q + 5];
                    l1 += fabsf(diff); ss += sv; l2 += diff * diff;
                }
            }
        }
        __syncthreads();  // hb and the gt tile are reused by the next channel
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        l1 += __shfl_xor_sync(0xffffffffu, l1, d);
        ss += __shfl_xor_sync(0xffffffffu, ss, d);
        l2 += __shfl_xor_sync(0xffffffffu, l2, d);
    }
    if ((threadIdx.x & 31) == 0) { sm.red[0][threadIdx.x >> 5] = l1; sm.red[1][threadIdx.x >> 5] = ss; sm.red[2][threadIdx.x >> 5] = l2; }
    __syncthreads();
    if (threadIdx.x < 3) {
        double t = 0;
        for (int w = 0; w < 8; ++w) t += (double)sm.red[threadIdx.x][w];
        atomicAdd(&sums[threadIdx.x], t);
    }
}

template <int KMAX>
__global__ void __launch_bounds__(256) rgs_ssim_composite_bwd_kernel(
    const __grid_constant__ RgsPartialPtrs parts, const __grid_constant__ RgsGradPtrs grads, int K, float bg0, float bg1,
    float bg2, const float* __restrict__ img, const float* __restrict__ gt, const float* __restrict__ dmaps, int H, int W,
    int row0, int row1, int vrow0, int vrow1, float w_l1, float w_ssim, float* __restrict__ g_image, int marked) {
    __shared__ float in[3][SH_][SH_ + 1];
    __shared__ float hb[3][SH_][ST];
    float gw[11];
    ssim_window(gw);
    const int x0 = blockIdx.x * ST, y0 = row0 + blockIdx.y * ST;
    const size_t HW = (size_t)H * W, plane = 3 * HW;
    const int q = threadIdx.x & 31;
    float g[4][3];
    for (int c = 0; c < 3; ++c) {
        const float* dm = dmaps + (size_t)c * HW;
        for (int idx = threadIdx.x; idx < SH_ * SH_; idx += 256) {
            const int r = idx / SH_, qq = idx % SH_;
            const int y = y0 + r - 5, x = x0 + qq - 5;
            const bool ok = y >= vrow0 && y < vrow1 && x >= 0 && x < W;
            const size_t o = (size_t)y * W + x;
            in[0][r][qq] = ok ? dm[o] : 0.f;
            in[1][r][qq] = ok ? dm[plane + o] : 0.f;
            in[2][r][qq] = ok ? dm[2 * plane + o] : 0.f;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < SH_ * ST; idx += 256) {
            const int r = idx / ST, qq = idx % ST;
            float s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const float w = gw[k];
                s0 += w * in[0][r][qq + k]; s1 += w * in[1][r][qq + k]; s2 += w * in[2][r][qq + k];
            }
            hb[0][r][qq] = s0; hb[1][r][qq] = s1; hb[2][r][qq] = s2;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = (threadIdx.x >> 5) + 8 * i;
            const int y = y0 + r, x = x0 + q;
            g[i][c] = 0.f;
            if (y < row1 && y < H && x < W) {
                float s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
                for (int k = 0; k < 11; ++k) {
                    const float w = gw[k];
                    s0 += w * hb[0][r + k][q]; s1 += w * hb[1][r + k][q]; s2 += w * hb[2][r + k][q];
                }
                const size_t pid = (size_t)c * HW + (size_t)y * W + x;
                const float p = img[pid], v = gt[pid];
                const float dssim = s0 + 2.0f * p * s1 + v * s2;
                const float diff = p - v;
                const float sgn = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
                g[i][c] = w_l1 * sgn - w_ssim * dssim;
                if (g_image) g_image[pid] = g[i][c];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = (threadIdx.x >> 5) + 8 * i;
        const int y = y0 + r, x = x0 + q;
        if (!(y < row1 && y < H && x < W)) continue;
        const size_t pid = (size_t)y * W + x;
        composite_pixel_grads<KMAX>(parts, grads, K, pid, g[i][0], g[i][1], g[i][2], bg0, bg1, bg2, marked);
    }
}

extern "C" {

int rgs_cuda_composite_fwd(const float* const* partials, int64_t K, const float* bg, int64_t H, int64_t W,
                           int64_t row0, int64_t row1, float* image, float* trans, void* stream) {
    if (K < 0 || K > RGS_MAX_PARTIALS) return 12;
    if (row1 <= row0) return 0;
    RgsPartialPtrs pp;
    for (int k = 0; k < K; ++k) pp.p[k] = partials[k];
    const int64_t n = (row1 - row0) * W;
    const int64_t want = (n + 255) / 256;
    const unsigned blocks = (unsigned)(want > RGS_SMS * 32 ? RGS_SMS * 32 : want);
    rgs_composite_fwd_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(pp, (int)K, bg[0], bg[1], bg[2], H, W, row0, row1,
                                                                      image, trans);
    return (int)cudaGetLastError();
}

int rgs_cuda_composite_bwd(const float* const* partials, float* const* grads, int64_t K, const float* bg, int64_t H,
                           int64_t W, int64_t row0, int64_t row1, const float* g_image, int64_t marked, void* stream) {
    if (K < 0 || K > RGS_MAX_PARTIALS) return 12;
    if (row1 <= row0) return 0;
    RgsPartialPtrs pp;
    RgsGradPtrs gp;
    for (int k = 0; k < K; ++k) { pp.p[k] = partials[k]; gp.p[k] = grads[k]; }
    const int64_t n = (row1 - row0) * W;
    const int64_t want = (n + 255) / 256;
    const unsigned blocks = (unsigned)(want > RGS_SMS * 32 ? RGS_SMS * 32 : want);
    if (K <= 8)
        rgs_composite_bwd_kernel<8><<<blocks, 256, 0, (cudaStream_t)stream>>>(pp, gp, (int)K, bg[0], bg[1], bg[2], H, W, row0,
                                                                             row1, g_image, marked ? 1 : 0);
    else
        rgs_composite_bwd_kernel<RGS_MAX_PARTIALS><<<blocks, 256, 0, (cudaStream_t)stream>>>(
            pp, gp, (int)K, bg[0], bg[1], bg[2], H, W, row0, row1, g_image, marked ? 1 : 0);
    return (int)cudaGetLastError();
}

// Statistics pass on rows [crow0,crow1) (derivative maps written there); the loss sums count rows
// [srow0,srow1) only. sums: 3 doubles on the device: sum|d|, sum ssim, sum d^2 (accumulated).
int rgs_cuda_ssim_fwd(const float* img, const float* gt, int64_t H, int64_t W, int64_t crow0, int64_t crow1,
                      int64_t srow0, int64_t srow1, float* dmaps, double* sums, void* stream) {
    if (crow1 <= crow0) return 0;
    dim3 grid((unsigned)((W + ST - 1) / ST), (unsigned)((crow1 - crow0 + ST - 1) / ST), 3);
    rgs_ssim_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(img, gt, (int)H, (int)W, (int)crow0, (int)crow1,
                                                                (int)srow0, (int)srow1, dmaps, sums);
    return (int)cudaGetLastError();
}

// Gradient pass on rows [row0,row1); derivative maps are valid on rows [vrow0,vrow1).
int rgs_cuda_ssim_bwd(const float* img, const float* gt, const float* dmaps, int64_t H, int64_t W, int64_t row0,
                      int64_t row1, int64_t vrow0, int64_t vrow1, double w_l1, double w_ssim, float* g_image,
                      void* stream) {
    if (row1 <= row0) return 0;
    dim3 grid((unsigned)((W + ST - 1) / ST), (unsigned)((row1 - row0 + ST - 1) / ST), 3);
    rgs_ssim_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(img, gt, dmaps, (int)H, (int)W, (int)row0, (int)row1,
                                                                (int)vrow0, (int)vrow1, (float)w_l1, (float)w_ssim,
                                                                g_image);
    return (int)cudaGetLastError();
}

// Fused forward of the training path: composite rows [crow0-5, crow1+5) of the K partials on the fly, write the
// composited image / transmittance on rows [crow0,crow1), the SSIM derivative maps there, and accumulate the loss
// sums over rows [srow0,srow1).
// 1: the fused forward runs as 2 x 2 thread-block clusters that share their rims through distributed shared memory
// (RGS_LOSS_CLUSTER=1); 0: every block composites its whole window (default: at 1600 x 1036 with two partials the
// cluster variant measured 0.45 ms per step against 0.41 ms; the partials it saves re-reading sit in L2, and the two
// cluster barriers cost more than those loads). Returns the old setting.
static int g_loss_cluster = -1;
int rgs_cuda_loss_cluster(int on) {
    if (g_loss_cluster < 0) {
        const char* e = getenv("RGS_LOSS_CLUSTER");
        g_loss_cluster = (e && e[0] == '1') ? 1 : 0;
    }
    const int old = g_loss_cluster;
    g_loss_cluster = on ? 1 : 0;
    return old;
}

int rgs_cuda_composite_ssim_fwd(const float* const* partials, int64_t K, const float* bg, const float* gt, int64_t H,
                                int64_t W, int64_t crow0, int64_t crow1, int64_t srow0, int64_t srow1, float* image,
                                float* trans, float* dmaps, double* sums, void* stream) {
    if (K < 0 || K > RGS_MAX_PARTIALS) return 12;
    if (crow1 <= crow0) return 0;
    RgsPartialPtrs pp;
    for (int k = 0; k < K; ++k) pp.p[k] = partials[k];
    if (g_loss_cluster < 0) {
        const char* e = getenv("RGS_LOSS_CLUSTER");
        g_loss_cluster = (e && e[0] == '1') ? 1 : 0;
    }
    const bool use_cluster = g_loss_cluster != 0;
    static bool attr_set = false;
    if (!attr_set) {
        RGS_CUDA_CHECK(cudaFuncSetAttribute(rgs_composite_ssim_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)sizeof(FusedFwdSmem)));
        RGS_CUDA_CHECK(cudaFuncSetAttribute(rgs_composite_ssim_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)sizeof(FusedFwdSmem)));
        attr_set = true;
    }
    dim3 grid((unsigned)((W + ST - 1) / ST), (unsigned)((crow1 - crow0 + ST - 1) / ST), 1);
    if (!use_cluster) {
        rgs_composite_ssim_fwd_kernel<1><<<grid, 256, sizeof(FusedFwdSmem), (cudaStream_t)stream>>>(
            pp, (int)K, bg[0], bg[1], bg[2], gt, (int)H, (int)W, (int)crow0, (int)crow1, (int)srow0, (int)srow1, image,
            trans, dmaps, sums);
        return (int)cudaGetLastError();
    }
    // clusters of 2 x 2 blocks: the grid is rounded up to whole clusters; a block beyond the image or the row band
    // writes nothing (every access is masked by the pixel's own coordinates) but still serves its neighbours' rims
    grid.x = (grid.x + 1) & ~1u;
    grid.y = (grid.y + 1) & ~1u;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = sizeof(FusedFwdSmem);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 2;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RGS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rgs_composite_ssim_fwd_kernel<2>, pp, (int)K, bg[0], bg[1], bg[2], gt, (int)H,
                                      (int)W, (int)crow0, (int)crow1, (int)srow0, (int)srow1, image, trans, dmaps, sums));
    return (int)cudaGetLastError();
}

// Fused backward: d(loss)/d(image) on rows [row0,row1) from the derivative maps (valid on [vrow0,vrow1)) and, in the
// same kernel, d(loss)/d(partial_k) into grads[k]; g_image (optional) receives d(loss)/d(image).
int rgs_cuda_ssim_composite_bwd(const float* const* partials, float* const* grads, int64_t K, const float* bg,
                                const float* img, const float* gt, const float* dmaps, int64_t H, int64_t W, int64_t row0,
                                int64_t row1, int64_t vrow0, int64_t vrow1, double w_l1, double w_ssim, float* g_image,
                                int64_t marked, void* stream) {
    if (K < 0 || K > RGS_MAX_PARTIALS) return 12;
    if (row1 <= row0) return 0;
    RgsPartialPtrs pp;
    RgsGradPtrs gp;
    for (int k = 0; k < K; ++k) { pp.p[k] = partials[k]; gp.p[k] = grads[k]; }
    dim3 grid((unsigned)((W + ST - 1) / ST), (unsigned)((row1 - row0 + ST - 1) / ST), 1);
    if (K <= 8)
        rgs_ssim_composite_bwd_kernel<8><<<grid, 256, 0, (cudaStream_t)stream>>>(
            pp, gp, (int)K, bg[0], bg[1], bg[2], img, gt, dmaps, (int)H, (int)W, (int)row0, (int)row1, (int)vrow0, (int)vrow1,
            (float)w_l1, (float)w_ssim, g_image, marked ? 1 : 0);
    else
        rgs_ssim_composite_bwd_kernel<RGS_MAX_PARTIALS><<<grid, 256, 0, (cudaStream_t)stream>>>(
            pp, gp, (int)K, bg[0], bg[1], bg[2], img, gt, dmaps, (int)H, (int)W, (int)row0, (int)row1, (int)vrow0, (int)vrow1,
            (float)w_l1, (float)w_ssim, g_image, marked ? 1 : 0);
    return (int)cudaGetLastError();
}

}  // extern "C"
