// Border-Gaussian exchange kernels for the peer-to-peer path.
//
// A sub-model lends the Gaussians whose extent reaches into a neighbour's box. The reference gathers them with
// boolean masks, concatenates 62-float rows and ships them with NCCL send/recv in both directions every iteration
// (parallel_utils/basic_parallel_trainer/result_aggregator.py:55-147, task_utils.py:230-362,
// trainer4tree_partition.py:354-388,521-571). Here
//   rgs_border_pack_kernel     gathers the selected rows from the owner's column groups and stores them straight
//                              into the borrowing rank's segment (column groups in peer-mapped memory: what
//                              arrives IS the render segment, nothing is unpacked);
//   rgs_border_grad_push_kernel stores the gradients of the borrowed rows (59 parameter gradients + the
//                              screen-gradient statistic) into the owner's return ring (peer-mapped);
//   rgs_border_grad_add_kernel adds the returned rows into the owner's gradient block and marks them touched.
// Plain peer stores only; ordering is by the epoch flags of rgs_p2p.cu.
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"
#include "rgs_border.h"

struct RgsColumns { float* xyz; float* sh; float* scale; float* rot; float* opacity; };
struct RgsConstColumns { const float* xyz; const float* sh; const float* scale; const float* rot; const float* opacity; };

// 15 units per row: 12 float4 of SH, xyz, scale+opacity, rotation
// only_if (optional, one byte per row of the owner): rows whose byte is 0 are skipped. The owner passes its `active`
// marks between two full packs: a row without Adam moments has not moved since the borrower received it.
__global__ void __launch_bounds__(256) rgs_border_pack_kernel(const RgsConstColumns src, const int64_t* __restrict__ idx,
                                                              int64_t n, const RgsColumns dst, int64_t dst_row0,
                                                              const uint8_t* __restrict__ only_if) {
    const int64_t total = n * 15;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = u / 15;
        const int k = (int)(u - r * 15);
        const int64_t i = idx[r], o = dst_row0 + r;
        if (only_if && !only_if[i]) continue;
        if (k < 12) {
            reinterpret_cast<float4*>(dst.sh + 48 * o)[k] = reinterpret_cast<const float4*>(src.sh + 48 * i)[k];
        } else if (k == 12) {
            dst.xyz[3 * o] = src.xyz[3 * i]; dst.xyz[3 * o + 1] = src.xyz[3 * i + 1]; dst.xyz[3 * o + 2] = src.xyz[3 * i + 2];
        } else if (k == 13) {
            dst.scale[3 * o] = src.scale[3 * i]; dst.scale[3 * o + 1] = src.scale[3 * i + 1]; dst.scale[3 * o + 2] = src.scale[3 * i + 2];
            dst.opacity[o] = src.opacity[i];
        } else {
            reinterpret_cast<float4*>(dst.rot)[o] = reinterpret_cast<const float4*>(src.rot)[i];
        }
    }
}

// rows: (n, 60) row-major = [g_xyz 3, stat 1 | g_sh 48 | g_scale 3, g_opacity 1 | g_rot 4] (16-byte aligned groups);
// flags: one byte per row. Only rows that received a gradient this step (the borrower's `touched` marks) travel:
// their flag is 1, every other row costs its flag byte alone. The borrower's marks and statistic are cleared on the
// way (second kernel), so that nothing has to be zeroed before the next step: the first gradient of a step is stored,
// not added (see rgs_geom_bwd_kernel).
__global__ void __launch_bounds__(256) rgs_border_grad_push_kernel(const RgsConstColumns g, const float* __restrict__ stat,
                                                                   const uint8_t* __restrict__ touched, int64_t row0,
                                                                   int64_t n, float* __restrict__ rows,
                                                                   uint8_t* __restrict__ flags) {
    const int64_t total = n * 15;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = u / 15;
        const int k = (int)(u - r * 15);
        const int64_t i = row0 + r;
        const bool live = !touched || touched[i] != 0;
        if (k == 12 && flags) flags[r] = live ? 1 : 0;
        if (!live) continue;
        float* o = rows + 60 * r;
        if (k < 12) {
            reinterpret_cast<float4*>(o + 4)[k] = reinterpret_cast<const float4*>(g.sh + 48 * i)[k];
        } else if (k == 12) {
            o[0] = g.xyz[3 * i]; o[1] = g.xyz[3 * i + 1]; o[2] = g.xyz[3 * i + 2]; o[3] = stat ? stat[i] : 0.f;
        } else if (k == 13) {
            o[52] = g.scale[3 * i]; o[53] = g.scale[3 * i + 1]; o[54] = g.scale[3 * i + 2]; o[55] = g.opacity[i];
        } else {
            reinterpret_cast<float4*>(o + 56)[0] = reinterpret_cast<const float4*>(g.rot)[i];
        }
    }
}

__global__ void __launch_bounds__(256) rgs_border_clear_marks_kernel(uint8_t* __restrict__ touched, float* __restrict__ stat,
                                                                     int64_t row0, int64_t n) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n; r += (int64_t)gridDim.x * blockDim.x)
        if (touched[row0 + r]) { touched[row0 + r] = 0; if (stat) stat[row0 + r] = 0.f; }
}

// inverse of the push layout: [xyz 3, stat 1 | sh 48 | scale 3, opacity 1 | rot 4]; rows whose flag is 0 are skipped
__global__ void __launch_bounds__(256) rgs_border_grad_add_kernel(const float* __restrict__ rows,
                                                                  const uint8_t* __restrict__ flags,
                                                                  const int64_t* __restrict__ idx,
                                                                  int64_t n, const RgsColumns g, float* __restrict__ stat,
                                                                  uint8_t* __restrict__ touched) {
    const int64_t total = n * 15;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = u / 15;
        const int k = (int)(u - r * 15);
        if (flags && !flags[r]) continue;
        const int64_t i = idx[r];
        const float* o = rows + 60 * r;
        // the owner's row may be untouched so far in this step: its gradient words are then stale, not zero
        const bool first = touched && touched[i] == 0;
        if (k < 12) {
            float4 a = first ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(g.sh + 48 * i)[k];
            const float4 b = reinterpret_cast<const float4*>(o + 4)[k];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            reinterpret_cast<float4*>(g.sh + 48 * i)[k] = a;
        } else if (k == 12) {
            if (first) { g.xyz[3 * i] = o[0]; g.xyz[3 * i + 1] = o[1]; g.xyz[3 * i + 2] = o[2]; }
            else { g.xyz[3 * i] += o[0]; g.xyz[3 * i + 1] += o[1]; g.xyz[3 * i + 2] += o[2]; }
            if (stat) stat[i] += o[3];
        } else if (k == 13) {
            if (first) { g.scale[3 * i] = o[52]; g.scale[3 * i + 1] = o[53]; g.scale[3 * i + 2] = o[54]; g.opacity[i] = o[55]; }
            else { g.scale[3 * i] += o[52]; g.scale[3 * i + 1] += o[53]; g.scale[3 * i + 2] += o[54]; g.opacity[i] += o[55]; }
        } else {
            float4 a = first ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<float4*>(g.rot)[i];
            const float4 b = reinterpret_cast<const float4*>(o + 56)[0];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            reinterpret_cast<float4*>(g.rot)[i] = a;
        }
    }
}

// after all units of the launch above have read the marks: the rows that received something count as touched
__global__ void __launch_bounds__(256) rgs_border_mark_touched_kernel(const uint8_t* __restrict__ flags,
                                                                      const int64_t* __restrict__ idx, int64_t n,
                                                                      uint8_t* __restrict__ touched) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n; r += (int64_t)gridDim.x * blockDim.x)
        if (!flags || flags[r]) touched[idx[r]] = 1;
}

// one destination bit mask per Gaussian (see rgs_border.h); boxes: M x 6 floats in device memory
__global__ void __launch_bounds__(256) rgs_border_mask_kernel(const float* __restrict__ xyz, const float* __restrict__ scale,
                                                              int64_t n, const float* __restrict__ boxes, int M, int self,
                                                              float margin, int64_t* __restrict__ masks) {
    __shared__ float sb[6 * RGS_MAX_BORDER_MODELS];
    for (int k = threadIdx.x; k < 6 * M; k += blockDim.x) sb[k] = boxes[k];
    __syncthreads();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float p[3] = {xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2]};
        const float s[3] = {scale[3 * i], scale[3 * i + 1], scale[3 * i + 2]};
        masks[i] = rgs_border_mask(p, s, sb, M, self, margin);
    }
}

static inline unsigned border_grid(int64_t n) {
    const int64_t want = (n * 15 + 255) / 256;
    return (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 16 ? RGS_SMS * 16 : want));
}

extern "C" {

// src/dst: 5 pointers each (xyz, sh, scale, rot, opacity); dst may be peer-mapped.
int rgs_cuda_border_pack(const float* const* src, const int64_t* idx, int64_t n, float* const* dst, int64_t dst_row0,
                         const uint8_t* only_if, void* stream) {
    if (n <= 0) return 0;
    RgsConstColumns s{src[0], src[1], src[2], src[3], src[4]};
    RgsColumns d{dst[0], dst[1], dst[2], dst[3], dst[4]};
    rgs_border_pack_kernel<<<border_grid(n), 256, 0, (cudaStream_t)stream>>>(s, idx, n, d, dst_row0, only_if);
    return (int)cudaGetLastError();
}

// masks[i]: bit d set when Gaussian i of sub-model `self` is lent to sub-model d (M <= 63 sub-models).
int rgs_cuda_border_mask(const float* xyz, const float* scale, int64_t n, const float* boxes, int64_t M, int64_t self,
                         double margin, int64_t* masks, void* stream) {
    if (M < 1 || M > RGS_MAX_BORDER_MODELS || self < 0 || self >= M) return 17;
    if (n <= 0) return 0;
    const int64_t want = (n + 255) / 256;
    const unsigned blocks = (unsigned)(want > RGS_SMS * 32 ? RGS_SMS * 32 : want);
    rgs_border_mask_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(xyz, scale, n, boxes, (int)M, (int)self, (float)margin, masks);
    return (int)cudaGetLastError();
}

// touched / stat belong to the borrower's segment (rows row0 .. row0+n); rows / flags are the owner's return ring
// (peer-mapped). The marks and the statistic of the pushed rows are cleared afterwards.
int rgs_cuda_border_grad_push(const float* const* g, float* stat, uint8_t* touched, int64_t row0, int64_t n, float* rows,
                              uint8_t* flags, void* stream) {
    if (n <= 0) return 0;
    RgsConstColumns s{g[0], g[1], g[2], g[3], g[4]};
    rgs_border_grad_push_kernel<<<border_grid(n), 256, 0, (cudaStream_t)stream>>>(s, stat, touched, row0, n, rows, flags);
    if (touched) {
        const int64_t want = (n + 255) / 256;
        rgs_border_clear_marks_kernel<<<(unsigned)(want > RGS_SMS * 8 ? RGS_SMS * 8 : want), 256, 0, (cudaStream_t)stream>>>(
            touched, stat, row0, n);
    }
    return (int)cudaGetLastError();
}

int rgs_cuda_border_grad_add(const float* rows, const uint8_t* flags, const int64_t* idx, int64_t n, float* const* g,
                             float* stat, uint8_t* touched, void* stream) {
    if (n <= 0) return 0;
    RgsColumns d{g[0], g[1], g[2], g[3], g[4]};
    rgs_border_grad_add_kernel<<<border_grid(n), 256, 0, (cudaStream_t)stream>>>(rows, flags, idx, n, d, stat, touched);
    if (touched) {
        const int64_t want = (n + 255) / 256;
        rgs_border_mark_touched_kernel<<<(unsigned)(want > RGS_SMS * 8 ? RGS_SMS * 8 : want), 256, 0, (cudaStream_t)stream>>>(
            flags, idx, n, touched);
    }
    return (int)cudaGetLastError();
}

}  // extern "C"
