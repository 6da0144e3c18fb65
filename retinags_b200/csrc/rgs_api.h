// C ABI of the native libraries.
//
// Two shared objects export the same entry points with different prefixes:
//   librgs_cpu.so   rgs_cpu_*   host pointers, OpenMP loops around the shared math (rgs_math.h)
//   librgs_cuda.so  rgs_cuda_*  device pointers, sm_100a kernels, last argument is a cudaStream_t
// Both are driven from Python through ctypes (retinags_b200/ops/native.py); nothing here allocates
// memory: every buffer, scratch space included, is owned by the caller.
//
// Replaces the pybind module of the reference
// (rasterization_kernels/diff-gaussian-rasterization-half-gaussian/ext.cpp:15-19,
//  rasterize_points.cu:35-220), which allocates its outputs and three resizable byte buffers per
// call and copies the instance count to the host between scan and sort.
#pragma once
#include <stdint.h>
#include "rgs_math.h"

// One block of Gaussians that a render task reads (the sub-model's own Gaussians, or the ones it
// borrows from neighbouring sub-models). Gradient/statistic pointers may be null.
struct RgsSegment {
    const float* xyz;      // (count,3)
    const float* sh;       // (count,16,3) coefficient-major
    const float* scale;    // (count,3)
    const float* rot;      // (count,4) (w,x,y,z)
    const float* opacity;  // (count,1)
    float* g_xyz;
    float* g_sh;
    float* g_scale;
    float* g_rot;
    float* g_opacity;
    float* g_mean2d;       // (count,2) NDC-scaled screen gradient of this view (overwritten), optional
    float* stat_grad;      // (count) += |screen gradient|, optional
    float* stat_denom;     // (count) += 1 for every view in which the Gaussian is visible, optional
    float* stat_maxrad;    // (count) = max(., radius), optional
    uint8_t* touched;      // (count) optional: 1 once a gradient row was written this step. Rows with 0 are
                           // known to hold zero gradients, so the first writer stores instead of adding and
                           // the optimiser neither reads nor clears them.
    int64_t count;
};

// counters layout (int32, device/host memory owned by the caller)
#define RGS_CNT_VIS 0       // number of visible splats written
#define RGS_CNT_INST 1      // number of (tile, splat) instances requested
#define RGS_CNT_OVERFLOW 2  // set to 1 when CNT_INST exceeded the capacity (instances were dropped)
#define RGS_CNT_STATUS 3    // error/status word of bounded waits (0 = ok)
#define RGS_CNT_CAND 4      // candidates that survived the conservative cull (two-phase projection)
#define RGS_CNT_INST2 5     // instances of the second depth slab (two-slab binning)
#define RGS_CNT_WORDS 8

// lr table of the fused Adam: columns of the 59-float record grouped by learning rate
#define RGS_LR_XYZ 0
#define RGS_LR_FDC 1
#define RGS_LR_FREST 2
#define RGS_LR_SCALE 3
#define RGS_LR_ROT 4
#define RGS_LR_OPACITY 5
