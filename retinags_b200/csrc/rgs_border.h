// Selection of border Gaussians, shared by the CUDA kernel (rgs_border.cu) and the CPU twin (rgs_cpu.cpp).
//
// A Gaussian is lent to sub-model d when the axis-aligned box around its centre with half-size
// 3 * exp(max log-scale) * (1 + margin) leaves its own sub-model's box and overlaps the box of d. The reference
// evaluates this with boolean-mask gathers per destination in every iteration
// (parallel_utils/basic_parallel_trainer/result_aggregator.py:55-121); here one pass yields a bit per destination.
#pragma once
#include <math.h>
#include <stdint.h>
#include "rgs_math.h"

#define RGS_MAX_BORDER_MODELS 63  // bits of the (signed 64-bit) mask

// boxes: M x 6 floats (lo xyz, hi xyz). Returns the mask of destinations (bit d), 0 for interior Gaussians.
RGS_HD int64_t rgs_border_mask(const float* xyz, const float* log_scale, const float* boxes, int M, int self, float margin) {
    const float ext = 3.0f * expf(fmaxf(log_scale[0], fmaxf(log_scale[1], log_scale[2]))) * (1.0f + margin);
    const float lo[3] = {xyz[0] - ext, xyz[1] - ext, xyz[2] - ext}, hi[3] = {xyz[0] + ext, xyz[1] + ext, xyz[2] + ext};
    const float* own = boxes + 6 * self;
    bool crosses = false;
    for (int a = 0; a < 3; ++a) crosses = crosses || lo[a] <= own[a] || hi[a] > own[3 + a];
    if (!crosses) return 0;
    int64_t mask = 0;
    for (int d = 0; d < M; ++d) {
        if (d == self) continue;
        const float* b = boxes + 6 * d;
        bool overlap = true;
        for (int a = 0; a < 3; ++a) overlap = overlap && hi[a] > b[a] && lo[a] <= b[3 + a];
        if (overlap) mask |= (int64_t)1 << d;
    }
    return mask;
}
