// Model surgery shared by the CUDA kernels (rgs_surgery.cu) and the CPU twin (rgs_cpu.cpp): adaptive density control
// (clone / split / prune decided per Gaussian, survivors and new Gaussians compacted into fresh buffers together with
// their Adam moments) and the 177-float migration records.
//
// The reference decides clone/split/prune with boolean masks and rebuilds the seven parameter tensors and their
// optimiser state with cat/mask surgery (scene/gaussian_nn_module.py:589-751, 1002-1026), sampling the split offsets
// on the CPU (:707-708).  Here one classification pass yields a 4-bit code per Gaussian, a scan turns the codes into
// destinations, and one gather pass writes parameters and moments of every survivor / clone / split child; the split
// offsets come from a counter-based Philox4x32-10 generator keyed by (seed, row, child), so that the result does not
// depend on the launch geometry and the host twin reproduces it.
#pragma once
#include <math.h>
#include <stdint.h>
#include "rgs_math.h"

#define RGS_SURGERY_KEEP 1u
#define RGS_SURGERY_CLONE 2u
#define RGS_SURGERY_CHILD_A 4u
#define RGS_SURGERY_CHILD_B 8u
#define RGS_SURGERY_BLOCK 1024  // rows per scan block

struct RgsDensifyCfg {
    float max_grad;      // threshold on the mean screen-space gradient
    float dense_extent;  // percent_dense * scene extent: clone below, split above
    float min_opacity;   // prune below
    float max_screen;    // prune when the largest screen radius exceeds it (<= 0: no size-based pruning at all)
    float world_max;     // prune when the largest axis exceeds it (only with size-based pruning)
    int skip_clone, skip_split, skip_prune, no_grow;
    uint64_t seed;
};

// five column groups of one buffer (xyz 3 | sh 48 | scale 3 | rot 4 | opacity 1), `cap` rows each
struct RgsBlock { float* xyz; float* sh; float* scale; float* rot; float* opacity; };
struct RgsConstBlock { const float* xyz; const float* sh; const float* scale; const float* rot; const float* opacity; };

RGS_HD RgsBlock rgs_block_of(float* base, int64_t cap) {
    return RgsBlock{base, base + 3 * cap, base + 51 * cap, base + 54 * cap, base + 58 * cap};
}
RGS_HD RgsConstBlock rgs_const_block_of(const float* base, int64_t cap) {
    return RgsConstBlock{base, base + 3 * cap, base + 51 * cap, base + 54 * cap, base + 58 * cap};
}

RGS_HD void rgs_philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t* out) {
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// three independent standard normals for (seed, row, child)
RGS_HD void rgs_normal3(uint64_t seed, int64_t row, int child, float* n) {
    uint32_t x[4];
    rgs_philox4x32((uint32_t)row, (uint32_t)((uint64_t)row >> 32), (uint32_t)child, 0x52474253u, (uint32_t)seed,
                   (uint32_t)(seed >> 32), x);
    const float k = 1.0f / 16777216.0f, two_pi = 6.28318530717958647692f;
    const float u0 = ((float)(x[0] >> 8) + 0.5f) * k, u1 = ((float)(x[1] >> 8) + 0.5f) * k;
    const float u2 = ((float)(x[2] >> 8) + 0.5f) * k, u3 = ((float)(x[3] >> 8) + 0.5f) * k;
    const float r0 = sqrtf(-2.0f * logf(u0)), r1 = sqrtf(-2.0f * logf(u2));
    n[0] = r0 * cosf(two_pi * u1);
    n[1] = r0 * sinf(two_pi * u1);
    n[2] = r1 * cosf(two_pi * u3);
}

// 4-bit fate of one Gaussian (see RGS_SURGERY_*)
RGS_HD uint32_t rgs_densify_code(const RgsDensifyCfg& c, const float* scale, float opacity_logit, float accum, float denom,
                                 float maxrad) {
    float g = accum / denom;
    if (!(g == g) || isinf(g)) g = 0.0f;
    const float ms = expf(fmaxf(scale[0], fmaxf(scale[1], scale[2])));
    const bool hot = !c.no_grow && g >= c.max_grad;
    const bool sel_clone = hot && ms <= c.dense_extent && !c.skip_clone;
    const bool sel_split = hot && ms > c.dense_extent && !c.skip_split;
    const bool size_rule = c.max_screen > 0.0f;
    const bool transparent = !c.skip_prune && rgs_sigmoid(opacity_logit) < c.min_opacity;
    const bool prune_self = transparent || (!c.skip_prune && size_rule && (ms > c.world_max || maxrad > c.max_screen));
    const bool prune_clone = transparent || (!c.skip_prune && size_rule && ms > c.world_max);
    const bool prune_child = transparent || (!c.skip_prune && size_rule && ms / 1.6f > c.world_max);
    uint32_t code = 0;
    if (!sel_split && !prune_self) code |= RGS_SURGERY_KEEP;
    if (sel_clone && !prune_clone) code |= RGS_SURGERY_CLONE;
    if (sel_split && !prune_child) code |= RGS_SURGERY_CHILD_A | RGS_SURGERY_CHILD_B;
    return code;
}

// Write row `i` of the source as row `o` of the destination.  kind 0: survivor (moments travel), 1: clone (zero
// moments), 2/3: split child A/B (sampled position, scale / 1.6, zero moments).
RGS_HD void rgs_surgery_emit(const RgsConstBlock& sp, const RgsConstBlock& sm, const RgsConstBlock& sv, int64_t i,
                             const RgsBlock& dp, const RgsBlock& dm, const RgsBlock& dv, int64_t o, int kind, uint64_t seed) {
    float p[3] = {sp.xyz[3 * i], sp.xyz[3 * i + 1], sp.xyz[3 * i + 2]};
    float s[3] = {sp.scale[3 * i], sp.scale[3 * i + 1], sp.scale[3 * i + 2]};
    const float q[4] = {sp.rot[4 * i], sp.rot[4 * i + 1], sp.rot[4 * i + 2], sp.rot[4 * i + 3]};
    if (kind >= 2) {
        float n[3], R[9];
        rgs_normal3(seed, i, kind - 2, n);
        const float inv = 1.0f / sqrtf(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
        const float qn[4] = {q[0] * inv, q[1] * inv, q[2] * inv, q[3] * inv};
        rgs_quat_to_rot(qn, R);
        const float e[3] = {expf(s[0]) * n[0], expf(s[1]) * n[1], expf(s[2]) * n[2]};
        for (int a = 0; a < 3; ++a) p[a] += R[3 * a] * e[0] + R[3 * a + 1] * e[1] + R[3 * a + 2] * e[2];
        for (int a = 0; a < 3; ++a) s[a] = logf(expf(s[a]) / 1.6f);
    }
    for (int a = 0; a < 3; ++a) { dp.xyz[3 * o + a] = p[a]; dp.scale[3 * o + a] = s[a]; }
    for (int a = 0; a < 4; ++a) dp.rot[4 * o + a] = q[a];
    dp.opacity[o] = sp.opacity[i];
    for (int a = 0; a < 48; ++a) dp.sh[48 * o + a] = sp.sh[48 * i + a];
    const bool carry = kind == 0;
    for (int a = 0; a < 3; ++a) {
        dm.xyz[3 * o + a] = carry ? sm.xyz[3 * i + a] : 0.0f; dv.xyz[3 * o + a] = carry ? sv.xyz[3 * i + a] : 0.0f;
        dm.scale[3 * o + a] = carry ? sm.scale[3 * i + a] : 0.0f; dv.scale[3 * o + a] = carry ? sv.scale[3 * i + a] : 0.0f;
    }
    for (int a = 0; a < 4; ++a) {
        dm.rot[4 * o + a] = carry ? sm.rot[4 * i + a] : 0.0f; dv.rot[4 * o + a] = carry ? sv.rot[4 * i + a] : 0.0f;
    }
    dm.opacity[o] = carry ? sm.opacity[i] : 0.0f; dv.opacity[o] = carry ? sv.opacity[i] : 0.0f;
    for (int a = 0; a < 48; ++a) {
        dm.sh[48 * o + a] = carry ? sm.sh[48 * i + a] : 0.0f; dv.sh[48 * o + a] = carry ? sv.sh[48 * i + a] : 0.0f;
    }
}

// position of column c (0..58) of row r inside a buffer with `cap` rows: record order xyz | sh | scale | rot | opacity
RGS_HD int64_t rgs_record_offset(int64_t cap, int64_t r, int c) {
    if (c < 3) return 3 * r + c;
    if (c < 51) return 3 * cap + 48 * r + (c - 3);
    if (c < 54) return 51 * cap + 3 * r + (c - 51);
    if (c < 58) return 54 * cap + 4 * r + (c - 54);
    return 58 * cap + r;
}
