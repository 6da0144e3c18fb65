// Per-Gaussian and per-pixel math shared by the sm_100a kernels and the native CPU backend.
//
// Every function here is `__host__ __device__`: the CUDA kernels and the C++ CPU library call the
// very same code, so the numerics of the GPU path can be validated on a machine without a GPU.
//
// Behavioural parity targets in the reference (paths within MooreThreads/RetinaGS):
//   rasterization_kernels/diff-gaussian-rasterization-half-gaussian/cuda_rasterizer_hgs/forward.cu:20-258
//       (SH colour, EWA covariance, conic, radius, tile rectangle)
//   .../cuda_rasterizer_hgs/forward.cu:340-390   (alpha, half-Gaussian box clip, early stop)
//   .../cuda_rasterizer_hgs/backward.cu:20-412   (gradients of all of the above)
//   .../cuda_rasterizer_hgs/auxiliary.h:41-75,150-180 (ndc2Pix, pix2Ndc, getRect, near cull 0.2)
// The code is a fresh derivation in plain row-major algebra (no glm), not a transcription.
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define RGS_HD __host__ __device__ __forceinline__
#else
#define RGS_HD inline
#endif

#if defined(__CUDACC__)
#define RGS_UNROLL _Pragma("unroll")
#else
#define RGS_UNROLL
#endif

#define RGS_TILE 16
#define RGS_NEAR_Z 0.2f
#define RGS_ALPHA_MIN (1.0f / 255.0f)
#define RGS_ALPHA_MAX 0.99f
#define RGS_T_STOP 0.0001f

// The transmittance a finished render hands to the compositor carries "this pixel stopped at the RGS_T_STOP rule" in
// its lowest mantissa bit (a change of at most one unit in the last place). The compositing backward may use it to
// give nothing to the partials behind such a pixel, as a single render gives nothing to the splats behind it.
RGS_HD float rgs_mark_finished(float T, int finished) {
#ifdef __CUDA_ARCH__
    return __uint_as_float((__float_as_uint(T) & ~1u) | (finished ? 1u : 0u));
#else
    uint32_t u;
    memcpy(&u, &T, 4);
    u = (u & ~1u) | (finished ? 1u : 0u);
    memcpy(&T, &u, 4);
    return T;
#endif
}
RGS_HD int rgs_is_finished(float T) {
#ifdef __CUDA_ARCH__
    return (int)(__float_as_uint(T) & 1u);
#else
    uint32_t u;
    memcpy(&u, &T, 4);
    return (int)(u & 1u);
#endif
}
#define RGS_SH_COEFFS 16

// Camera + sub-model description handed by value to every kernel of one render task.
// Matrices use the 3DGS storage convention: the 4x4 is stored transposed, i.e. element
// m[4*j+i] multiplies input component j and feeds output component i.
struct RgsCamera {
    float view[16];   // world -> view
    float proj[16];   // world -> clip (view * projection)
    float c2w[16];    // view -> world
    float campos[3];
    float tan_fovx, tan_fovy;
    float focal_x, focal_y;
    int W, H;
    int tiles_x, tiles_y;
    float box_lo[3];  // half-open world box of the sub-model: lo < p <= hi
    float box_hi[3];
    float bg[3];
    int sh_degree;    // active SH degree (0..3)
    float scale_modifier;
    int raw_params;   // 1: inputs are raw (log-scale, logit opacity, unnormalised quaternion)
    int tight_rect;   // 1: shrink the tile rectangle to the alpha >= 1/255 extent (exact); 2: additionally drop every
                      //    tile of the rectangle that holds no contributing pixel (exact; depth-first binning only)
};

// Projected splat. 12 floats = three 16-byte vectors; this is the record the blend kernels stage
// into shared memory with bulk asynchronous copies.
struct __attribute__((aligned(16))) RgsSplat {
    float px, py;        // pixel-space mean
    float ca, cb, cc;    // conic (inverse 2D covariance): power = -.5(ca dx^2 + cc dy^2) - cb dx dy
    float opacity;
    float r, g, b;
    float w;             // clip-space w == view-space z (projection has P[3][2] = 1)
    float depth;         // view-space z
    float pmin;          // powers below this give alpha < 1/255: lets the blend loops skip the exponential
};

struct RgsRect { int x0, y0, x1, y1; };

static const float RGS_SH_C0 = 0.28209479177387814f;
static const float RGS_SH_C1 = 0.4886025119029199f;
#define RGS_SH_C2_0 1.0925484305920792f
#define RGS_SH_C2_1 -1.0925484305920792f
#define RGS_SH_C2_2 0.31539156525252005f
#define RGS_SH_C2_3 -1.0925484305920792f
#define RGS_SH_C2_4 0.5462742152960396f
#define RGS_SH_C3_0 -0.5900435899266435f
#define RGS_SH_C3_1 2.890611442640554f
#define RGS_SH_C3_2 -0.4570457994644658f
#define RGS_SH_C3_3 0.3731763325901154f
#define RGS_SH_C3_4 -0.4570457994644658f
#define RGS_SH_C3_5 1.445305721320277f
#define RGS_SH_C3_6 -0.5900435899266435f

RGS_HD float rgs_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
RGS_HD float rgs_ndc2pix(float v, int S) { return ((v + 1.0f) * S - 1.0f) * 0.5f; }
RGS_HD float rgs_pix2ndc(float p, int S) { return (2.0f * p + 1.0f) / S - 1.0f; }
RGS_HD int rgs_imin(int a, int b) { return a < b ? a : b; }
RGS_HD int rgs_imax(int a, int b) { return a > b ? a : b; }

// SH basis for a unit direction, degrees 0..3 (16 values; entries beyond `deg` are left at 0).
RGS_HD void rgs_sh_basis(int deg, float x, float y, float z, float* B) {
    for (int i = 0; i < 16; ++i) B[i] = 0.0f;
    B[0] = RGS_SH_C0;
    if (deg > 0) {
        B[1] = -RGS_SH_C1 * y; B[2] = RGS_SH_C1 * z; B[3] = -RGS_SH_C1 * x;
        if (deg > 1) {
            float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
            B[4] = RGS_SH_C2_0 * xy; B[5] = RGS_SH_C2_1 * yz;
            B[6] = RGS_SH_C2_2 * (2.0f * zz - xx - yy);
            B[7] = RGS_SH_C2_3 * xz; B[8] = RGS_SH_C2_4 * (xx - yy);
            if (deg > 2) {
                B[9] = RGS_SH_C3_0 * y * (3.0f * xx - yy);
                B[10] = RGS_SH_C3_1 * xy * z;
                B[11] = RGS_SH_C3_2 * y * (4.0f * zz - xx - yy);
                B[12] = RGS_SH_C3_3 * z * (2.0f * zz - 3.0f * xx - 3.0f * yy);
                B[13] = RGS_SH_C3_4 * x * (4.0f * zz - xx - yy);
                B[14] = RGS_SH_C3_5 * z * (xx - yy);
                B[15] = RGS_SH_C3_6 * x * (xx - 3.0f * yy);
            }
        }
    }
}

// d(basis)/d(x,y,z) for a unit direction (each 16 values).
RGS_HD void rgs_sh_basis_grad(int deg, float x, float y, float z, float* Bx, float* By, float* Bz) {
    for (int i = 0; i < 16; ++i) { Bx[i] = 0.0f; By[i] = 0.0f; Bz[i] = 0.0f; }
    if (deg > 0) {
        By[1] = -RGS_SH_C1; Bz[2] = RGS_SH_C1; Bx[3] = -RGS_SH_C1;
        if (deg > 1) {
            float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
            Bx[4] = RGS_SH_C2_0 * y; By[4] = RGS_SH_C2_0 * x;
            By[5] = RGS_SH_C2_1 * z; Bz[5] = RGS_SH_C2_1 * y;
            Bx[6] = RGS_SH_C2_2 * -2.0f * x; By[6] = RGS_SH_C2_2 * -2.0f * y; Bz[6] = RGS_SH_C2_2 * 4.0f * z;
            Bx[7] = RGS_SH_C2_3 * z; Bz[7] = RGS_SH_C2_3 * x;
            Bx[8] = RGS_SH_C2_4 * 2.0f * x; By[8] = RGS_SH_C2_4 * -2.0f * y;
            if (deg > 2) {
                Bx[9] = RGS_SH_C3_0 * 6.0f * xy; By[9] = RGS_SH_C3_0 * 3.0f * (xx - yy);
                Bx[10] = RGS_SH_C3_1 * yz; By[10] = RGS_SH_C3_1 * xz; Bz[10] = RGS_SH_C3_1 * xy;
                Bx[11] = RGS_SH_C3_2 * -2.0f * xy; By[11] = RGS_SH_C3_2 * (4.0f * zz - xx - 3.0f * yy);
                Bz[11] = RGS_SH_C3_2 * 8.0f * yz;
                Bx[12] = RGS_SH_C3_3 * -6.0f * xz; By[12] = RGS_SH_C3_3 * -6.0f * yz;
                Bz[12] = RGS_SH_C3_3 * 3.0f * (2.0f * zz - xx - yy);
                Bx[13] = RGS_SH_C3_4 * (4.0f * zz - 3.0f * xx - yy); By[13] = RGS_SH_C3_4 * -2.0f * xy;
                Bz[13] = RGS_SH_C3_4 * 8.0f * xz;
                Bx[14] = RGS_SH_C3_5 * 2.0f * xz; By[14] = RGS_SH_C3_5 * -2.0f * yz; Bz[14] = RGS_SH_C3_5 * (xx - yy);
                Bx[15] = RGS_SH_C3_6 * 3.0f * (xx - yy); By[15] = RGS_SH_C3_6 * -6.0f * xy;
            }
        }
    }
}

// Rotation matrix (row-major R[3*i+j]) of a quaternion (r,x,y,z); the quaternion is used as given.
RGS_HD void rgs_quat_to_rot(const float* q, float* R) {
    float r = q[0], x = q[1], y = q[2], z = q[3];
    R[0] = 1.f - 2.f * (y * y + z * z); R[1] = 2.f * (x * y - r * z); R[2] = 2.f * (x * z + r * y);
    R[3] = 2.f * (x * y + r * z); R[4] = 1.f - 2.f * (x * x + z * z); R[5] = 2.f * (y * z - r * x);
    R[6] = 2.f * (x * z - r * y); R[7] = 2.f * (y * z + r * x); R[8] = 1.f - 2.f * (x * x + y * y);
}

// Intermediates of the EWA projection that forward and backward share.
struct RgsEwa {
    float t[3];        // view-space mean
    float txc, tyc;    // clamped x,y used inside the Jacobian
    int clamp_x, clamp_y;
    float M[6];        // 2x3 = J * Wrot  (row-major)
    float Sigma[6];    // 3D covariance xx xy xz yy yz zz
    float a, b, c;     // 2D covariance after the 0.3 low-pass
    float det;
};

RGS_HD void rgs_view_point(const float* m, const float* p, float* t) {
    t[0] = m[0] * p[0] + m[4] * p[1] + m[8] * p[2] + m[12];
    t[1] = m[1] * p[0] + m[5] * p[1] + m[9] * p[2] + m[13];
    t[2] = m[2] * p[0] + m[6] * p[1] + m[10] * p[2] + m[14];
}

RGS_HD void rgs_ewa(const RgsCamera& cam, const float* p, const float* s, const float* q, RgsEwa& e) {
    rgs_view_point(cam.view, p, e.t);
    float tz = e.t[2];
    float limx = 1.3f * cam.tan_fovx, limy = 1.3f * cam.tan_fovy;
    float txtz = e.t[0] / tz, tytz = e.t[1] / tz;
    e.clamp_x = (txtz < -limx || txtz > limx);
    e.clamp_y = (tytz < -limy || tytz > limy);
    e.txc = fminf(limx, fmaxf(-limx, txtz)) * tz;
    e.tyc = fminf(limy, fmaxf(-limy, tytz)) * tz;
    float J00 = cam.focal_x / tz, J02 = -(cam.focal_x * e.txc) / (tz * tz);
    float J11 = cam.focal_y / tz, J12 = -(cam.focal_y * e.tyc) / (tz * tz);
    // Wrot[i][j] = view[4*j+i]
    const float* v = cam.view;
    for (int j = 0; j < 3; ++j) {
        e.M[j] = J00 * v[4 * j + 0] + J02 * v[4 * j + 2];
        e.M[3 + j] = J11 * v[4 * j + 1] + J12 * v[4 * j + 2];
    }
    float R[9];
    rgs_quat_to_rot(q, R);
    float sm = cam.scale_modifier;
    float L[9];  // L = R * diag(s)
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) L[3 * i + j] = R[3 * i + j] * (sm * s[j]);
    e.Sigma[0] = L[0] * L[0] + L[1] * L[1] + L[2] * L[2];
    e.Sigma[1] = L[0] * L[3] + L[1] * L[4] + L[2] * L[5];
    e.Sigma[2] = L[0] * L[6] + L[1] * L[7] + L[2] * L[8];
    e.Sigma[3] = L[3] * L[3] + L[4] * L[4] + L[5] * L[5];
    e.Sigma[4] = L[3] * L[6] + L[4] * L[7] + L[5] * L[8];
    e.Sigma[5] = L[6] * L[6] + L[7] * L[7] + L[8] * L[8];
    // N = M * Sigma (2x3), cov = N * M^T
    const float* S = e.Sigma;
    float N0 = e.M[0] * S[0] + e.M[1] * S[1] + e.M[2] * S[2];
    float N1 = e.M[0] * S[1] + e.M[1] * S[3] + e.M[2] * S[4];
    float N2 = e.M[0] * S[2] + e.M[1] * S[4] + e.M[2] * S[5];
    float N3 = e.M[3] * S[0] + e.M[4] * S[1] + e.M[5] * S[2];
    float N4 = e.M[3] * S[1] + e.M[4] * S[3] + e.M[5] * S[4];
    float N5 = e.M[3] * S[2] + e.M[4] * S[4] + e.M[5] * S[5];
    e.a = N0 * e.M[0] + N1 * e.M[1] + N2 * e.M[2] + 0.3f;
    e.b = N0 * e.M[3] + N1 * e.M[4] + N2 * e.M[5];
    e.c = N3 * e.M[3] + N4 * e.M[4] + N5 * e.M[5] + 0.3f;
    e.det = e.a * e.c - e.b * e.b;
}

// Activations of the raw optimisable parameters.
RGS_HD void rgs_activate(int raw, const float* s_in, const float* q_in, float o_in, float* s, float* q, float& o,
                         float& qnorm) {
    if (raw) {
        s[0] = expf(s_in[0]); s[1] = expf(s_in[1]); s[2] = expf(s_in[2]);
        qnorm = sqrtf(q_in[0] * q_in[0] + q_in[1] * q_in[1] + q_in[2] * q_in[2] + q_in[3] * q_in[3]);
        float inv = 1.0f / fmaxf(qnorm, 1e-12f);
        q[0] = q_in[0] * inv; q[1] = q_in[1] * inv; q[2] = q_in[2] * inv; q[3] = q_in[3] * inv;
        o = rgs_sigmoid(o_in);
    } else {
        s[0] = s_in[0]; s[1] = s_in[1]; s[2] = s_in[2];
        q[0] = q_in[0]; q[1] = q_in[1]; q[2] = q_in[2]; q[3] = q_in[3];
        o = o_in; qnorm = 1.0f;
    }
}

// The first 3*nc of the 48 SH coefficients of one Gaussian (`sh` is 16-byte aligned: rows of 192 bytes in a buffer
// whose column group starts on a 16-byte boundary). Device code fetches them as 128-bit words, 12 requests instead of
// 48, from global or shared memory alike.
RGS_HD void rgs_sh_load(const float* sh, int nc, float* out) {
#ifdef __CUDA_ARCH__
    const float4* v = reinterpret_cast<const float4*>(sh);
    RGS_UNROLL
    for (int j = 0; j < 12; ++j) {
        if (4 * j < 3 * nc) {
            const float4 q = v[j];
            out[4 * j] = q.x; out[4 * j + 1] = q.y; out[4 * j + 2] = q.z; out[4 * j + 3] = q.w;
        }
    }
#else
    for (int e = 0; e < 3 * nc; ++e) out[e] = sh[e];
#endif
}

// View-dependent colour of one Gaussian from its SH coefficients (16 RGB triples, coefficient-major): the colour part
// of the projection, also run on its own for the splats that turn out to have tile instances (rgs_colour_slab_kernel).
// `clamped` receives 3 bits (colour channel was clamped at 0).
RGS_HD void rgs_splat_colour(const RgsCamera& cam, const float* p, const float* sh, float& r, float& g, float& b,
                             unsigned& clamped) {
    float dx = p[0] - cam.campos[0], dy = p[1] - cam.campos[1], dz = p[2] - cam.campos[2];
    float inv = 1.0f / sqrtf(dx * dx + dy * dy + dz * dz);
    float B[16];
    rgs_sh_basis(cam.sh_degree, dx * inv, dy * inv, dz * inv, B);
    int nc = (cam.sh_degree + 1) * (cam.sh_degree + 1);
    float c0 = 0.5f, c1 = 0.5f, c2 = 0.5f;
    float shv[48];
    rgs_sh_load(sh, nc, shv);
    RGS_UNROLL
    for (int k = 0; k < 16; ++k)
        if (k < nc) { c0 += B[k] * shv[3 * k]; c1 += B[k] * shv[3 * k + 1]; c2 += B[k] * shv[3 * k + 2]; }
    clamped = (c0 < 0.0f ? 1u : 0u) | (c1 < 0.0f ? 2u : 0u) | (c2 < 0.0f ? 4u : 0u);
    r = fmaxf(c0, 0.0f); g = fmaxf(c1, 0.0f); b = fmaxf(c2, 0.0f);
}

// Forward projection of one Gaussian. Returns false when it is culled (near plane, singular
// covariance, empty tile rectangle). `sh` points at 16 RGB triples (coefficient-major); with a null `sh` the colour
// is left at zero for a later rgs_splat_colour (the geometry decides whether the splat is ever blended).
// `clamped` receives 3 bits (colour channel was clamped at 0), `radius` the 3-sigma pixel radius.
RGS_HD bool rgs_project(const RgsCamera& cam, const float* p, const float* s_in, const float* q_in, float o_in,
                        const float* sh, RgsSplat& out, RgsRect& rect, int& radius, unsigned& clamped) {
    radius = 0; clamped = 0;
    float t[3];
    rgs_view_point(cam.view, p, t);
    if (t[2] <= RGS_NEAR_Z) return false;
    float s[3], q[4], o, qn;
    rgs_activate(cam.raw_params, s_in, q_in, o_in, s, q, o, qn);
    RgsEwa e;
    rgs_ewa(cam, p, s, q, e);
    if (e.det == 0.0f) return false;
    float det_inv = 1.0f / e.det;
    float mid = 0.5f * (e.a + e.c);
    float sq = sqrtf(fmaxf(0.1f, mid * mid - e.det));
    float lambda1 = mid + sq, lambda2 = mid - sq;
    float rad = ceilf(3.0f * sqrtf(fmaxf(lambda1, lambda2)));
    const float* m = cam.proj;
    float hx = m[0] * p[0] + m[4] * p[1] + m[8] * p[2] + m[12];
    float hy = m[1] * p[0] + m[5] * p[1] + m[9] * p[2] + m[13];
    float hw = m[3] * p[0] + m[7] * p[1] + m[11] * p[2] + m[15];
    float pw = 1.0f / (hw + 0.0000001f);
    float px = rgs_ndc2pix(hx * pw, cam.W), py = rgs_ndc2pix(hy * pw, cam.H);
    int irad = (int)rad;
    rect.x0 = rgs_imin(cam.tiles_x, rgs_imax(0, (int)((px - irad) / RGS_TILE)));
    rect.y0 = rgs_imin(cam.tiles_y, rgs_imax(0, (int)((py - irad) / RGS_TILE)));
    rect.x1 = rgs_imin(cam.tiles_x, rgs_imax(0, (int)((px + irad + RGS_TILE - 1) / RGS_TILE)));
    rect.y1 = rgs_imin(cam.tiles_y, rgs_imax(0, (int)((py + irad + RGS_TILE - 1) / RGS_TILE)));
    if ((rect.x1 - rect.x0) * (rect.y1 - rect.y0) <= 0) return false;
    if (cam.tight_rect) {
        // alpha = o*exp(power) >= 1/255 needs d^T conic d <= 2 ln(255 o); the axis-aligned extent of
        // that ellipse is sqrt(2 ln(255 o) * cov_ii). Pixels outside contribute exactly nothing, so
        // dropping the tiles that hold only such pixels changes no output bit.
        float k = 2.0f * logf(255.0f * o);
        if (!(k > 0.0f)) return false;
        float ex = sqrtf(k * e.a) * 1.001f + 0.02f, ey = sqrtf(k * e.c) * 1.001f + 0.02f;
        int tx0 = (int)floorf((px - ex) / RGS_TILE), tx1 = (int)floorf((px + ex) / RGS_TILE) + 1;
        int ty0 = (int)floorf((py - ey) / RGS_TILE), ty1 = (int)floorf((py + ey) / RGS_TILE) + 1;
        rect.x0 = rgs_imax(rect.x0, tx0); rect.x1 = rgs_imin(rect.x1, tx1);
        rect.y0 = rgs_imax(rect.y0, ty0); rect.y1 = rgs_imin(rect.y1, ty1);
        if (rect.x1 <= rect.x0 || rect.y1 <= rect.y0) return false;
    }
    out.r = 0.0f; out.g = 0.0f; out.b = 0.0f;
    if (sh) rgs_splat_colour(cam, p, sh, out.r, out.g, out.b, clamped);
    out.px = px; out.py = py;
    out.ca = e.c * det_inv; out.cb = -e.b * det_inv; out.cc = e.a * det_inv;
    out.opacity = o;
    out.w = hw; out.depth = t[2];
    // alpha = o exp(power) < 1/255  <=>  power < -ln(255 o); slightly lowered so that the cheap test never rejects a
    // pair the exact test would keep
    out.pmin = -logf(255.0f * o) * 1.00001f - 0.00001f;
    radius = irad;
    return true;
}

// Exact tile culling. A splat contributes to a pixel only where alpha = o exp(-q/2) >= 1/255, i.e. where
// q(d) = ca dx^2 + 2 cb dx dy + cc dy^2 <= 2 ln(255 o). The minimum of the convex form q over the rectangle of
// pixel centres of a tile is 0 when the mean lies inside, else it is attained on one of the four edges (a 1-D
// quadratic each). A tile whose minimum exceeds the bound holds no contributing pixel and can be skipped without
// changing any output bit; a small margin absorbs rounding differences to the per-pixel evaluation.
RGS_HD float rgs_edge_min(float a, float b2, float c, float fixed, float lo, float hi) {
    // minimise a*fixed^2 + b2*fixed*t + c*t^2 over t in [lo, hi]
    float t = -0.5f * b2 * fixed / c;
    t = fminf(hi, fmaxf(lo, t));
    return a * fixed * fixed + b2 * fixed * t + c * t * t;
}

// Same test for an arbitrary rectangle of pixel centres [x0,x1] x [y0,y1].
RGS_HD bool rgs_rect_hit(float px, float py, float ca, float cb, float cc, float bound, float x0, float y0, float x1,
                         float y1) {
    // d = mean - pixel: ranges of dx, dy over the rectangle
    const float dx_lo = px - x1, dx_hi = px - x0, dy_lo = py - y1, dy_hi = py - y0;
    if (dx_lo <= 0.0f && dx_hi >= 0.0f && dy_lo <= 0.0f && dy_hi >= 0.0f) return true;
    const float b2 = 2.0f * cb;
    float m = rgs_edge_min(ca, b2, cc, dx_lo, dy_lo, dy_hi);
    m = fminf(m, rgs_edge_min(ca, b2, cc, dx_hi, dy_lo, dy_hi));
    m = fminf(m, rgs_edge_min(cc, b2, ca, dy_lo, dx_lo, dx_hi));
    m = fminf(m, rgs_edge_min(cc, b2, ca, dy_hi, dx_lo, dx_hi));
    return !(m > bound * 1.0005f + 0.001f);
}

RGS_HD bool rgs_tile_hit(float px, float py, float ca, float cb, float cc, float bound, int tx, int ty, int W, int H) {
    const float x0 = (float)(tx * RGS_TILE), y0 = (float)(ty * RGS_TILE);
    const float x1 = fminf(x0 + (RGS_TILE - 1), (float)(W - 1)), y1 = fminf(y0 + (RGS_TILE - 1), (float)(H - 1));
    return rgs_rect_hit(px, py, ca, cb, cc, bound, x0, y0, x1, y1);
}

RGS_HD float rgs_alpha_bound(float opacity) { return 2.0f * logf(255.0f * opacity); }

// Gradients of the image-space quantities of one splat, accumulated by the blend backward.
// 12 floats so that three 16-byte vector reductions update one record.
struct __attribute__((aligned(16))) RgsSplatGrad {
    float dpx, dpy;       // d/d(pixel-space mean)
    float dca, dcb, dcc;  // d/d(conic); dcb is the full derivative wrt the off-diagonal term
    float dopacity;
    float dr, dg, db;
    float ddepth;
    float pad0, pad1;
};

// Backward of rgs_project for one Gaussian. Adds into the parameter gradients
// (g_xyz[3], g_sh[48], g_scale[3], g_rot[4], g_opacity[1]); when cam.raw_params is set the
// gradients are with respect to the raw parameters. Returns the norm of the NDC-scaled screen
// gradient (the densification statistic).
// When `g_sh` is null the SH gradients are not accumulated; the caller can form them itself from the basis
// (`basis_out`, 16 values) and the clamped colour gradient (`gc_out`, 3 values): d/dsh[k][c] = basis[k] * gc[c].
RGS_HD float rgs_project_bwd(const RgsCamera& cam, const float* p, const float* s_in, const float* q_in, float o_in,
                             const float* sh, unsigned clamped, const RgsSplatGrad& g, float* g_xyz, float* g_sh,
                             float* g_scale, float* g_rot, float* g_opacity, float* basis_out = nullptr,
                             float* gc_out = nullptr) {
    float s[3], q[4], o, qn;
    rgs_activate(cam.raw_params, s_in, q_in, o_in, s, q, o, qn);
    RgsEwa e;
    rgs_ewa(cam, p, s, q, e);
    float gp[3] = {0.f, 0.f, 0.f};

    // ---- conic -> 2D covariance
    float a = e.a, b = e.b, c = e.c, det = e.det;
    float d2inv = 1.0f / (det * det + 0.0000001f);
    float dLa = d2inv * (-c * c * g.dca + b * c * g.dcb - b * b * g.dcc);
    float dLc = d2inv * (-b * b * g.dca + a * b * g.dcb - a * a * g.dcc);
    float dLb = d2inv * (2.f * b * c * g.dca - (det + 2.f * b * b) * g.dcb + 2.f * a * b * g.dcc);
    // symmetric 2x2 gradient G2 = [[dLa, dLb/2],[dLb/2, dLc]]
    float h = 0.5f * dLb;
    const float* M = e.M;
    // GS = M^T G2 M  (3x3 symmetric): gradient wrt the full matrix Sigma
    float GM0[3], GM1[3];  // rows of G2*M
    for (int j = 0; j < 3; ++j) { GM0[j] = dLa * M[j] + h * M[3 + j]; GM1[j] = h * M[j] + dLc * M[3 + j]; }
    float GS[9];
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) GS[3 * i + j] = M[i] * GM0[j] + M[3 + i] * GM1[j];
    // dL/dM = 2 * G2 * M * Sigma
    const float* S = e.Sigma;
    float Sf[9] = {S[0], S[1], S[2], S[1], S[3], S[4], S[2], S[4], S[5]};
    float dM[6];
    for (int j = 0; j < 3; ++j) {
        dM[j] = 2.f * (GM0[0] * Sf[j] + GM0[1] * Sf[3 + j] + GM0[2] * Sf[6 + j]);
        dM[3 + j] = 2.f * (GM1[0] * Sf[j] + GM1[1] * Sf[3 + j] + GM1[2] * Sf[6 + j]);
    }
    // M = J * Wrot, Wrot[i][j] = view[4j+i]  ->  dJ[r][i] = sum_j dM[r][j] * Wrot[i][j]
    const float* v = cam.view;
    float dJ00 = dM[0] * v[0] + dM[1] * v[4] + dM[2] * v[8];
    float dJ02 = dM[0] * v[2] + dM[1] * v[6] + dM[2] * v[10];
    float dJ11 = dM[3] * v[1] + dM[4] * v[5] + dM[5] * v[9];
    float dJ12 = dM[3] * v[2] + dM[4] * v[6] + dM[5] * v[10];
    float tz = e.t[2], tz2 = 1.0f / (tz * tz), tz3 = tz2 / tz;
    float dtx = e.clamp_x ? 0.0f : -cam.focal_x * tz2 * dJ02;
    float dty = e.clamp_y ? 0.0f : -cam.focal_y * tz2 * dJ12;
    float dtz = -cam.focal_x * tz2 * dJ00 - cam.focal_y * tz2 * dJ11 + 2.f * cam.focal_x * e.txc * tz3 * dJ02 +
                2.f * cam.focal_y * e.tyc * tz3 * dJ12;
    // t = Wrot p + trans; the splat's depth is t_z itself (gradient of the depth output, zero in training)
    dtz += g.ddepth;
    for (int j = 0; j < 3; ++j) gp[j] += v[4 * j + 0] * dtx + v[4 * j + 1] * dty + v[4 * j + 2] * dtz;

    // ---- Sigma = L L^T, L = R diag(s*mod)
    float R[9];
    rgs_quat_to_rot(q, R);
    float sm = cam.scale_modifier;
    float L[9];
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) L[3 * i + j] = R[3 * i + j] * (sm * s[j]);
    float dL[9];  // 2 * GS * L
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j)
            dL[3 * i + j] = 2.f * (GS[3 * i] * L[j] + GS[3 * i + 1] * L[3 + j] + GS[3 * i + 2] * L[6 + j]);
    float ds[3], dR[9];
    for (int j = 0; j < 3; ++j) {
        ds[j] = sm * (dL[j] * R[j] + dL[3 + j] * R[3 + j] + dL[6 + j] * R[6 + j]);
        for (int i = 0; i < 3; ++i) dR[3 * i + j] = dL[3 * i + j] * sm * s[j];
    }
    float r = q[0], x = q[1], y = q[2], z = q[3];
    float dq[4];
    dq[0] = 2.f * (-z * dR[1] + y * dR[2] + z * dR[3] - x * dR[5] - y * dR[6] + x * dR[7]);
    dq[1] = 2.f * (y * dR[1] + z * dR[2] + y * dR[3] - 2.f * x * dR[4] - r * dR[5] + z * dR[6] + r * dR[7] -
                   2.f * x * dR[8]);
    dq[2] = 2.f * (-2.f * y * dR[0] + x * dR[1] + r * dR[2] + x * dR[3] + z * dR[5] - r * dR[6] + z * dR[7] -
                   2.f * y * dR[8]);
    dq[3] = 2.f * (-2.f * z * dR[0] - r * dR[1] + x * dR[2] + r * dR[3] - 2.f * z * dR[4] + y * dR[5] + x * dR[6] +
                   y * dR[7]);
    if (cam.raw_params) {
        float dot = q[0] * dq[0] + q[1] * dq[1] + q[2] * dq[2] + q[3] * dq[3];
        float inv = 1.0f / fmaxf(qn, 1e-12f);
        for (int k = 0; k < 4; ++k) g_rot[k] += (dq[k] - q[k] * dot) * inv;
        for (int k = 0; k < 3; ++k) g_scale[k] += ds[k] * s[k];
        g_opacity[0] += g.dopacity * o * (1.0f - o);
    } else {
        for (int k = 0; k < 4; ++k) g_rot[k] += dq[k];
        for (int k = 0; k < 3; ++k) g_scale[k] += ds[k];
        g_opacity[0] += g.dopacity;
    }

    // ---- screen position
    const float* m = cam.proj;
    float hx = m[0] * p[0] + m[4] * p[1] + m[8] * p[2] + m[12];
    float hy = m[1] * p[0] + m[5] * p[1] + m[9] * p[2] + m[13];
    float hw = m[3] * p[0] + m[7] * p[1] + m[11] * p[2] + m[15];
    float pw = 1.0f / (hw + 0.0000001f);
    float gnx = g.dpx * 0.5f * cam.W, gny = g.dpy * 0.5f * cam.H;  // gradient wrt NDC x,y
    float mul1 = hx * pw * pw, mul2 = hy * pw * pw;
    for (int j = 0; j < 3; ++j)
        gp[j] += (m[4 * j + 0] * pw - m[4 * j + 3] * mul1) * gnx + (m[4 * j + 1] * pw - m[4 * j + 3] * mul2) * gny;

    // ---- colour
    float dxr = p[0] - cam.campos[0], dyr = p[1] - cam.campos[1], dzr = p[2] - cam.campos[2];
    float len2 = dxr * dxr + dyr * dyr + dzr * dzr;
    float inv = 1.0f / sqrtf(len2);
    float ux = dxr * inv, uy = dyr * inv, uz = dzr * inv;
    float gc0 = (clamped & 1u) ? 0.f : g.dr, gc1 = (clamped & 2u) ? 0.f : g.dg, gc2 = (clamped & 4u) ? 0.f : g.db;
    float B[16], Bx[16], By[16], Bz[16];
    rgs_sh_basis(cam.sh_degree, ux, uy, uz, B);
    rgs_sh_basis_grad(cam.sh_degree, ux, uy, uz, Bx, By, Bz);
    int nc = (cam.sh_degree + 1) * (cam.sh_degree + 1);
    float gux = 0.f, guy = 0.f, guz = 0.f;
    if (gc_out) { gc_out[0] = gc0; gc_out[1] = gc1; gc_out[2] = gc2; }
    RGS_UNROLL
    for (int k = 0; k < 16; ++k) {
        if (basis_out) basis_out[k] = k < nc ? B[k] : 0.0f;
        if (k >= nc) continue;
        if (g_sh) { g_sh[3 * k] += B[k] * gc0; g_sh[3 * k + 1] += B[k] * gc1; g_sh[3 * k + 2] += B[k] * gc2; }
        float wsum = sh[3 * k] * gc0 + sh[3 * k + 1] * gc1 + sh[3 * k + 2] * gc2;
        gux += Bx[k] * wsum; guy += By[k] * wsum; guz += Bz[k] * wsum;
    }
    // through the normalisation u = d/|d|
    float dotu = ux * gux + uy * guy + uz * guz;
    gp[0] += (gux - ux * dotu) * inv; gp[1] += (guy - uy * dotu) * inv; gp[2] += (guz - uz * dotu) * inv;

    g_xyz[0] += gp[0]; g_xyz[1] += gp[1]; g_xyz[2] += gp[2];
    return sqrtf(gnx * gnx + gny * gny);
}

// ------------------------------------------------------------------------------------------
// Per-pixel blending
// ------------------------------------------------------------------------------------------

// Per-pixel constants: the world-space ray through the pixel centre, scaled to unit view depth,
// so that the sample point at clip w is campos' + (w + 1e-7) * dirxy + w * dirz (see below).
struct RgsPixelRay {
    float ax[3];  // world increment per unit of (w + 1e-7): c2w columns 0,1 weighted by the pixel's NDC*tan
    float az[3];  // world increment per unit of w: c2w column 2
    float o[3];   // c2w translation
};

RGS_HD void rgs_pixel_ray(const RgsCamera& cam, float pixx, float pixy, RgsPixelRay& ray) {
    float nx = rgs_pix2ndc(pixx, cam.W) * cam.tan_fovx, ny = rgs_pix2ndc(pixy, cam.H) * cam.tan_fovy;
    const float* m = cam.c2w;
    for (int i = 0; i < 3; ++i) {
        ray.ax[i] = m[i] * nx + m[4 + i] * ny;
        ray.az[i] = m[8 + i];
        ray.o[i] = m[12 + i];
    }
}

// Half-Gaussian clip: the point of the pixel ray at the splat's centre depth must lie in the
// sub-model's half-open box. Both neighbours of a shared face evaluate the identical float
// expression, so exactly one of them keeps the (pixel, splat) pair.
RGS_HD bool rgs_in_box(const RgsCamera& cam, const RgsPixelRay& ray, float w) {
    float we = w + 0.0000001f;
    for (int i = 0; i < 3; ++i) {
        float pw = fmaf(we, ray.ax[i], fmaf(w, ray.az[i], ray.o[i]));
        if (pw <= cam.box_lo[i] || pw > cam.box_hi[i]) return false;
    }
    return true;
}

struct RgsPixelState {
    float T;
    float C[3];
    float D;
    int contributor;   // splats visited so far
    int last;          // index (1-based) of the last splat that contributed
    int done;
};

RGS_HD void rgs_pixel_init(RgsPixelState& st) {
    st.T = 1.0f; st.C[0] = st.C[1] = st.C[2] = 0.0f; st.D = 0.0f; st.contributor = 0; st.last = 0; st.done = 0;
}

// Evaluate alpha of a splat at a pixel; returns false when the pair is skipped.
RGS_HD bool rgs_alpha(const RgsCamera& cam, const RgsPixelRay& ray, float pixx, float pixy, const RgsSplat& sp,
                      float& alpha, float& G, float& dx, float& dy) {
    dx = sp.px - pixx; dy = sp.py - pixy;
    float power = -0.5f * (sp.ca * dx * dx + sp.cc * dy * dy) - sp.cb * dx * dy;
    if (power > 0.0f || power < sp.pmin) return false;
    G = expf(power);
    alpha = fminf(RGS_ALPHA_MAX, sp.opacity * G);
    if (alpha < RGS_ALPHA_MIN) return false;
    return rgs_in_box(cam, ray, sp.w);
}

RGS_HD void rgs_blend_fwd_step(const RgsCamera& cam, const RgsPixelRay& ray, float pixx, float pixy,
                               const RgsSplat& sp, RgsPixelState& st) {
    st.contributor++;
    float alpha, G, dx, dy;
    if (!rgs_alpha(cam, ray, pixx, pixy, sp, alpha, G, dx, dy)) return;
    float test_T = st.T * (1.0f - alpha);
    if (test_T < RGS_T_STOP) { st.done = 1; return; }
    float wgt = alpha * st.T;
    st.C[0] += sp.r * wgt; st.C[1] += sp.g * wgt; st.C[2] += sp.b * wgt;
    st.D += sp.depth * wgt;
    st.T = test_T;
    st.last = st.contributor;
}

// Backward state of a pixel while the splats are replayed back to front.
struct RgsPixelBwd {
    float T;            // running transmittance in front of the current splat
    float T_final;
    float acc[3];       // colour accumulated behind the current splat
    float last_alpha;
    float last_c[3];
    float gC[3];        // dL/dC of this pixel
    float gT;           // dL/dT_final of this pixel (the background term is folded in by the caller)
};

RGS_HD void rgs_pixel_bwd_init(RgsPixelBwd& st, float T_final, const float* gC, float gT) {
    st.T = T_final; st.T_final = T_final;
    st.acc[0] = st.acc[1] = st.acc[2] = 0.0f;
    st.last_alpha = 0.0f; st.last_c[0] = st.last_c[1] = st.last_c[2] = 0.0f;
    st.gC[0] = gC[0]; st.gC[1] = gC[1]; st.gC[2] = gC[2]; st.gT = gT;
}

// Extra backward state of a pixel when the depth output D = sum depth_i alpha_i T_i carries a gradient
// (the reference's dL/ddepth path, cuda_rasterizer_hgs/backward.cu:391-403,584). Training never sets it.
struct RgsPixelBwdDepth {
    float acc;      // depth accumulated behind the current splat
    float last_d;   // depth of the splat visited before (the one behind)
    float gD;       // dL/dD of this pixel
};

// One (pixel, splat) step of the backward. Returns false when the pair did not contribute;
// otherwise fills `g` with this pixel's contribution to the splat's image-space gradients.
// `dep` (optional): also propagate the gradient of the depth output.
RGS_HD bool rgs_blend_bwd_step(const RgsCamera& cam, const RgsPixelRay& ray, float pixx, float pixy,
                               const RgsSplat& sp, RgsPixelBwd& st, RgsSplatGrad& g,
                               RgsPixelBwdDepth* dep = nullptr) {
    float alpha, G, dx, dy;
    if (!rgs_alpha(cam, ray, pixx, pixy, sp, alpha, G, dx, dy)) return false;
    st.T = st.T / (1.0f - alpha);
    float wgt = alpha * st.T;
    float dL_dalpha = 0.0f;
    const float col[3] = {sp.r, sp.g, sp.b};
    float* gcol = &g.dr;
    for (int ch = 0; ch < 3; ++ch) {
        st.acc[ch] = st.last_alpha * st.last_c[ch] + (1.0f - st.last_alpha) * st.acc[ch];
        st.last_c[ch] = col[ch];
        dL_dalpha += (col[ch] - st.acc[ch]) * st.gC[ch];
        gcol[ch] = wgt * st.gC[ch];
    }
    float g_depth = 0.0f;
    if (dep) {  // same recurrence as a colour channel, with the splat's view depth as its "colour"
        dep->acc = st.last_alpha * dep->last_d + (1.0f - st.last_alpha) * dep->acc;
        dep->last_d = sp.depth;
        dL_dalpha += (sp.depth - dep->acc) * dep->gD;
        g_depth = wgt * dep->gD;
    }
    dL_dalpha *= st.T;
    st.last_alpha = alpha;
    // T_final = prod(1 - alpha_i): d T_final / d alpha = -T_final / (1 - alpha)
    dL_dalpha += (-st.T_final / (1.0f - alpha)) * st.gT;
    float dL_dG = sp.opacity * dL_dalpha;
    float gdx = G * dx, gdy = G * dy;
    float dG_ddx = -gdx * sp.ca - gdy * sp.cb;
    float dG_ddy = -gdy * sp.cc - gdx * sp.cb;
    g.dpx = dL_dG * dG_ddx; g.dpy = dL_dG * dG_ddy;
    g.dca = -0.5f * gdx * dx * dL_dG;
    g.dcb = -gdx * dy * dL_dG;
    g.dcc = -0.5f * gdy * dy * dL_dG;
    g.dopacity = G * dL_dalpha;
    g.ddepth = g_depth; g.pad0 = 0.0f; g.pad1 = 0.0f;
    return true;
}

// ------------------------------------------------------------------------------------------
// Adam over the parameter block
// ------------------------------------------------------------------------------------------
RGS_HD void rgs_adam_elem(float& p, float g, float& m, float& v, float lr, float beta1, float beta2, float eps,
                          float inv_bc1, float inv_bc2_sqrt) {
    // torch.optim.Adam: m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ;
    // p -= lr / bc1 * m / (sqrt(v)/sqrt(bc2) + eps); the two bias corrections arrive as reciprocals.
    // Every product and sum is rounded on its own: left to the compiler, a*b + c*d is contracted into a fused
    // multiply-add around either product, and the choice differs between the kernels this function is inlined
    // into (and from the host build), so that two work distributions of the same update disagreed in the last bit.
#ifdef __CUDA_ARCH__
    m = __fadd_rn(__fmul_rn(beta1, m), __fmul_rn(1.0f - beta1, g));
    v = __fadd_rn(__fmul_rn(beta2, v), __fmul_rn(__fmul_rn(1.0f - beta2, g), g));
    const float denom = __fadd_rn(__fmul_rn(__fsqrt_rn(v), inv_bc2_sqrt), eps);
    p = __fsub_rn(p, __fmul_rn(__fmul_rn(lr, inv_bc1), __fdiv_rn(m, denom)));
#else
    const float a = beta1 * m, b = (1.0f - beta1) * g;
    m = a + b;
    const float c = beta2 * v, d = ((1.0f - beta2) * g) * g;
    v = c + d;
    const float e = sqrtf(v) * inv_bc2_sqrt;
    const float denom = e + eps;
    const float step = (lr * inv_bc1) * (m / denom);
    p = p - step;
#endif
}
