// SSIM statistics pass with the horizontal 11-tap Gaussian filter on the 5th-generation tensor cores.
//
// The five windowed moments of SSIM (mu1, mu2, E[x^2], E[y^2], E[xy]) are separable filters. The horizontal
// pass over a tile of 128 rows x 64 output columns is the banded GEMM
//     D[128 x 64] = A[128 x 80] * B^T,   B[n][k] = w[k - n - 3]  (0 <= k-n-3 <= 10, else 0)
// where A holds 80 input columns starting 8 left of the tile (a 16-byte aligned TMA x coordinate; out-of-image
// columns and rows arrive as zeros, which is exactly the zero padding SSIM uses).  Data flow per CTA:
//   TMA (cp.async.bulk.tensor.2d, no multicast) -> raw image / target tiles in shared memory
//   threads form each moment, split it into two TF32 terms (hi + lo) and lay it out as a K-major UMMA operand
//   tcgen05.mma.kind::tf32 (one elected thread): D += A_hi B_hi + A_lo B_hi + A_hi B_lo   (3xTF32: fp32-class result)
//   accumulators live in TMEM (5 moments x 64 columns), read back with tcgen05.ld
//   vertical pass, SSIM map, derivative maps and loss sums on the CUDA cores, as in rgs_loss.cu.
// Every mbarrier wait is bounded; on expiry the CTA records a status word, frees its TMEM and returns.
// Reference: utils/loss_utils.py:43-63 (five cuDNN depthwise convolutions).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"
#include "rgs_loss_math.h"

#define TC_M 128          // input rows per tile (118 output rows + 10 halo)
#define TC_N 64           // output columns per tile
#define TC_K 80           // input columns per tile
#define TC_OUT_ROWS (TC_M - 10)
#define TC_XSHIFT 8       // tile starts 8 columns left of its first output column (TMA needs 16-byte aligned x)
#define TC_WAIT_LIMIT (1u << 24)

// shared memory map (bytes)
#define SM_RAW_X 0                                   // [128][80] fp32
#define SM_RAW_Y (SM_RAW_X + TC_M * TC_K * 4)        // [128][80] fp32
#define SM_A_HI (SM_RAW_Y + TC_M * TC_K * 4)         // canonical K-major, 128 x 80
#define SM_A_LO (SM_A_HI + TC_M * TC_K * 4)
#define SM_B_HI (SM_A_LO + TC_M * TC_K * 4)          // canonical K-major, 64 x 80
#define SM_B_LO (SM_B_HI + TC_N * TC_K * 4)
#define SM_BARS (SM_B_LO + TC_N * TC_K * 4)          // 2 mbarriers + tmem address word
#define SM_TOTAL (SM_BARS + 64)
#define SM_HBUF 0                                    // [5][128][64] fp32 overlays raw + A buffers after the MMAs

static_assert(5 * TC_M * TC_N * 4 <= SM_B_HI, "H buffer must fit below the B operands");

// canonical no-swizzle K-major layout: 8x(16 byte) core matrices, K-adjacent core matrices `groups*128` bytes apart
__device__ __forceinline__ uint32_t canon_off(int row, int k, int groups) {
    return (uint32_t)(((k >> 2) * groups + (row >> 3)) * 128 + (row & 7) * 16 + (k & 3) * 4);
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);         // start address
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;    // leading (K) byte offset
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;    // stride (M/N) byte offset
    d |= (uint64_t)1 << 46;                               // descriptor version of sm_100
    return d;                                             // layout type 0: no swizzle
}

__device__ __forceinline__ uint32_t tf32_round(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

__global__ void __launch_bounds__(128, 1) rgs_ssim_tc_kernel(const __grid_constant__ CUtensorMap map_img,
                                                             const __grid_constant__ CUtensorMap map_gt,
                                                             const float* __restrict__ img, const float* __restrict__ gt,
                                                             int H, int W, int crow0, int crow1, int srow0, int srow1,
                                                             float* __restrict__ dmaps, double* __restrict__ sums,
                                                             uint32_t* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned long long* bar_tma = reinterpret_cast<unsigned long long*>(smem + SM_BARS);
    unsigned long long* bar_mma = bar_tma + 1;
    uint32_t* tmem_word = reinterpret_cast<uint32_t*>(smem + SM_BARS + 16);
    const int c = blockIdx.z;
    const int col0 = blockIdx.x * TC_N;                    // first output column
    const int orow0 = crow0 + blockIdx.y * TC_OUT_ROWS;    // first output row
    const int in_row0 = orow0 - 5, in_col0 = col0 - TC_XSHIFT;

    if (tid == 0) { rgs_mbar_init(bar_tma, 1); rgs_mbar_init(bar_mma, 1); rgs_fence_mbar_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(rgs_smem_addr(tmem_word)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // band matrices (hi/lo TF32 split of the window)
    {
        float gw[11];
        rgs_gauss_window(gw);
        for (int e = tid; e < TC_N * TC_K; e += 128) {
            const int n = e / TC_K, k = e % TC_K;
            const int j = k - n - (TC_XSHIFT - 5);
            const float w = (j >= 0 && j <= 10) ? gw[j] : 0.f;
            const uint32_t hi = tf32_round(w);
            const uint32_t lo = tf32_round(w - __uint_as_float(hi));
            const uint32_t off = canon_off(n, k, TC_N / 8);
            *reinterpret_cast<uint32_t*>(smem + SM_B_HI + off) = hi;
            *reinterpret_cast<uint32_t*>(smem + SM_B_LO + off) = lo;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_word;

    bool failed = false;
    if (tid == 0) {
        rgs_mbar_expect_tx(bar_tma, 2u * TC_M * TC_K * 4u);
        // 3-D tensor (x, y, channel); x is a multiple of 4 floats (16 bytes) by construction
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
                     "r"(rgs_smem_addr(smem + SM_RAW_X)), "l"(&map_img), "r"(in_col0), "r"(in_row0), "r"(c), "r"(rgs_smem_addr(bar_tma)) : "memory");
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
                     "r"(rgs_smem_addr(smem + SM_RAW_Y)), "l"(&map_gt), "r"(in_col0), "r"(in_row0), "r"(c), "r"(rgs_smem_addr(bar_tma)) : "memory");
    }
    if (!rgs_mbar_wait(bar_tma, 0, TC_WAIT_LIMIT)) failed = true;

    // instruction descriptor: D=f32, A=B=tf32, both K-major, N=64, M=128
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TC_N >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
    const float* rawx = reinterpret_cast<const float*>(smem + SM_RAW_X);
    const float* rawy = reinterpret_cast<const float*>(smem + SM_RAW_Y);
    for (int q = 0; q < 5 && !failed; ++q) {
        // moment q of every input pixel, split into two TF32 terms, in operand layout
        for (int e = tid; e < TC_M * TC_K; e += 128) {
            const int m = e / TC_K, k = e % TC_K;
            const float x = rawx[e], y = rawy[e];
            const float v = q == 0 ? x : (q == 1 ? y : (q == 2 ? x * x : (q == 3 ? y * y : x * y)));
            const uint32_t hi = tf32_round(v);
            const uint32_t lo = tf32_round(v - __uint_as_float(hi));
            const uint32_t off = canon_off(m, k, TC_M / 8);
            *reinterpret_cast<uint32_t*>(smem + SM_A_HI + off) = hi;
            *reinterpret_cast<uint32_t*>(smem + SM_A_LO + off) = lo;
        }
        rgs_fence_proxy_async();  // generic-proxy writes -> visible to the tensor-core (async) proxy
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = rgs_smem_addr(smem + SM_A_HI), a_lo = rgs_smem_addr(smem + SM_A_LO);
            const uint32_t b_hi = rgs_smem_addr(smem + SM_B_HI), b_lo = rgs_smem_addr(smem + SM_B_LO);
            const uint32_t lbo_a = (TC_M / 8) * 128, lbo_b = (TC_N / 8) * 128;
            const uint32_t d_addr = tmem_base + (uint32_t)(q * TC_N);
            uint32_t acc = 0;
            for (int ks = 0; ks < TC_K / 8; ++ks) {
                const uint32_t ao = (uint32_t)ks * 2u * lbo_a, bo = (uint32_t)ks * 2u * lbo_b;
                const uint64_t dah = umma_desc(a_hi + ao, lbo_a, 128), dal = umma_desc(a_lo + ao, lbo_a, 128);
                const uint64_t dbh = umma_desc(b_hi + bo, lbo_b, 128), dbl = umma_desc(b_lo + bo, lbo_b, 128);
                const uint64_t pa[3] = {dah, dal, dah};
                const uint64_t pb[3] = {dbh, dbh, dbl};
#pragma unroll
                for (int t = 0; t < 3; ++t) {
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(d_addr), "l"(pa[t]), "l"(pb[t]), "r"(idesc), "r"(acc) : "memory");
                    acc = 1;
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(rgs_smem_addr(bar_mma)) : "memory");
        }
        // the operand buffers may only be overwritten once the tensor core has consumed them
        if (!rgs_mbar_wait(bar_mma, (uint32_t)(q & 1), TC_WAIT_LIMIT)) failed = true;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    failed = __syncthreads_or(failed);

    float* hbuf = reinterpret_cast<float*>(smem + SM_HBUF);
    if (!failed) {
        // TMEM -> registers -> shared: warp w owns lanes (= tile rows) 32w..32w+31
        for (int q = 0; q < 5; ++q) {
            for (int c0 = 0; c0 < TC_N; c0 += 16) {
                uint32_t r[16];
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(q * TC_N + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float* dst = hbuf + ((size_t)q * TC_M + (warp * 32 + lane)) * TC_N + c0;
#pragma unroll
                for (int j = 0; j < 16; ++j) dst[j] = __uint_as_float(r[j]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
    if (failed) {
        if (tid == 0) atomicExch(status, 3u);
        return;
    }
    // vertical pass + SSIM on the CUDA cores: thread t handles column t & 63, rows (t >> 6), +2, ...
    float gw[11];
    rgs_gauss_window(gw);
    float l1 = 0.f, ss = 0.f, l2 = 0.f;
    const size_t plane = (size_t)3 * H * W;
    for (int e = tid; e < TC_OUT_ROWS * TC_N; e += 128) {
        const int r = e / TC_N, q = e % TC_N;
        const int y = orow0 + r, x = col0 + q;
        if (y >= crow1 || y >= H || x >= W) continue;
        float m[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < 11; ++k) {
            const float w = gw[k];
#pragma unroll
            for (int j = 0; j < 5; ++j) m[j] += w * hbuf[((size_t)j * TC_M + r + k) * TC_N + q];
        }
        float d[3];
        const float s = rgs_ssim_pixel(m[0], m[1], m[2], m[3], m[4], d);
        const size_t pid = (size_t)c * H * W + (size_t)y * W + x;
        dmaps[pid] = d[0]; dmaps[plane + pid] = d[1]; dmaps[2 * plane + pid] = d[2];
        if (y >= srow0 && y < srow1) {
            const float diff = img[pid] - gt[pid];
            l1 += fabsf(diff); ss += s; l2 += diff * diff;
        }
    }
    __shared__ float red[3][4];
#pragma unroll
    for (int dlt = 16; dlt > 0; dlt >>= 1) {
        l1 += __shfl_xor_sync(0xffffffffu, l1, dlt);
        ss += __shfl_xor_sync(0xffffffffu, ss, dlt);
        l2 += __shfl_xor_sync(0xffffffffu, l2, dlt);
    }
    if (lane == 0) { red[0][warp] = l1; red[1][warp] = ss; red[2][warp] = l2; }
    __syncthreads();
    if (tid < 3) {
        double t = 0;
        for (int w = 0; w < 4; ++w) t += (double)red[tid][w];
        atomicAdd(&sums[tid], t);
    }
}

// ---------------------------------------------------------------------------------------------
// host: tensor maps through the driver entry point (the library links against the runtime only)
// ---------------------------------------------------------------------------------------------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode() {
    static PFN_encodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(p);
    }
    return fn;
}

static int make_map(CUtensorMap* map, const float* base, int H, int W) {
    PFN_encodeTiled enc = get_encode();
    if (!enc) return 20;
    const cuuint64_t dims[3] = {(cuuint64_t)W, (cuuint64_t)H, 3};
    const cuuint64_t strides[2] = {(cuuint64_t)W * 4, (cuuint64_t)W * H * 4};
    const cuuint32_t box[3] = {TC_K, TC_M, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 21;
}

extern "C" {

// 1 when the tensor-core path can serve an image of this shape (row pitch must be a multiple of 16 bytes).
int rgs_cuda_ssim_tc_supported(int64_t H, int64_t W) { return (W % 4 == 0 && W >= TC_K && H >= 16 && get_encode() != nullptr) ? 1 : 0; }

// Same contract as rgs_cuda_ssim_fwd; `status` receives 3 when a bounded wait expired.
int rgs_cuda_ssim_fwd_tc(const float* img, const float* gt, int64_t H, int64_t W, int64_t crow0, int64_t crow1,
                         int64_t srow0, int64_t srow1, float* dmaps, double* sums, int32_t* status, void* stream) {
    if (crow1 <= crow0) return 0;
    if (W % 4 != 0 || (reinterpret_cast<uintptr_t>(img) & 15) || (reinterpret_cast<uintptr_t>(gt) & 15)) return 22;
    CUtensorMap mi, mg;
    int rc = make_map(&mi, img, (int)H, (int)W);
    if (rc) return rc;
    rc = make_map(&mg, gt, (int)H, (int)W);
    if (rc) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        RGS_CUDA_CHECK(cudaFuncSetAttribute(rgs_ssim_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL));
        attr_set = true;
    }
    dim3 grid((unsigned)((W + TC_N - 1) / TC_N), (unsigned)((crow1 - crow0 + TC_OUT_ROWS - 1) / TC_OUT_ROWS), 3);
    rgs_ssim_tc_kernel<<<grid, 128, SM_TOTAL, (cudaStream_t)stream>>>(mi, mg, img, gt, (int)H, (int)W, (int)crow0, (int)crow1,
                                                                      (int)srow0, (int)srow1, dmaps, sums,
                                                                      reinterpret_cast<uint32_t*>(status));
    return (int)cudaGetLastError();
}

}  // extern "C"
