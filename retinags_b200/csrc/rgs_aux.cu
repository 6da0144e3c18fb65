// Small sm_100a kernels around the model: kNN scale initialiser, load histogram for the partition, frustum mask.
//   rgs_knn3_kernel        replaces simple_knn.distCUDA2 (absent submodule of the reference)
//   rgs_histogram_kernel   replaces the CPU numba scatter-add accum_on_3Dgrid (parallel_utils/grid_utils/utils.py:140-151)
//   rgs_mark_visible_kernel replaces checkFrustum / markVisible (cuda_rasterizer_hgs/rasterizer_impl.cu:54-66,141-153)
#include <cuda_runtime.h>
#include <stdint.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"
#include "rgs_knn.h"

__global__ void __launch_bounds__(128) rgs_knn3_kernel(const __grid_constant__ RgsKnnGrid g, const float* __restrict__ pts,
                                                       const int* __restrict__ cell_start, int64_t n, float* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = rgs_knn3(g, pts, cell_start, n, i);
}

__global__ void __launch_bounds__(256) rgs_histogram_kernel(const float* __restrict__ xyz, const float* __restrict__ weight,
                                                            int64_t n, float lo0, float lo1, float lo2, float v0, float v1,
                                                            float v2, int d0, int d1, int d2, float* __restrict__ grid) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int a = (int)floorf((xyz[3 * i] - lo0) / v0), b = (int)floorf((xyz[3 * i + 1] - lo1) / v1),
            c = (int)floorf((xyz[3 * i + 2] - lo2) / v2);
        a = min(max(a, 0), d0 - 1); b = min(max(b, 0), d1 - 1); c = min(max(c, 0), d2 - 1);
        atomicAdd(&grid[((int64_t)a * d1 + b) * d2 + c], weight ? weight[i] : 1.0f);
    }
}

__global__ void __launch_bounds__(256) rgs_mark_visible_kernel(const float* __restrict__ xyz, int64_t n,
                                                               const __grid_constant__ RgsCamera cam, uint8_t* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float p[3] = {xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2]};
        float t[3];
        rgs_view_point(cam.view, p, t);
        out[i] = t[2] > RGS_NEAR_Z ? 1 : 0;
    }
}

static inline unsigned aux_grid(int64_t n, int threads) {
    const int64_t want = (n + threads - 1) / threads;
    return (unsigned)(want < 1 ? 1 : (want > RGS_SMS * 32 ? RGS_SMS * 32 : want));
}

extern "C" {

int rgs_cuda_knn3(const RgsKnnGrid* g, const float* pts, const int32_t* cell_start, int64_t n, float* out, void* stream) {
    if (n <= 0) return 0;
    rgs_knn3_kernel<<<aux_grid(n, 128), 128, 0, (cudaStream_t)stream>>>(*g, pts, cell_start, n, out);
    return (int)cudaGetLastError();
}

int rgs_cuda_histogram(const float* xyz, const float* weight, int64_t n, const double* lo, const double* voxel,
                       const int64_t* dims, float* grid, void* stream) {
    if (n <= 0) return 0;
    rgs_histogram_kernel<<<aux_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(xyz, weight, n, (float)lo[0], (float)lo[1],
                                                                             (float)lo[2], (float)voxel[0], (float)voxel[1],
                                                                             (float)voxel[2], (int)dims[0], (int)dims[1],
                                                                             (int)dims[2], grid);
    return (int)cudaGetLastError();
}

int rgs_cuda_mark_visible(const float* xyz, int64_t n, const RgsCamera* cam, uint8_t* out, void* stream) {
    if (n <= 0) return 0;
    rgs_mark_visible_kernel<<<aux_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(xyz, n, *cam, out);
    return (int)cudaGetLastError();
}

}  // extern "C"
