// Peer-to-peer plumbing of the fused compositing path: CUDA IPC allocation/mapping of the
// per-rank exchange region and the flag kernels that order producers and consumers across GPUs.
//
// The reference moves partial images and their gradients with NCCL send/recv batches followed by
// a device-wide synchronise (parallel_utils/communicate_utils/core.py:37-65). Here the bytes are
// stored by the producing kernels themselves (rgs_raster.cu: blend epilogue; rgs_loss.cu:
// compositing backward) through peer-mapped pointers over NVLink; what remains is ordering:
//   signal: after its producing kernels, a rank release-stores an epoch number into its word of
//           every peer's flag array (system scope);
//   wait:   before its consuming kernels, a rank acquire-loads its own flag array until every
//           word has reached the epoch. The wait is bounded by a cycle budget; on expiry it writes
//           a status word that the host checks, and returns normally.
// Plain peer stores/loads only: no multimem, no multicast, no TMA on peer memory.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include "rgs_api.h"
#include "rgs_cuda_common.cuh"

// Layout of a rank's flag array (RGS_P2P_FLAG_WORDS 32-bit words): [0,32) the epoch word of every rank,
// [32,64) and [64,96) two banks of one payload word per rank. A signal of epoch e stores the sender's payload into
// bank e & 1 before it releases the epoch word; a peer is never more than one signal ahead of a waiting rank, so the
// bank a wait reads is not overwritten under it. The payload carries the sender's "this step overflowed" word: every
// rank leaves the wait with the OR over all ranks and drops the optimiser update together.
#define RGS_P2P_MAX_WORLD 32
#define RGS_P2P_FLAG_WORDS 96
#define RGS_MAX_PARTIALS_MAPS 64  // most sub-models in front of one (the compositing kernels handle as many partials)

struct RgsPeerFlagPtrs { uint32_t* p[RGS_P2P_MAX_WORLD]; };

__global__ void rgs_p2p_signal_kernel(const __grid_constant__ RgsPeerFlagPtrs flags, int world, int my_rank,
                                      uint32_t epoch, const uint32_t* __restrict__ payload_src) {
    const int o = threadIdx.x;
    if (o < world) {
        if (payload_src) flags.p[o][RGS_P2P_MAX_WORLD * (1 + (epoch & 1u)) + my_rank] = *payload_src;
        __threadfence_system();
        rgs_st_release_sys(flags.p[o] + my_rank, epoch);
    }
}

__global__ void rgs_p2p_wait_kernel(const uint32_t* __restrict__ my_flags, int world, uint32_t epoch,
                                    long long budget_cycles, uint32_t* __restrict__ status,
                                    uint32_t* __restrict__ payload_out) {
    const int r = threadIdx.x;
    if (r >= world) return;
    const long long t0 = clock64();
    bool arrived = true;
    while (true) {
        const uint32_t v = rgs_ld_acquire_sys(my_flags + r);
        if ((int32_t)(v - epoch) >= 0) break;
        if (clock64() - t0 > budget_cycles) {
            atomicExch(status, 0x100u | (uint32_t)r);  // gave up waiting for rank r
            arrived = false;
            break;
        }
        __nanosleep(200);
    }
    if (arrived && payload_out) {
        const uint32_t pv = *reinterpret_cast<const volatile uint32_t*>(my_flags + RGS_P2P_MAX_WORLD * (1 + (epoch & 1u)) + r);
        if (pv) atomicOr(payload_out, pv);
    }
    __threadfence_system();
}

// Per-tile "finished" maps (one byte per tile) that sub-models publish so that sub-models behind them skip hidden
// tiles. rgs_tile_maps_or: dst |= OR of n source maps (local memory; remote maps were pushed here first).
// rgs_tile_map_push: one local map is stored into the map slots of up to RGS_P2P_MAX_WORLD ranks (plain peer stores).
struct RgsMapPtrs { const uint8_t* p[RGS_MAX_PARTIALS_MAPS]; };
struct RgsMapDsts { uint8_t* p[RGS_P2P_MAX_WORLD]; };

__global__ void rgs_tile_maps_or_kernel(const __grid_constant__ RgsMapPtrs srcs, int n, uint8_t* __restrict__ dst,
                                        int nbytes, int overwrite) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += gridDim.x * blockDim.x) {
        uint8_t v = overwrite ? 0 : dst[i];
        for (int k = 0; k < n; ++k) v |= srcs.p[k][i];
        dst[i] = v ? 1 : 0;
    }
}

__global__ void rgs_tile_map_push_kernel(const uint8_t* __restrict__ src, const __grid_constant__ RgsMapDsts dsts,
                                         int nbytes) {
    uint8_t* dst = dsts.p[blockIdx.y];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

extern "C" {

int rgs_cuda_tile_maps_or(const uint8_t* const* srcs, int64_t n, uint8_t* dst, int64_t nbytes, int64_t overwrite,
                          void* stream) {
    if (n < 0 || n > RGS_MAX_PARTIALS_MAPS || nbytes < 0 || nbytes > 0x7fffffffll) return 14;
    if (nbytes == 0 || (n == 0 && !overwrite)) return 0;
    RgsMapPtrs s;
    for (int k = 0; k < n; ++k) s.p[k] = srcs[k];
    const unsigned blocks = (unsigned)((nbytes + 255) / 256 > 64 ? 64 : (nbytes + 255) / 256);
    rgs_tile_maps_or_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(s, (int)n, dst, (int)nbytes, (int)overwrite);
    return (int)cudaGetLastError();
}

int rgs_cuda_tile_map_push(const uint8_t* src, uint8_t* const* dsts, int64_t n_dst, int64_t nbytes, void* stream) {
    if (n_dst < 0 || n_dst > RGS_P2P_MAX_WORLD || nbytes < 0 || nbytes > 0x7fffffffll) return 14;
    if (n_dst == 0 || nbytes == 0) return 0;
    RgsMapDsts d;
    for (int k = 0; k < n_dst; ++k) d.p[k] = dsts[k];
    dim3 grid((unsigned)((nbytes + 255) / 256 > 16 ? 16 : (nbytes + 255) / 256), (unsigned)n_dst);
    rgs_tile_map_push_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(src, d, (int)nbytes);
    return (int)cudaGetLastError();
}

int rgs_cuda_ipc_alloc(int64_t bytes, void** out) {
    void* p = nullptr;
    RGS_CUDA_CHECK(cudaMalloc(&p, (size_t)bytes));
    RGS_CUDA_CHECK(cudaMemset(p, 0, (size_t)bytes));
    RGS_CUDA_CHECK(cudaDeviceSynchronize());
    *out = p;
    return 0;
}

int rgs_cuda_ipc_free(void* p) { return (int)cudaFree(p); }

int rgs_cuda_ipc_get_handle(void* p, char* out64) {
    cudaIpcMemHandle_t h;
    RGS_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
    static_assert(sizeof(h) == 64, "handle size");
    memcpy(out64, &h, 64);
    return 0;
}

int rgs_cuda_ipc_open(const char* in64, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, in64, 64);
    void* p = nullptr;
    RGS_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *out = p;
    return 0;
}

int rgs_cuda_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// flag_ptrs: `world` device pointers (host array): the flag array of every rank as mapped here. payload_src
// (optional, device): one word that travels with the signal (see the layout above).
int rgs_cuda_p2p_signal(uint32_t* const* flag_ptrs, int64_t world, int64_t my_rank, int64_t epoch,
                        const uint32_t* payload_src, void* stream) {
    if (world < 1 || world > RGS_P2P_MAX_WORLD) return 14;
    RgsPeerFlagPtrs f;
    for (int i = 0; i < world; ++i) f.p[i] = flag_ptrs[i];
    rgs_p2p_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, (int)world, (int)my_rank, (uint32_t)epoch, payload_src);
    return (int)cudaGetLastError();
}

// payload_out (optional, device): receives the OR of the payload words of all ranks whose signal arrived.
int rgs_cuda_p2p_wait(const uint32_t* my_flags, int64_t world, int64_t epoch, int64_t budget_cycles, int32_t* status,
                      uint32_t* payload_out, void* stream) {
    if (world < 1 || world > RGS_P2P_MAX_WORLD) return 14;
    rgs_p2p_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(my_flags, (int)world, (uint32_t)epoch,
                                                           (long long)budget_cycles,
                                                           reinterpret_cast<uint32_t*>(status), payload_out);
    return (int)cudaGetLastError();
}

int64_t rgs_cuda_p2p_flag_bytes() { return RGS_P2P_FLAG_WORDS * 4; }
int64_t rgs_cuda_p2p_max_world() { return RGS_P2P_MAX_WORLD; }

}  // extern "C"
