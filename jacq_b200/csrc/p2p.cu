// Peer-memory exchange of the tensor-parallel decode step: the push kernel and the region
// management entry points. Layout, protocol and the reasoning behind them are in p2p.cuh.
#include <cstring>

#include "p2p.cuh"

namespace kivi {
namespace {

constexpr int kPushThreads = 256;

// Delivers `pairs` pairs of 32-bit payload words from local memory into this rank's slot in every
// peer's region (its own included), each pair as one 16-byte store of two {data, sequence} words.
__global__ void __launch_bounds__(kPushThreads) p2p_push_kernel(const uint2* __restrict__ src, size_t pairs,
                                                                 const P2pPush push) {
    const P2pTarget t = p2p_target(push);
    for (size_t i = (size_t)blockIdx.x * kPushThreads + threadIdx.x; i < pairs; i += (size_t)gridDim.x * kPushThreads) {
        const uint2 a = src[i];
        p2p_write2(push, t, i, a.x, a.y);
    }
}

}  // namespace

// bytes is rounded up to whole pairs of words; src must be readable that far and 8-byte aligned.
cudaError_t launch_p2p_push(const void* src, size_t bytes, const P2pPush& push, cudaStream_t stream) {
    const size_t pairs = (bytes + 7) / 8;
    int blocks = (int)((pairs + kPushThreads - 1) / kPushThreads);
    if (blocks < 1) blocks = 1;
    if (blocks > 296) blocks = 296;
    p2p_push_kernel<<<blocks, kPushThreads, 0, stream>>>(static_cast<const uint2*>(src), pairs, push);
    return cudaGetLastError();
}

}  // namespace kivi

using namespace kivi;

extern "C" int kivi_b200_p2p_region_create(size_t bytes, void** region, unsigned char* handle_out) {
    if (!region || !handle_out) return KIVI_ERR_NULL_POINTER;
    if (bytes == 0) return KIVI_ERR_RANGE;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return KIVI_ERR_CUDA;
    if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return KIVI_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return KIVI_ERR_CUDA; }
    static_assert(sizeof(h) == KIVI_B200_P2P_HANDLE_BYTES, "IPC handle size");
    memcpy(handle_out, &h, sizeof(h));
    *region = p;
    return KIVI_OK;
}

extern "C" int kivi_b200_p2p_region_open(const unsigned char* handle, void** peer_region) {
    if (!handle || !peer_region) return KIVI_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return KIVI_ERR_CUDA;
    *peer_region = p;
    return KIVI_OK;
}

extern "C" int kivi_b200_p2p_region_close(void* peer_region) {
    if (!peer_region) return KIVI_ERR_NULL_POINTER;
    return cudaIpcCloseMemHandle(peer_region) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

extern "C" int kivi_b200_p2p_region_destroy(void* region) {
    if (!region) return KIVI_ERR_NULL_POINTER;
    return cudaFree(region) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

extern "C" int kivi_b200_p2p_status(const void* region, uint32_t* status_out, cudaStream_t stream) {
    if (!region || !status_out) return KIVI_ERR_NULL_POINTER;
    const P2pHeader* h = static_cast<const P2pHeader*>(region);
    if (cudaMemcpyAsync(status_out, &h->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
        return KIVI_ERR_CUDA;
    return cudaStreamSynchronize(stream) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}
