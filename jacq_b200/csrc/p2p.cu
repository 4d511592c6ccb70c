// Peer-memory exchange of the tensor-parallel decode step: the push kernel and the region
// management entry points. Layout, protocol and the reasoning behind them are in p2p.cuh.
#include <cstring>

#include "p2p.cuh"

namespace kivi {
namespace {

constexpr int kPushThreads = 256;

// Copies `vecs` 16-byte vectors from local memory into this rank's slot in every peer's region
// (its own included), then the last CTA to finish publishes the step number in every peer's flag.
__global__ void __launch_bounds__(kPushThreads) p2p_push_kernel(const uint4* __restrict__ src, size_t vecs,
                                                                 const P2pPush push) {
    pdl_trigger();   // the projection that consumes this exchange may start streaming its weights now
    pdl_wait();      // the producer of `src` has finished
    const unsigned step_no = ld_step_no(push.header);
    const size_t half_off = (size_t)p2p_half(step_no, push.site) * push.half_stride;
    for (size_t v = (size_t)blockIdx.x * kPushThreads + threadIdx.x; v < vecs; v += (size_t)gridDim.x * kPushThreads) {
        const uint4 a = src[v];
        for (int r = 0; r < push.tp; ++r) reinterpret_cast<uint4*>(push.slot[r] + half_off)[v] = a;
    }
    __threadfence_system();   // this thread's stores are visible to every GPU before the CTA reports in
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(push.arrive, 1u);
        if (prev == gridDim.x - 1) {
            *push.arrive = 0u;           // ready for the next launch on this stream
            __threadfence_system();      // orders every CTA's stores (seen through the counter) before the flags
            for (int r = 0; r < push.tp; ++r) st_release_sys(push.flag[r], step_no);
        }
    }
}

}  // namespace

cudaError_t launch_p2p_push(const void* src, size_t bytes, const P2pPush& push, cudaStream_t stream) {
    const size_t vecs = (bytes + 15) / 16;
    int blocks = (int)((vecs + kPushThreads - 1) / kPushThreads);
    if (blocks < 1) blocks = 1;
    if (blocks > 64) blocks = 64;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(kPushThreads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, p2p_push_kernel, static_cast<const uint4*>(src), vecs, push);
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
