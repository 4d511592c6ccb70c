// Peer-memory exchange for the tensor-parallel decode step: plain stores into the other GPUs'
// memory over NVLink and flags polled in local memory. No multimem, no TMA, nothing from NCCL.
//
// Every rank owns one region with the same layout, mapped into every other rank's address space:
//
//   header   step_no   bumped by the first kernel of every step on this rank
//            status    bit r set when a wait for rank r gave up
//            arrive    arrival counter of the push kernel (zero between launches)
//   flags    [sites][tp]   flags[s][r] = the step in which rank r last delivered site s
//   slots    [2][tp][slot_bytes]   what rank r delivered; the half used by (step, site) alternates
//
// A site is one exchange point of the step (after o_proj and after down_proj of every layer, and
// the arg-max candidates at the end: 2 L + 1 per step, an odd number, so consecutive exchanges
// always use different halves even across steps). An all-reduce is "everybody pushes its partial to
// everybody" followed by a consumer that waits for the tp flags of the site and adds the tp slots up
// in rank order in fp32 -- the same sum in the same order on every rank. The consumer is the kernel
// that needed the sum anyway (residual add + RMSNorm, fused into the next projection for small
// batches), so the reduction costs no launch of its own.
//
// Why a half cannot be overwritten early: rank B reaches exchange k + 2 only after consuming k + 1,
// for which every rank pushed k + 1, which each did after consuming k.
//
// Every wait is bounded: after kP2pSpinLimit polls the waiting thread records the peer in `status`
// and goes on (the step's result is then meaningless, but the kernel ends and the host can read why);
// once `status` is non-zero no later wait polls at all.
#pragma once
#include "kivi_common.cuh"

namespace kivi {

constexpr int kMaxTp = 8;
constexpr unsigned kP2pSpinLimit = 1u << 21;   // polls, each followed by a short sleep: of the order of a second

struct P2pHeader {
    unsigned step_no;
    unsigned status;
    unsigned arrive;
    unsigned pad;
};

struct P2pLayout {
    size_t flags_off, slots_off, slot_bytes, total;
    int sites, tp;
};

inline P2pLayout p2p_layout(int tp, int sites, size_t payload_bytes) {
    P2pLayout l;
    l.tp = tp;
    l.sites = sites;
    l.flags_off = 256;
    l.slots_off = l.flags_off + ((size_t)sites * tp * sizeof(unsigned) + 255) / 256 * 256;
    l.slot_bytes = (payload_bytes + 255) / 256 * 256;
    l.total = l.slots_off + 2 * (size_t)tp * l.slot_bytes;
    return l;
}

// Consumer side of one site, all pointers local.
struct P2pGather {
    const unsigned* flags;        // [tp] flags of this site
    const P2pHeader* header;
    unsigned* status;
    const unsigned char* slots;   // slots of half 0; half 1 follows at tp * slot_bytes
    size_t slot_bytes;
    int tp;                       // 0: no exchange, the consumer reads its plain local input
    int site;
    unsigned spin_limit;
};

// Producer side of one site: where this rank's slot and flag live in every peer's region.
struct P2pPush {
    unsigned char* slot[kMaxTp];  // peer r: its slots (half 0) + my_rank * slot_bytes
    unsigned* flag[kMaxTp];       // peer r: its flags[site][my_rank]
    const P2pHeader* header;      // local
    unsigned* arrive;             // local
    size_t half_stride;           // tp * slot_bytes
    int tp;
    int site;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_step_no(const P2pHeader* h) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&h->step_no) : "memory");
    return v;
}

// Which half of the slots exchange (step, site) uses.
__device__ __forceinline__ unsigned p2p_half(unsigned step_no, int site) { return (step_no + (unsigned)site) & 1u; }

// All threads of the CTA call this. Returns the slots of the site's half once every rank has
// delivered this step's data (or the poll limit ran out, recorded in status).
__device__ __forceinline__ const unsigned char* p2p_wait(const P2pGather& g) {
    const unsigned step_no = ld_step_no(g.header);
    // a wait that already gave up (this step or an earlier one) is not repeated: the error is sticky, so a
    // lost peer costs one poll budget, not one per kernel
    if ((int)threadIdx.x < g.tp && *reinterpret_cast<volatile unsigned*>(g.status) == 0u) {
        unsigned spins = 0;
        while ((int)(ld_acquire_sys(g.flags + threadIdx.x) - step_no) < 0) {
            if (++spins > g.spin_limit) {
                atomicOr(g.status, 1u << threadIdx.x);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    return g.slots + (size_t)p2p_half(step_no, g.site) * g.tp * g.slot_bytes;
}

// Sum over ranks of eight fp16 values at 16-byte index `vec` of every slot: fp32, rank order, one rounding.
__device__ __forceinline__ uint4 p2p_sum8(const unsigned char* slots, size_t slot_bytes, int tp, size_t vec) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    for (int r = 0; r < tp; ++r) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slots + (size_t)r * slot_bytes) + vec);
        const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += __half2float(h[k]);
    }
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) oh[k] = __float2half(acc[k]);
    return o;
}

// Host side (p2p.cu).
cudaError_t launch_p2p_push(const void* src, size_t bytes, const P2pPush& push, cudaStream_t stream);

}  // namespace kivi
