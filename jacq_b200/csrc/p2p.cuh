// Peer-memory exchange for the tensor-parallel decode step: plain stores into the other GPUs'
// memory over NVLink, polled in local memory. No multimem, no TMA, nothing from NCCL.
//
// Every rank owns one region with the same layout, mapped into every other rank's address space:
//
//   header   step_no   bumped by the first kernel of every step on this rank
//            status    bit r set when a wait for rank r gave up
//   slots    [2][tp][slot_bytes]   what rank r delivered; the half used by an exchange alternates
//
// The payload travels as 8-byte words {32 bits of data, 32-bit sequence number}, each written with
// one store, so a word is either entirely old or entirely new and the data needs no separate flag,
// fence or arrival count: the reader polls the word itself until it carries the sequence number
// of the current exchange (the "LL" idea of collective libraries). The sequence number is
// step_no * sites + site + 1, unique per exchange.
//
// A site is one exchange point of the step (after o_proj and after down_proj of every layer, and
// the arg-max candidates at the end: 2 L + 1 per step, an odd number, so consecutive exchanges
// always use different halves even across steps). An all-reduce is "everybody writes its partial to
// everybody" -- from the epilogue of the projection that produced it when the batch is small, from
// a copy kernel otherwise -- followed by a consumer that reads the tp slots and adds them up in rank
// order in fp32: the same sum in the same order on every rank. The consumer is the kernel that
// needed the sum anyway (residual add + RMSNorm, fused into the next projection for small batches),
// so the reduction costs no launch of its own.
//
// Why a half cannot be overwritten early: rank B reaches exchange k + 2 only after consuming k + 1,
// for which every rank wrote k + 1, which each did after consuming k.
//
// Every wait is bounded: after spin_limit polls of one word the reader records the peer in
// `status` and goes on with whatever the word holds (the step's result is then meaningless, but the
// kernel ends and the host can read why); once `status` is non-zero no later read polls at all.
#pragma once
#include "kivi_common.cuh"

namespace kivi {

constexpr int kMaxTp = 8;
constexpr unsigned kP2pSpinLimit = 1u << 21;   // polls of one word, each followed by a short sleep: about a second

struct P2pHeader {
    unsigned step_no;
    unsigned status;
    unsigned pad[2];
};

struct P2pLayout {
    size_t slots_off, slot_bytes, total;
    int sites, tp;
};

// payload_bytes: the largest payload one rank delivers at a site; a slot holds it as 8-byte words.
inline P2pLayout p2p_layout(int tp, int sites, size_t payload_bytes) {
    P2pLayout l;
    l.tp = tp;
    l.sites = sites;
    l.slots_off = 256;
    l.slot_bytes = (2 * ((payload_bytes + 3) / 4 * 4) + 255) / 256 * 256;
    l.total = l.slots_off + 2 * (size_t)tp * l.slot_bytes;
    return l;
}

// Consumer side of one site, all pointers local.
struct P2pGather {
    const P2pHeader* header;
    unsigned* status;
    const unsigned char* slots;   // slots of half 0; half 1 follows at tp * slot_bytes
    size_t slot_bytes;
    int tp;                       // 0: no exchange, the consumer reads its plain local input
    int site, sites;
    unsigned spin_limit;
};

// Producer side of one site: this rank's slot (half 0) in every peer's region.
struct P2pPush {
    unsigned char* slot[kMaxTp];
    const P2pHeader* header;      // local
    size_t half_stride;           // tp * slot_bytes
    int tp;                       // 0: nothing to deliver
    int site, sites;
};

__device__ __forceinline__ unsigned ld_step_no(const P2pHeader* h) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&h->step_no) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile8(void* p, unsigned data, unsigned seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(seq) : "memory");
}
__device__ __forceinline__ void st_volatile16(void* p, unsigned d0, unsigned d1, unsigned seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%2};" ::"l"(p), "r"(d0), "r"(seq), "r"(d1) : "memory");
}

// Sequence number and half of exchange (step, site).
__device__ __forceinline__ unsigned p2p_seq(unsigned step_no, int site, int sites) {
    return step_no * (unsigned)sites + (unsigned)site + 1u;
}
__device__ __forceinline__ unsigned p2p_half(unsigned step_no, int site) { return (step_no + (unsigned)site) & 1u; }

// What a reader needs after looking the exchange up once.
struct P2pView {
    const unsigned char* slots;   // slots of the exchange's half
    size_t slot_bytes;
    unsigned seq;
    unsigned spin_limit;          // 0 once a wait has failed: read without polling
    unsigned* status;
    int tp;
};

__device__ __forceinline__ P2pView p2p_view(const P2pGather& g) {
    const unsigned step_no = ld_step_no(g.header);
    P2pView v;
    v.slots = g.slots + (size_t)p2p_half(step_no, g.site) * g.tp * g.slot_bytes;
    v.slot_bytes = g.slot_bytes;
    v.seq = p2p_seq(step_no, g.site, g.sites);
    v.spin_limit = *reinterpret_cast<volatile unsigned*>(g.status) == 0u ? g.spin_limit : 0u;
    v.status = g.status;
    v.tp = g.tp;
    return v;
}

// Data words 2 i and 2 i + 1 of rank r's payload (one 16-byte load of two 8-byte words). `w` is a first look at
// them, possibly from before they arrived: polled again until both carry the exchange's sequence number.
__device__ __forceinline__ uint2 p2p_settle2(P2pView& v, int r, const unsigned char* p, uint4 w) {
    unsigned spins = 0;
    while ((w.y != v.seq || w.w != v.seq) && spins < v.spin_limit) {
        __nanosleep(40);
        w = ld_volatile16(p);
        ++spins;
    }
    if (w.y != v.seq || w.w != v.seq) {
        if (v.spin_limit) atomicOr(v.status, 1u << r);
        v.spin_limit = 0u;   // this thread does not poll again
    }
    return make_uint2(w.x, w.z);
}
__device__ __forceinline__ uint2 p2p_read2(P2pView& v, int r, size_t i) {
    const unsigned char* p = v.slots + (size_t)r * v.slot_bytes + i * 16;
    return p2p_settle2(v, r, p, ld_volatile16(p));
}

// Sum over ranks of eight fp16 values (data words 4 vec .. 4 vec + 3 of every payload): fp32, rank
// order, one rounding. The loads of two ranks go out together before any of them is looked at: a load
// that bypasses the L1 takes the better part of a microsecond, and one after the other (two per rank) they were
// most of what an exchange cost -- 20 round trips per thread on four ranks, 40 on eight. (Four ranks together made
// the projection kernels, which call this from their prologue with weights already prefetched into registers, spill.)
template <int kTogether = 2>   // ranks whose words are requested together (two 16-byte loads, 8 registers, each)
__device__ __forceinline__ uint4 p2p_sum8(P2pView& v, size_t vec) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    const unsigned char* base = v.slots + vec * 32;
    for (int r0 = 0; r0 < v.tp; r0 += kTogether) {
        uint4 first[kTogether][2];
#pragma unroll
        for (int k = 0; k < kTogether; ++k)
            if (r0 + k < v.tp) {
                const unsigned char* p = base + (size_t)(r0 + k) * v.slot_bytes;
                first[k][0] = ld_volatile16(p);
                first[k][1] = ld_volatile16(p + 16);
            }
#pragma unroll
        for (int k = 0; k < kTogether; ++k)
            if (r0 + k < v.tp) {
                const unsigned char* p = base + (size_t)(r0 + k) * v.slot_bytes;
                const uint2 a = p2p_settle2(v, r0 + k, p, first[k][0]), b = p2p_settle2(v, r0 + k, p + 16, first[k][1]);
                const unsigned w[4] = {a.x, a.y, b.x, b.y};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                    acc[2 * e] += f.x;
                    acc[2 * e + 1] += f.y;
                }
            }
    }
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) oh[k] = __float2half(acc[k]);
    return o;
}

// Producer: where data word i of this exchange goes in peer r's region, and the number it carries.
struct P2pTarget {
    unsigned seq;
    size_t half_off;
};
__device__ __forceinline__ P2pTarget p2p_target(const P2pPush& push) {
    const unsigned step_no = ld_step_no(push.header);
    P2pTarget t;
    t.seq = p2p_seq(step_no, push.site, push.sites);
    t.half_off = (size_t)p2p_half(step_no, push.site) * push.half_stride;
    return t;
}
__device__ __forceinline__ void p2p_write1(const P2pPush& push, const P2pTarget& t, size_t i, unsigned data) {
    for (int r = 0; r < push.tp; ++r) st_volatile8(push.slot[r] + t.half_off + i * 8, data, t.seq);
}
__device__ __forceinline__ void p2p_write2(const P2pPush& push, const P2pTarget& t, size_t pair, unsigned d0, unsigned d1) {
    for (int r = 0; r < push.tp; ++r) st_volatile16(push.slot[r] + t.half_off + pair * 16, d0, d1, t.seq);
}

// Host side (p2p.cu): copy kernel for payloads that no projection epilogue delivers itself.
cudaError_t launch_p2p_push(const void* src, size_t bytes, const P2pPush& push, cudaStream_t stream);

}  // namespace kivi
