// int4-KIVI cache writer for B200.
//
// What it computes is the reference's writer (hand-CUDA form,
// integrations/vllm_kivi/source_patch.py:1532-1697, asserted equal to the DSL form
// crates/jac-codegen-cuda/src/variants.rs:2936-3067): append new K/V rows to the fp16 residual
// scratch; whenever R+G rows are present, quantise the oldest G rows (keys per channel over the
// G tokens, values per token over each channel group; asymmetric int4, scale = (max-min)/15,
// zero = min, codes from the unrounded fp32 scale/zero) into the pages the block table names, and
// move the remaining rows to the front.
//
// How it is laid out differs: the reference launches 1-thread blocks with strided 2-byte loads and
// a serial row-by-row shift, one sequence and at most one age-out per call. Here one launch covers
// every sequence of the batch and every group a chunk ages out:
//   pack kernel    one CTA per (sequence, kv head, keys | values, run of aged-out groups): the G x D tile of a group
//                  arrives by 16-byte asynchronous copies in a shared-memory tile (the next group's while the
//                  current one is packed) and is packed from registers; min/max are reduced in parallel
//                  (min/max are order-independent, so the result is bit-identical to the serial scan) and
//                  codes leave as 32-bit words, 8 channels each, fully coalesced. The CTA of a tensor's first
//                  run also moves and appends that tensor's scratch rows (the rows that stay come in through
//                  the same tile while the last group is packed). Run-time geometries stage the tile in shared
//                  memory and leave the scratch to a second kernel;
//   scratch kernel one CTA per (sequence, kv head): overlapping move-to-front through registers
//                  with a barrier per step, then the append of the rows that stay unquantised.
// A token at absolute position p comes from scratch row p - old_tokens when it predates the call,
// else from the new rows; that indirection is what lets one call cross several boundaries and
// still equal the token-by-token writer.
#include "kivi_common.cuh"
#include "step_math.cuh"

#include <type_traits>

namespace kivi {
namespace {

constexpr int kThreads = 256;

// Geometry as seen by the writer kernels: compile-time for the shapes the decode kernel's fast
// path covers (index arithmetic becomes shifts and masks), run-time for everything else.
template <int D_, int G_, int B_>
struct StaticShape {
    __device__ __forceinline__ explicit StaticShape(const Geom&) {}
    static constexpr int d = D_, g = G_, b = B_;
    static constexpr int vg = G_ < D_ ? G_ : D_, hg = D_ / vg, pages_per_group = G_ / B_;
    // The register-tile form of the pack (pack_group_regs below) covers every shape of this kind.
    static constexpr bool in_registers = true;
};
struct DynamicShape {
    __device__ __forceinline__ explicit DynamicShape(const Geom& x)
        : d(x.d), g(x.g), b(x.b), vg(x.vg), hg(x.hg), pages_per_group(x.pages_per_group) {}
    const int d, g, b, vg, hg, pages_per_group;
    static constexpr bool in_registers = false;
};

// Sequences whose write was refused because a slot or page id lay outside the pools (since the library was loaded).
__device__ unsigned int g_writer_rejected;

struct SeqWrite {
    int start, num_new, end, prev_old, next_old, new_row0, slot;
    const int* bt;
};

__device__ __forceinline__ SeqWrite seq_write(const WriteParams& p, int i) {
    SeqWrite s;
    s.start = seq_len_of(p.seq, i);
    if (s.start < 0) s.start = 0;
    if (p.new_offsets) {
        s.new_row0 = p.new_offsets[i];
        s.num_new = p.new_offsets[i + 1] - s.new_row0;
    } else {
        s.new_row0 = i * p.num_new_scalar;
        s.num_new = p.num_new_scalar;
    }
    if (s.num_new < 0) s.num_new = 0;
    s.end = s.start + s.num_new;
    s.prev_old = split_old(s.start, p.geom.r, p.geom.g);
    s.next_old = split_old(s.end, p.geom.r, p.geom.g);
    s.slot = slot_of(p.seq, i);
    s.bt = p.seq.block_tables + (size_t)i * p.seq.bt_stride;
    // Ids from device memory become addresses: the slot and every page this write packs into must lie in the
    // pools. A sequence that fails is left untouched by all of its CTAs (they all see the same ids) and counted.
    // The threads of the CTA share the page ids between them (every thread of the CTA calls this function).
    bool ok = index_in_pool(s.slot, p.cache.num_slots);
    const int page0 = s.prev_old / p.geom.b, page1 = s.next_old / p.geom.b;
    for (int lp = page0 + (int)threadIdx.x; lp < page1; lp += (int)blockDim.x)
        ok = ok && lp < p.seq.bt_width && index_in_pool(s.bt[lp], p.cache.num_blocks);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && s.num_new > 0) atomicAdd(&g_writer_rejected, 1u);
        s.num_new = 0; s.end = s.start; s.next_old = s.prev_old; s.slot = 0;
    }
    return s;
}

// Source row of absolute token `pos` for kv head h: old scratch or new rows.
__device__ __forceinline__ const __half* token_row(const WriteParams& p, const SeqWrite& s, const __half* scratch,
                                                   const __half* fresh, int h, int pos) {
    const Geom& g = p.geom;
    if (pos < s.start)
        return scratch + (((size_t)s.slot * g.nkv + h) * g.scratch_rows + (pos - s.prev_old)) * g.d;
    return fresh + ((size_t)(s.new_row0 + pos - s.start) * g.nkv + h) * g.d;
}

// clamp_code of the reference (source_patch.py:1517-1522). __float2int_rn rounds to nearest even
// like rintf, saturates, and maps NaN to 0.
__device__ __forceinline__ unsigned clamp_code(float q) {
    int c = __float2int_rn(q);
    c = c < 0 ? 0 : c;
    return (unsigned)(c > 15 ? 15 : c);
}

// The code of one element. The reference computes clamp(rintf((x - mn) / scale), 0, 15) with an
// IEEE division: code_exact. Fast form, bit-identical whenever mn and scale are finite:
//   * quotient from the correctly rounded reciprocal rcp = 1/scale (computed once per scale):
//     q0 = a*rcp, r = a - scale*q0 (exact in an FMA), q = q0 + r*rcp is the correctly rounded
//     quotient (Markstein);
//   * 0 <= q <= 15 then holds by construction (mn <= x <= mx, scale = (mx-mn)/15), so no clamp;
//   * q + 1.5*2^23 leaves rint(q), ties to even, in the low mantissa bits: the bits are 0x4B400000 + code.
//     A NaN element would give NaN + magic = NaN; where NaN elements can reach the fast form (the staged
//     pack) NaN is squashed to 0 first (fmaxf with 0), as the reference's conversion does.
__device__ __forceinline__ unsigned code_exact(float x, float mn, float scale) {
    return clamp_code(__fdiv_rn(__fsub_rn(x, mn), scale));
}

// The fast form, two elements at a time with the packed fp32 instructions of sm_100 (add / mul / fma .f32x2:
// two independent IEEE round-to-nearest operations per instruction). Returns the raw bits of both
// q + magic values.
__device__ __forceinline__ unsigned long long f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint2 code_bits_fast2(float x0, float x1, unsigned long long neg_mn, unsigned long long neg_scale,
                                                 unsigned long long rcp) {
    unsigned long long a, q, r;
    const unsigned long long x = f32x2(x0, x1);
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(a) : "l"(x), "l"(neg_mn));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q) : "l"(a), "l"(rcp));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(neg_scale), "l"(q), "l"(a));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(r), "l"(rcp), "l"(q));
    float q0, q1;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(q0), "=f"(q1) : "l"(q));
    q0 = fmaxf(q0, 0.0f);   // NaN -> 0
    q1 = fmaxf(q1, 0.0f);
    const unsigned long long magic = f32x2(12582912.0f, 12582912.0f);
    unsigned long long m;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(m) : "l"(f32x2(q0, q1)), "l"(magic));
    uint2 bits;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(bits.x), "=r"(bits.y) : "l"(m));
    return bits;
}

template <class Shape>
__device__ __forceinline__ void stage_tile(const Shape& g, const WriteParams& p, const SeqWrite& s,
                                           const __half* scratch, const __half* fresh, int h, int pos0, __half* tile) {
    const int chunks_per_row = g.d / 8;
    const int total = g.g * chunks_per_row;
    for (int c = threadIdx.x; c < total; c += kThreads) {
        int t = c / chunks_per_row, w = c - t * chunks_per_row;
        const uint4* src = reinterpret_cast<const uint4*>(token_row(p, s, scratch, fresh, h, pos0 + t));
        cp_async16(reinterpret_cast<uint4*>(tile) + c, src + w);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Pack 8 channels of one token (16 bytes of fp16) into one 32-bit word of codes. `exact` selects
// the plain IEEE division for tiles that hold an Inf/NaN scale or zero-point.
__device__ __forceinline__ unsigned pack_word(const uint4& v, const float* mn, const float* sc, const float* rc,
                                              bool exact) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float x[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        x[2 * e] = f.x;
        x[2 * e + 1] = f.y;
    }
    unsigned word = 0;
    if (!exact) {
        // Horner over the nibbles: every term is 0x4B400000 + code
#pragma unroll
        for (int e = 6; e >= 0; e -= 2) {
            const uint2 b = code_bits_fast2(x[e], x[e + 1], f32x2(-mn[e], -mn[e + 1]), f32x2(-sc[e], -sc[e + 1]),
                                            f32x2(rc[e], rc[e + 1]));
            word = (word * 16u + b.y) * 16u + b.x;
        }
        word -= 0x4B400000u * 0x11111111u;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) word |= code_exact(x[e], mn[e], sc[e]) << (4 * e);
    }
    return word;
}

// ---------------------------------------------------------------------------------------------
// Register-tile pack (compile-time shapes). Thread (w, r) = (tid % WPR, tid / WPR), WPR = D / 8 words per row,
// owns the 16-byte word w of rows r, r + RPP, r + 2 RPP, ... (RPP = 256 / WPR rows per pass) -- sixteen (or
// eight) neighbouring lanes cover one row, so the copies are whole 128/256-byte rows. The words arrive by
// asynchronous copies in a shared-memory tile that only their owner reads back, and stay in registers
// for both passes over the data. Minima and maxima are taken on the fp16 values themselves, two per
// instruction (min/max return one of their inputs, so nothing is rounded and the result equals the
// reference's fp32 scan; -0 orders below +0 exactly as fminf/fmaxf do). The first pass uses the
// NaN-propagating forms: a NaN anywhere shows in the extremes, and so does an infinity. Tiles whose
// extremes are all finite -- nearly all -- are packed with the reciprocal form, which then needs no NaN
// handling per element; the others repeat the pass with the NaN-skipping forms the reference's scan amounts to
// and are packed with the plain IEEE division.

struct PackPairs {   // parameters of eight channels as f32x2 operands
    unsigned long long neg_mn[4], neg_sc[4], rcp[4];
};

// KIVI_PACK_MIXED_ADD: 1 forms x - zero with the mixed-precision add of sm_100 (fp16 element + fp32 operand, the fp16
// side widened exactly, one IEEE rounding: the same bits as convert-then-add), 0 converts first and adds in pairs.
#ifndef KIVI_PACK_MIXED_ADD
#define KIVI_PACK_MIXED_ADD 1
#endif

__device__ __forceinline__ unsigned pack_word_pairs(const uint4& v, const PackPairs& pp) {
    const unsigned long long magic = f32x2(12582912.0f, 12582912.0f);
    // Every rounded quotient comes out as the bits 0x4B400000 + code. Two of them fold into a byte (b0 + 16 b1: the
    // low byte is exact, what the constants add lies above it), and byte permutes gather the four bytes: seven
    // independent integer instructions per eight codes.
    unsigned bytes[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        unsigned long long a, q, r, m;
#if KIVI_PACK_MIXED_ADD
        const unsigned hw = reinterpret_cast<const unsigned*>(&v)[e];
        unsigned short h0, h1;
        float z0, z1, a0, a1;
        asm("mov.b32 {%0, %1}, %2;" : "=h"(h0), "=h"(h1) : "r"(hw));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(z0), "=f"(z1) : "l"(pp.neg_mn[e]));
        asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(a0) : "h"(h0), "f"(z0));
        asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(a1) : "h"(h1), "f"(z1));
        a = f32x2(a0, a1);
#else
        const float2 f = __half22float2(reinterpret_cast<const __half2*>(&v)[e]);
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(a) : "l"(f32x2(f.x, f.y)), "l"(pp.neg_mn[e]));
#endif
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q) : "l"(a), "l"(pp.rcp[e]));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(pp.neg_sc[e]), "l"(q), "l"(a));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(r), "l"(pp.rcp[e]), "l"(q));
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(m) : "l"(q), "l"(magic));
        uint2 b;
        asm("mov.b64 {%0, %1}, %2;" : "=r"(b.x), "=r"(b.y) : "l"(m));
        bytes[e] = b.x + (b.y << 4);
    }
    return __byte_perm(__byte_perm(bytes[0], bytes[1], 0x0040), __byte_perm(bytes[2], bytes[3], 0x0040), 0x5410);
}

__device__ __forceinline__ unsigned h2_bits(__half2 v) { return *reinterpret_cast<unsigned*>(&v); }
__device__ __forceinline__ __half2 bits_h2(unsigned v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ bool half_bits_nonfinite(unsigned short b) { return (b & 0x7C00u) == 0x7C00u; }

// Minimum / maximum of half2 pairs. The reference scans with fminf / fmaxf, which skip NaN; kDropNan gives exactly
// that. The other form propagates NaN, so that one pass yields both the extremes and the fact that the tile holds
// a NaN (or, through the extremes themselves, an infinity) -- such tiles are redone with the NaN-skipping form.
template <bool kDropNan> __device__ __forceinline__ __half2 min2(__half2 a, __half2 b) {
    if constexpr (kDropNan) return __hmin2(a, b); else return __hmin2_nan(a, b);
}
template <bool kDropNan> __device__ __forceinline__ __half2 max2(__half2 a, __half2 b) {
    if constexpr (kDropNan) return __hmax2(a, b); else return __hmax2_nan(a, b);
}
template <bool kDropNan> __device__ __forceinline__ __half min1(__half a, __half b) {
    if constexpr (kDropNan) return __hmin(a, b); else return __hmin_nan(a, b);
}
template <bool kDropNan> __device__ __forceinline__ __half max1(__half a, __half b) {
    if constexpr (kDropNan) return __hmax(a, b); else return __hmax_nan(a, b);
}

// scale, zero-point and reciprocal of one group from its extremes (reference arithmetic)
__device__ __forceinline__ float4 group_params(float mn, float mx) {
    float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
    if (!(scale > 0.0f)) scale = 1.0f;
    return make_float4(mn, scale, __frcp_rn(scale), 0.0f);
}

// What a thread of the register-tile pack keeps for a run of groups of one (sequence, kv head, keys | values):
// a few base pointers and 32-bit strides, so that one multiply-add per row forms an address. Thread (w, r) =
// (tid % WPR, tid / WPR) owns the 16-byte word w of rows r, r + RPP, ... of every group.
template <class Shape>
struct TileCtx {
    static constexpr int D = Shape::d, G = Shape::g, B = Shape::b;
    static constexpr int WPR = D / 8, RPP = kThreads / WPR, NK = G / RPP;
    // Either a pass covers whole pages (the row within the page is the same in every pass) or a page takes several
    // passes (r < RPP <= B); both make the page and the row of pass k compile-time functions of k on top of r.
    static constexpr bool kWholePages = RPP % B == 0;
    static_assert(kThreads % WPR == 0 && G % RPP == 0 && NK >= 1 && NK <= 8, "shape not covered by the register tile");
    static_assert(kWholePages || B % RPP == 0, "rows per pass and page size must divide one another");
    const unsigned char* scratch_w;   // word w of scratch row r (scratch row 0 holds absolute position prev_old)
    const unsigned char* fresh_w;     // word w of the new row at absolute position prev_old + r: before the array while that
                                      // position predates the call, and never dereferenced then
    uint32_t fresh_row_bytes;         // bytes between consecutive new rows of one kv head
    int n_scratch;                    // positions prev_old .. prev_old + n_scratch - 1 predate the call (scratch rows)
    int r;
    unsigned char* codes_w;           // the thread's code word in its row of a page whose id is 0
    uint32_t page_bytes;              // bytes of codes per page, all kv heads
    const int* pages;                 // block-table entry of the page of position prev_old (+ r / B with whole pages)
    uint32_t tile32;                  // shared-window address of the thread's 16 bytes of pass 0 in the tile
};

template <class Shape>
__device__ __forceinline__ TileCtx<Shape> tile_ctx(const WriteParams& p, const SeqWrite& s, int h, bool values, uint4* tile) {
    using C = TileCtx<Shape>;
    C c;
    const int tid = threadIdx.x, w = tid % C::WPR, r = tid / C::WPR;
    const uint32_t nkv = (uint32_t)p.geom.nkv;
    const __half* scratch = values ? p.cache.v_scratch : p.cache.k_scratch;
    const __half* fresh = values ? p.new_v : p.new_k;
    c.scratch_w = reinterpret_cast<const unsigned char*>(
        scratch + (((size_t)s.slot * nkv + h) * p.geom.scratch_rows + r) * C::D + w * 8);
    c.fresh_row_bytes = nkv * C::D * 2u;
    c.fresh_w = reinterpret_cast<const unsigned char*>(fresh) +
                ((long long)(s.new_row0 + s.prev_old + r - s.start) * nkv + h) * (C::D * 2) + w * 16;
    c.n_scratch = s.start - s.prev_old;
    c.r = r;
    c.codes_w = (values ? p.cache.v_code : p.cache.k_code) + (((size_t)h * C::B + (C::kWholePages ? r % C::B : r)) * C::WPR + w) * 4;
    c.page_bytes = nkv * C::B * C::WPR * 4u;
    c.pages = s.bt + s.prev_old / C::B + (C::kWholePages ? r / C::B : 0);
    c.tile32 = smem_u32(tile) + tid * 16;
    return c;
}

// Requests the thread's words of group j (counted from prev_old) as asynchronous 16-byte copies into the tile:
// word k of thread tid lands at tile[k * kThreads + tid], so a thread later reads back only what it asked for
// itself (cp.async.wait_all, no barrier). A group nearly always lies wholly in the scratch or wholly in the new
// rows; then its rows are a fixed stride apart.
template <class Shape>
__device__ __forceinline__ void request_tile(const TileCtx<Shape>& c, int j) {
    using C = TileCtx<Shape>;
    const int rel0 = j * C::G;
    if (rel0 >= c.n_scratch) {
        const unsigned char* src = c.fresh_w + (unsigned long long)(uint32_t)rel0 * c.fresh_row_bytes;
        const uint32_t pass_bytes = C::RPP * c.fresh_row_bytes;
#pragma unroll
        for (int k = 0; k < C::NK; ++k)
            cp_async16_32(c.tile32 + k * kThreads * 16, src + (unsigned long long)pass_bytes * (uint32_t)k);
    } else if (rel0 + C::G <= c.n_scratch) {
        const unsigned char* src = c.scratch_w + rel0 * (C::D * 2);
#pragma unroll
        for (int k = 0; k < C::NK; ++k) cp_async16_32(c.tile32 + k * kThreads * 16, src + k * C::RPP * C::D * 2);
    } else {
#pragma unroll
        for (int k = 0; k < C::NK; ++k) {
            const int rel = rel0 + k * C::RPP;   // row r of the pass; c.r is folded into both base pointers
            const unsigned char* src = rel + c.r < c.n_scratch ? c.scratch_w + rel * (C::D * 2)
                                                               : c.fresh_w + (unsigned long long)(uint32_t)rel * c.fresh_row_bytes;
            cp_async16_32(c.tile32 + k * kThreads * 16, src);
        }
    }
}

// Quantises group j of the run from its tile in registers (x[k] = the thread's word of row r + RPP k) into the
// group's pages. `work` is pack_smem_bytes() of shared memory; the function ends without a barrier: its first
// write to `work` for the next group comes before a barrier every thread has to reach after its last read here.
template <class Shape>
__device__ __forceinline__ void pack_tile(const WriteParams& p, const TileCtx<Shape>& c, int h, int j, bool values,
                                          uint4 (&x)[TileCtx<Shape>::NK], unsigned char* work) {
    using C = TileCtx<Shape>;
    constexpr int D = C::D, B = C::B, WPR = C::WPR, RPP = C::RPP, NK = C::NK, PPG = Shape::pages_per_group;
    constexpr bool kWholePages = C::kWholePages;
    const int tid = threadIdx.x, w = tid % WPR, lane = tid & 31, warp = tid >> 5;
    const uint32_t nkv = (uint32_t)p.geom.nkv;
    // the group's pages; pass k of this thread lies in page pages[...] at a compile-time row offset
    const int* pages = c.pages + j * PPG;
    const int* group_pages = pages - (kWholePages ? c.r / B : 0);   // the same for every thread
    // (read where the codes are stored, not here: the ids would only occupy registers through the reduction)
    auto code_word = [&](int k) -> uint32_t* {
        const uint32_t page = (uint32_t)pages[kWholePages ? (RPP / B) * k : (RPP * k) / B];
        return reinterpret_cast<uint32_t*>(c.codes_w + (unsigned long long)page * c.page_bytes) + (kWholePages ? 0 : ((RPP * k) % B) * WPR);
    };

    if (!values) {
        // ---------------- keys: per channel over the G tokens ----------------
        uint4* part = reinterpret_cast<uint4*>(work);                                    // [8 warps][WPR][min, max]
        float* p_neg_min = reinterpret_cast<float*>(part + (kThreads / 32) * WPR * 2);   // [D] each: -zero, -scale, 1/scale
        float* p_neg_scale = p_neg_min + D;
        float* p_rcp = p_neg_scale + D;
        __half* p_scale16 = reinterpret_cast<__half*>(p_rcp + D);                        // [D] each: what the pages store
        __half* p_zero16 = p_scale16 + D;
        // One round: extremes of the thread's rows, of the warp's rows (lanes that differ above the word index), the
        // warps' partial results through shared memory, and per channel (thread c < D) the group's parameters.
        // Returns whether this thread's channel has a NaN or an infinity among its extremes.
        auto round = [&](auto drop) -> bool {
            constexpr bool kDrop = decltype(drop)::value;
            __half2 mn[4], mx[4];
            {
                const __half2* h0 = reinterpret_cast<const __half2*>(&x[0]);
#pragma unroll
                for (int e = 0; e < 4; ++e) { mn[e] = h0[e]; mx[e] = h0[e]; }
            }
#pragma unroll
            for (int k = 1; k < NK; ++k) {
                const __half2* hk = reinterpret_cast<const __half2*>(&x[k]);
#pragma unroll
                for (int e = 0; e < 4; ++e) { mn[e] = min2<kDrop>(mn[e], hk[e]); mx[e] = max2<kDrop>(mx[e], hk[e]); }
            }
#pragma unroll
            for (int off = WPR; off < 32; off <<= 1)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    mn[e] = min2<kDrop>(mn[e], bits_h2(__shfl_xor_sync(0xffffffffu, h2_bits(mn[e]), off)));
                    mx[e] = max2<kDrop>(mx[e], bits_h2(__shfl_xor_sync(0xffffffffu, h2_bits(mx[e]), off)));
                }
            if (lane < WPR) {
                part[(warp * WPR + w) * 2] = make_uint4(h2_bits(mn[0]), h2_bits(mn[1]), h2_bits(mn[2]), h2_bits(mn[3]));
                part[(warp * WPR + w) * 2 + 1] = make_uint4(h2_bits(mx[0]), h2_bits(mx[1]), h2_bits(mx[2]), h2_bits(mx[3]));
            }
            __syncthreads();
            bool nonfinite = false;
            if (tid < D) {
                const int ch = tid;
                const __half* col = reinterpret_cast<const __half*>(part) + (ch / 8) * 16 + (ch % 8);
                __half lo = col[0], hi = col[8];
#pragma unroll
                for (int q = 1; q < kThreads / 32; ++q) {
                    lo = min1<kDrop>(lo, col[q * WPR * 16]);
                    hi = max1<kDrop>(hi, col[q * WPR * 16 + 8]);
                }
                nonfinite = half_bits_nonfinite(__half_as_ushort(lo)) || half_bits_nonfinite(__half_as_ushort(hi));
                const float4 gp = group_params(__half2float(lo), __half2float(hi));
                p_neg_min[ch] = -gp.x;
                p_neg_scale[ch] = -gp.y;
                p_rcp[ch] = gp.z;
                p_scale16[ch] = __float2half_rn(gp.y);
                p_zero16[ch] = __float2half_rn(gp.x);
            }
            return nonfinite;
        };
        bool exact = __syncthreads_or(round(std::false_type{}));
        if (exact) {
            // rare: some channel holds a NaN or an infinity. Extremes as the reference takes them (NaN skipped), and
            // the plain IEEE division below.
            round(std::true_type{});
            __syncthreads();
        }
        // scale and zero-point of every channel into each of the group's pages, two channels per store
        {
            constexpr int kPairs = D / 2, kStores = 2 * PPG * kPairs;
            const uint32_t page_param_bytes = nkv * D * 2u;   // bytes of scales (or zero-points) per page
#pragma unroll
            for (int base = 0; base < kStores; base += kThreads) {
                const int idx = base + tid;
                if (kStores % kThreads == 0 || idx < kStores) {
                    const int row = idx / kPairs, cp = idx % kPairs, zero = row / PPG, pi = row % PPG;
                    const uint32_t page = (uint32_t)group_pages[pi];
                    unsigned char* dst = reinterpret_cast<unsigned char*>(zero ? p.cache.k_zero : p.cache.k_scale) +
                                         (unsigned long long)page * page_param_bytes + (uint32_t)((h * D + 2 * cp) * 2);
                    *reinterpret_cast<__half2*>(dst) = reinterpret_cast<const __half2*>(zero ? p_zero16 : p_scale16)[cp];
                }
            }
        }
        // a thread packs the same eight channels of all its rows: their parameters stay in registers, already
        // negated and paired the way the packed arithmetic takes them
        if (!exact) {
            PackPairs pp;
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const ulonglong2 a = *reinterpret_cast<const ulonglong2*>(p_neg_min + w * 8 + 2 * e);
                const ulonglong2 b = *reinterpret_cast<const ulonglong2*>(p_neg_scale + w * 8 + 2 * e);
                const ulonglong2 cc = *reinterpret_cast<const ulonglong2*>(p_rcp + w * 8 + 2 * e);
                pp.neg_mn[e] = a.x; pp.neg_mn[e + 1] = a.y;
                pp.neg_sc[e] = b.x; pp.neg_sc[e + 1] = b.y;
                pp.rcp[e] = cc.x; pp.rcp[e + 1] = cc.y;
            }
#pragma unroll
            for (int k = 0; k < NK; ++k) *code_word(k) = pack_word_pairs(x[k], pp);
        } else {
            float pmn[8], psc[8], prc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) { pmn[e] = -p_neg_min[w * 8 + e]; psc[e] = -p_neg_scale[w * 8 + e]; prc[e] = p_rcp[w * 8 + e]; }
#pragma unroll
            for (int k = 0; k < NK; ++k) *code_word(k) = pack_word(x[k], pmn, psc, prc, true);
        }
        return;
    }

    // ---------------- values: per token over each channel group ----------------
    // LPI neighbouring lanes hold one (token, channel group). Each lane folds its word into the half2
    // (min, -max); the warp's folded words go through shared memory so that lane i can finish group i of
    // the warp: the parameter arithmetic is then issued once per warp, not once per row.
    constexpr int VG = Shape::vg, HG = Shape::hg, LPI = VG / 8, GPP = 32 / LPI, IPW = GPP * NK;   // groups per pass / per warp
    static_assert(LPI >= 4 && LPI <= 32 && (LPI & (LPI - 1)) == 0 && IPW <= 32, "value groups not covered");
    unsigned* folded = reinterpret_cast<unsigned*>(work) + warp * (NK * 32);                  // [NK][32 lanes]
    float4* params = reinterpret_cast<float4*>(work + (kThreads / 32) * NK * 32 * 4) + warp * IPW * 2;   // [IPW][2]:
    // (-zero, -zero, -scale, -scale), (1/scale, 1/scale, zero, scale): operand pairs of the packed arithmetic
    auto round = [&](auto drop) -> bool {
        constexpr bool kDrop = decltype(drop)::value;
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const __half2* hk = reinterpret_cast<const __half2*>(&x[k]);
            const __half2 lo = min2<kDrop>(min2<kDrop>(hk[0], hk[1]), min2<kDrop>(hk[2], hk[3]));
            const __half2 hi = max2<kDrop>(max2<kDrop>(hk[0], hk[1]), max2<kDrop>(hk[2], hk[3]));
            const unsigned nhi = h2_bits(hi) ^ 0x80008000u;   // -max: the maximum becomes a minimum
            const __half2 a = bits_h2(__byte_perm(h2_bits(lo), nhi, 0x5410));   // (lo.x, -hi.x)
            const __half2 b = bits_h2(__byte_perm(h2_bits(lo), nhi, 0x7632));   // (lo.y, -hi.y)
            folded[k * 32 + lane] = h2_bits(min2<kDrop>(a, b));
        }
        __syncwarp();
        bool nonfinite = false;
        if (lane < IPW) {
            const uint4* src = reinterpret_cast<const uint4*>(folded + lane * LPI);
            uint4 v = src[0];
#pragma unroll
            for (int q = 1; q < LPI / 4; ++q) {
                const uint4 u = src[q];
                v.x = h2_bits(min2<kDrop>(bits_h2(v.x), bits_h2(u.x))); v.y = h2_bits(min2<kDrop>(bits_h2(v.y), bits_h2(u.y)));
                v.z = h2_bits(min2<kDrop>(bits_h2(v.z), bits_h2(u.z))); v.w = h2_bits(min2<kDrop>(bits_h2(v.w), bits_h2(u.w)));
            }
            const __half2 m = min2<kDrop>(min2<kDrop>(bits_h2(v.x), bits_h2(v.y)), min2<kDrop>(bits_h2(v.z), bits_h2(v.w)));
            const __half lo = __low2half(m), hi = __hneg(__high2half(m));
            nonfinite = half_bits_nonfinite(__half_as_ushort(lo)) || half_bits_nonfinite(__half_as_ushort(hi));
            const float4 gp = group_params(__half2float(lo), __half2float(hi));
            params[lane * 2] = make_float4(-gp.x, -gp.x, -gp.y, -gp.y);
            params[lane * 2 + 1] = make_float4(gp.z, gp.z, gp.x, gp.y);
        }
        return nonfinite;
    };
    const bool exact = __any_sync(0xffffffffu, round(std::false_type{}));
    if (exact) {   // rare: a NaN or an infinity somewhere in the warp's rows; extremes as the reference takes them
        __syncwarp();
        round(std::true_type{});
    }
    if (lane < IPW) {
        // group `lane` of the warp: pass k, lanes [first, first + LPI) of that pass
        const int k = lane / GPP, first = (lane % GPP) * LPI;
        const int t = (warp * 32 + first) / WPR + RPP * k, cg = ((first % WPR) * 8) / VG;
        const uint32_t page = (uint32_t)group_pages[t / B];
        const unsigned long long param = (unsigned long long)page * (nkv * B * HG * 2u) + (uint32_t)(((h * B + (t % B)) * HG + cg) * 2);
        const float4 gp = params[lane * 2 + 1];
        *reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(p.cache.v_scale) + param) = __float2half_rn(gp.w);
        *reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(p.cache.v_zero) + param) = __float2half_rn(gp.z);
    }
    __syncwarp();
    if (!exact) {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const float4* gp = params + (k * GPP + lane / LPI) * 2;
            const ulonglong2 a = *reinterpret_cast<const ulonglong2*>(gp);
            const unsigned long long cc = *reinterpret_cast<const unsigned long long*>(gp + 1);
            PackPairs pp;
#pragma unroll
            for (int e = 0; e < 4; ++e) { pp.neg_mn[e] = a.x; pp.neg_sc[e] = a.y; pp.rcp[e] = cc; }
            *code_word(k) = pack_word_pairs(x[k], pp);
        }
    } else {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const float4 gp = params[(k * GPP + lane / LPI) * 2 + 1];
            const float pmn[8] = {gp.z, gp.z, gp.z, gp.z, gp.z, gp.z, gp.z, gp.z};
            const float psc[8] = {gp.w, gp.w, gp.w, gp.w, gp.w, gp.w, gp.w, gp.w};
            const float prc[8] = {gp.x, gp.x, gp.x, gp.x, gp.x, gp.x, gp.x, gp.x};
            *code_word(k) = pack_word(x[k], pmn, psc, prc, true);
        }
    }
}

// One group on its own (the kernels that write a token or a few per call): request the tile, wait, pack.
// smem_raw holds pack_smem_bytes(): the tile first, then the pack's work area.
template <class Shape>
__device__ __forceinline__ void pack_group_regs(const WriteParams& p, const SeqWrite& s, int h, int j, bool values,
                                                unsigned char* smem_raw) {
    using C = TileCtx<Shape>;
    const C c = tile_ctx<Shape>(p, s, h, values, reinterpret_cast<uint4*>(smem_raw));
    request_tile(c, j);
    cp_async_wait_all();
    uint4 x[C::NK];
#pragma unroll
    for (int k = 0; k < C::NK; ++k) x[k] = lds128(c.tile32 + k * kThreads * 16);
    pack_tile<Shape>(p, c, h, j, values, x, smem_raw + (size_t)C::G * C::D * sizeof(__half));
}

// Quantises the keys (values == false) or the values of aged-out group j of (sequence s, kv head h) into
// its pages. Called by every thread of a CTA of kThreads threads; smem_raw holds pack_smem_bytes().
template <class Shape>
__device__ __forceinline__ void pack_group_staged(const WriteParams& p, const Shape& g, const SeqWrite& s, int h, int j,
                                                  bool values, unsigned char* smem_raw) {
    const int nkv = p.geom.nkv;

    const int nparam = g.d > g.g * g.hg ? g.d : g.g * g.hg;
    __half* tile = reinterpret_cast<__half*>(smem_raw);                  // keys or values [G, D]
    float* p_min = reinterpret_cast<float*>(tile + (size_t)g.g * g.d);   // [nparam] each
    float* p_scale = p_min + nparam;
    float* p_rcp = p_scale + nparam;
    float* part_min = p_rcp + nparam;                                    // [parts, D]
    float* part_max = part_min + kThreads * 2;

    __shared__ int s_exact;   // some scale or zero-point of the tile is Inf/NaN: use the plain division
    if (threadIdx.x == 0) s_exact = 0;
    const int pos0 = s.prev_old + j * g.g;
    const int lp0 = pos0 / g.b;
    if (lp0 + g.pages_per_group > p.seq.bt_width) return;  // table too narrow: host validation failed
    const int words_per_row = g.d / 8;

    if (values) stage_tile(g, p, s, p.cache.v_scratch, p.new_v, h, pos0, tile);
    else stage_tile(g, p, s, p.cache.k_scratch, p.new_k, h, pos0, tile);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---------------- keys: per channel over the G tokens ----------------
    if (!values) {
    {
        // thread = (channel pair, slice of the rows); fminf/fmaxf drop NaN and order -0 below +0, so
        // any reduction order gives the reference's serial result
        const int pairs = g.d / 2, parts = kThreads / pairs;
        const int cp = threadIdx.x % pairs, part = threadIdx.x / pairs;
        if (part < parts) {
            const int rows = (g.g + parts - 1) / parts;
            const int r0 = part * rows, r1 = min(g.g, r0 + rows);
            float mn0 = NAN, mx0 = NAN, mn1 = NAN, mx1 = NAN;   // NaN is the neutral element of fmin/fmax
#pragma unroll 8
            for (int t = r0; t < r1; ++t) {
                const float2 x = __half22float2(reinterpret_cast<const __half2*>(tile + (size_t)t * g.d)[cp]);
                mn0 = fminf(mn0, x.x); mx0 = fmaxf(mx0, x.x);
                mn1 = fminf(mn1, x.y); mx1 = fmaxf(mx1, x.y);
            }
            part_min[part * g.d + 2 * cp] = mn0; part_max[part * g.d + 2 * cp] = mx0;
            part_min[part * g.d + 2 * cp + 1] = mn1; part_max[part * g.d + 2 * cp + 1] = mx1;
        }
        __syncthreads();
        for (int c = threadIdx.x; c < g.d; c += kThreads) {
            float mn = part_min[c], mx = part_max[c];
            for (int q = 1; q < parts; ++q) { mn = fminf(mn, part_min[q * g.d + c]); mx = fmaxf(mx, part_max[q * g.d + c]); }
            float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
            if (!(scale > 0.0f)) scale = 1.0f;
            p_min[c] = mn;
            p_scale[c] = scale;
            p_rcp[c] = __frcp_rn(scale);
            if (!(fabsf(mn) < INFINITY && scale < INFINITY)) s_exact = 1;
            const __half hs = __float2half_rn(scale), hz = __float2half_rn(mn);
            for (int pi = 0; pi < g.pages_per_group; ++pi) {
                size_t page = (size_t)s.bt[lp0 + pi];
                p.cache.k_scale[(page * nkv + h) * g.d + c] = hs;
                p.cache.k_zero[(page * nkv + h) * g.d + c] = hz;
            }
        }
    }
    __syncthreads();
    if (kThreads % words_per_row == 0) {
        // a thread packs the same eight channels of every token it visits: their parameters stay in registers
        const int w = threadIdx.x % words_per_row;
        float mn[8], sc[8], rc[8];
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
            *reinterpret_cast<float4*>(mn + e) = *reinterpret_cast<const float4*>(p_min + w * 8 + e);
            *reinterpret_cast<float4*>(sc + e) = *reinterpret_cast<const float4*>(p_scale + w * 8 + e);
            *reinterpret_cast<float4*>(rc + e) = *reinterpret_cast<const float4*>(p_rcp + w * 8 + e);
        }
        const bool exact = s_exact != 0;
#pragma unroll 4
        for (int idx = threadIdx.x; idx < g.g * words_per_row; idx += kThreads) {
            const int t = idx / words_per_row;
            const uint4 v = reinterpret_cast<const uint4*>(tile)[idx];
            const size_t page = (size_t)s.bt[lp0 + t / g.b];
            uint32_t* dst = reinterpret_cast<uint32_t*>(p.cache.k_code + ((page * nkv + h) * g.b + (t % g.b)) * (g.d / 2));
            dst[w] = pack_word(v, mn, sc, rc, exact);
        }
        return;
    }
#pragma unroll 4
    for (int idx = threadIdx.x; idx < g.g * words_per_row; idx += kThreads) {
        const int t = idx / words_per_row, w = idx - t * words_per_row;
        const uint4 v = reinterpret_cast<const uint4*>(tile)[idx];
        float mn[8], sc[8], rc[8];
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
            *reinterpret_cast<float4*>(mn + e) = *reinterpret_cast<const float4*>(p_min + w * 8 + e);
            *reinterpret_cast<float4*>(sc + e) = *reinterpret_cast<const float4*>(p_scale + w * 8 + e);
            *reinterpret_cast<float4*>(rc + e) = *reinterpret_cast<const float4*>(p_rcp + w * 8 + e);
        }
        const size_t page = (size_t)s.bt[lp0 + t / g.b];
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.cache.k_code + ((page * nkv + h) * g.b + (t % g.b)) * (g.d / 2));
        dst[w] = pack_word(v, mn, sc, rc, s_exact != 0);
    }
    return;
    }

    // ---------------- values: per token over each channel group ----------------
    {
        // two adjacent lanes share one (token, channel group); each starts at a different word to
        // spread the shared-memory banks
        const int items = g.g * g.hg, seg_words = g.vg / 2, half_words = seg_words / 2;
        for (int base = 0; base < items * 2; base += kThreads) {
            const int id = base + threadIdx.x;
            const int item = id >> 1, side = id & 1;
            float mn = NAN, mx = NAN;
            if (item < items) {
                const int t = item / g.hg, cg = item - t * g.hg;
                const __half2* seg = reinterpret_cast<const __half2*>(tile + (size_t)t * g.d + cg * g.vg) + side * half_words;
#pragma unroll 8
                for (int k = 0; k < half_words; ++k) {
                    const float2 x = __half22float2(seg[(k + t) % half_words]);
                    mn = fminf(mn, fminf(x.x, x.y));
                    mx = fmaxf(mx, fmaxf(x.x, x.y));
                }
            }
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            if (item < items && side == 0) {
                const int t = item / g.hg, cg = item - t * g.hg;
                float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
                if (!(scale > 0.0f)) scale = 1.0f;
                p_min[item] = mn;
                p_scale[item] = scale;
                p_rcp[item] = __frcp_rn(scale);
                if (!(fabsf(mn) < INFINITY && scale < INFINITY)) s_exact = 1;
                const size_t page = (size_t)s.bt[lp0 + t / g.b];
                const size_t param = ((page * nkv + h) * g.b + (t % g.b)) * g.hg + cg;
                p.cache.v_scale[param] = __float2half_rn(scale);
                p.cache.v_zero[param] = __float2half_rn(mn);
            }
        }
    }
    __syncthreads();
#pragma unroll 4
    for (int idx = threadIdx.x; idx < g.g * words_per_row; idx += kThreads) {
        const int t = idx / words_per_row, w = idx - t * words_per_row;
        const uint4 v = reinterpret_cast<const uint4*>(tile)[idx];
        const int item = t * g.hg + (w * 8) / g.vg;
        const float m1 = p_min[item], s1 = p_scale[item], r1 = p_rcp[item];
        const float mn[8] = {m1, m1, m1, m1, m1, m1, m1, m1};
        const float sc[8] = {s1, s1, s1, s1, s1, s1, s1, s1};
        const float rc[8] = {r1, r1, r1, r1, r1, r1, r1, r1};
        const size_t page = (size_t)s.bt[lp0 + t / g.b];
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.cache.v_code + ((page * nkv + h) * g.b + (t % g.b)) * (g.d / 2));
        dst[w] = pack_word(v, mn, sc, rc, s_exact != 0);
    }
}

template <class Shape>
__device__ __forceinline__ void pack_group(const WriteParams& p, const Shape& g, const SeqWrite& s, int h, int j,
                                           bool values, unsigned char* smem_raw) {
    if constexpr (Shape::in_registers) pack_group_regs<Shape>(p, s, h, j, values, smem_raw);
    else pack_group_staged(p, g, s, h, j, values, smem_raw);
}

// The scratch update of (sequence s, kv head h) for the keys, the values or both: move-to-front of the rows that
// stay, then append of the new rows that stay. Called by every thread of a CTA of kThreads threads.
template <bool kKeys, bool kValues>
__device__ __forceinline__ void scratch_shift_of(const WriteParams& p, const SeqWrite& s, int h) {
    const Geom& g = p.geom;
    const int delta = s.next_old - s.prev_old;
    if (delta <= 0 || s.start <= s.next_old) return;
    const int chunks_per_row = g.d / 8;
    uint4* ks = reinterpret_cast<uint4*>(p.cache.k_scratch + ((size_t)s.slot * g.nkv + h) * g.scratch_rows * g.d);
    uint4* vs = reinterpret_cast<uint4*>(p.cache.v_scratch + ((size_t)s.slot * g.nkv + h) * g.scratch_rows * g.d);
    // rows [delta, delta + keep) -> [0, keep); destination below source, ascending steps.
    const int keep = s.start - s.next_old;
    const int total = keep * chunks_per_row;
    const int shift = delta * chunks_per_row;
    for (int base = 0; base < total; base += kThreads) {
        int c = base + threadIdx.x;
        uint4 a = make_uint4(0, 0, 0, 0), b = a;
        if (c < total) {
            if (kKeys) a = ks[c + shift];
            if (kValues) b = vs[c + shift];
        }
        __syncthreads();
        if (c < total) {
            if (kKeys) ks[c] = a;
            if (kValues) vs[c] = b;
        }
    }
    __syncthreads();
}
// New rows whose absolute position is at or beyond next_old stay in the scratch; the first `skip` of them are
// somebody else's business (the pack kernel brings them in through its tile).
template <bool kKeys, bool kValues>
__device__ __forceinline__ void scratch_append_of(const WriteParams& p, const SeqWrite& s, int h, int skip) {
    const Geom& g = p.geom;
    const int chunks_per_row = g.d / 8;
    uint4* ks = reinterpret_cast<uint4*>(p.cache.k_scratch + ((size_t)s.slot * g.nkv + h) * g.scratch_rows * g.d);
    uint4* vs = reinterpret_cast<uint4*>(p.cache.v_scratch + ((size_t)s.slot * g.nkv + h) * g.scratch_rows * g.d);
    const int first = (s.start > s.next_old ? s.start : s.next_old) + skip;
    const int rows = s.end - first;
    const int total = rows * chunks_per_row;
    const uint32_t row_words = (uint32_t)g.nkv * chunks_per_row;
    const size_t row0 = ((size_t)(s.new_row0 + first - s.start) * g.nkv + h) * chunks_per_row;
    const uint4* src_k = reinterpret_cast<const uint4*>(p.new_k) + row0;
    const uint4* src_v = reinterpret_cast<const uint4*>(p.new_v) + row0;
    const int dst0 = (first - s.next_old) * chunks_per_row;
    for (int c = threadIdx.x; c < total; c += kThreads) {
        const int t = c / chunks_per_row, w = c - t * chunks_per_row;
        const size_t src = (size_t)((uint32_t)t * row_words) + w;
        if (kKeys) ks[dst0 + c] = src_k[src];
        if (kValues) vs[dst0 + c] = src_v[src];
    }
}
__device__ __forceinline__ void scratch_update(const WriteParams& p, const SeqWrite& s, int h) {
    scratch_shift_of<true, true>(p, s, h);
    scratch_append_of<true, true>(p, s, h, 0);
}

// keys and values of a group are quantised independently (per channel / per token): one CTA each, so a
// tile's worth of shared memory per CTA and twice the loads in flight per SM
template <class Shape>
__global__ void __launch_bounds__(kThreads, Shape::in_registers ? 3 : 1) pack_groups_kernel(const WriteParams p, int per_cta,
                                                                                             int with_scratch_update) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Shape g(p.geom);
    const int i = blockIdx.z, h = blockIdx.y, lane_j = blockIdx.x >> 1, lanes = gridDim.x >> 1;
    const bool values = blockIdx.x & 1;
    pdl_trigger();
    pdl_wait();   // new rows, lengths and tables may come from the kernel before this one
    const SeqWrite s = seq_write(p, i);
    const int ngroups = (s.next_old - s.prev_old) / g.g;
    if constexpr (Shape::in_registers) {
        // A CTA takes a run of `per_cta` consecutive groups of its tensor (keys | values): the next group's rows are
        // on their way (asynchronous copies into a shared-memory tile) while the current one is packed.
        const int j0 = lane_j * per_cta, j1 = min(ngroups, j0 + per_cta);
        // with_scratch_update: the CTA of the first run also moves and appends its tensor's scratch rows when its
        // groups are packed (the launcher sees to it that every group read from the scratch lies in the first run)
        const bool updates = with_scratch_update && lane_j == 0 && s.num_new > 0;
        if (j0 >= j1 && !updates) return;
        // shared memory: the tile first, then what pack_tile needs for itself
        using C = TileCtx<Shape>;
        const C c = tile_ctx<Shape>(p, s, h, values, reinterpret_cast<uint4*>(smem_raw));
        unsigned char* work = smem_raw + (size_t)Shape::g * Shape::d * sizeof(__half);
        // The new rows that stay in the scratch are positions [first, end). As many of them as the tile holds (G
        // rows) are requested into it while the last group is packed, and written out from there afterwards.
        const int first = s.start > s.next_old ? s.start : s.next_old;
        const int early = updates ? min(s.end - first, C::G) : 0;
        auto request_staying_rows = [&]() {
            const int rel0 = first - s.prev_old;   // c.fresh_w belongs to position prev_old + r
#pragma unroll
            for (int k = 0; k < C::NK; ++k)
                if (c.r + C::RPP * k < early)
                    cp_async16_32(c.tile32 + k * kThreads * 16,
                                  c.fresh_w + (unsigned long long)(uint32_t)(rel0 + C::RPP * k) * c.fresh_row_bytes);
        };
        // the block-table entries of a group are read when its codes are stored; asked for one group ahead, they
        // are in the L1 by then
        auto touch_pages = [&](int j) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(c.pages + j * Shape::pages_per_group));
        };
        if (j0 < j1) { request_tile(c, j0); touch_pages(j0); }
        else request_staying_rows();
        for (int j = j0; j < j1; ++j) {
            cp_async_wait_all();
            // the tile into registers, and the same shared-memory words are free for the next group's rows
            // (a thread overwrites only what it has just read itself)
            uint4 x[C::NK];
#pragma unroll
            for (int k = 0; k < C::NK; ++k) x[k] = lds128(c.tile32 + k * kThreads * 16);
            if (j + 1 < j1) { request_tile(c, j + 1); touch_pages(j + 1); }
            else request_staying_rows();
            pack_tile<Shape>(p, c, h, j, values, x, work);
        }
        if (updates) {
            cp_async_wait_all();
            __syncthreads();   // every thread's copies out of the scratch have landed: its rows may be overwritten
            if (values) scratch_shift_of<false, true>(p, s, h);
            else scratch_shift_of<true, false>(p, s, h);
            unsigned char* dst = const_cast<unsigned char*>(c.scratch_w) + (size_t)(first - s.next_old) * (C::D * 2);
#pragma unroll
            for (int k = 0; k < C::NK; ++k)
                if (c.r + C::RPP * k < early)
                    *reinterpret_cast<uint4*>(dst + k * C::RPP * C::D * 2) = lds128(c.tile32 + k * kThreads * 16);
            if (s.end - first > early) {
                if (values) scratch_append_of<false, true>(p, s, h, early);
                else scratch_append_of<true, false>(p, s, h, early);
            }
        }
    } else {
        (void)per_cta; (void)with_scratch_update;
        for (int j = lane_j; j < ngroups; j += lanes) {
            pack_group(p, g, s, h, j, values, smem_raw);
            __syncthreads();
        }
    }
}

__global__ void __launch_bounds__(kThreads) scratch_update_kernel(const WriteParams p) {
    const int i = blockIdx.y, h = blockIdx.x;
    pdl_trigger();
    pdl_wait();   // the pack kernel has read the rows this kernel moves
    const SeqWrite s = seq_write(p, i);
    if (s.num_new == 0) return;
    scratch_update(p, s, h);
}

// A few new tokens per sequence (decode steps, speculative drafts): everything the writer does for (sequence i,
// kv head h) in one CTA and one launch -- quantise the group that ages out, if one does, move the scratch, append.
// The two-kernel form above spreads a long chunk's groups over many CTAs; for a token or two per sequence its
// group CTAs would nearly all leave at once and the second launch would only add latency.
template <class Shape>
__global__ void __launch_bounds__(kThreads) append_write_kernel(const WriteParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Shape g(p.geom);
    const int h = blockIdx.x, i = blockIdx.y;
    pdl_trigger();
    pdl_wait();   // new rows, lengths and tables may come from the kernel before this one
    const SeqWrite s = seq_write(p, i);
    if (s.num_new == 0) return;
    const int ngroups = (s.next_old - s.prev_old) / g.g;
    for (int j = 0; j < ngroups; ++j) {
        pack_group(p, g, s, h, j, false, smem_raw);
        __syncthreads();
        pack_group(p, g, s, h, j, true, smem_raw);
        __syncthreads();
    }
    scratch_update(p, s, h);
}

// One decode step's worth of the path between the QKV projection and the attention, in one launch:
// bias add + RoPE + q/k/v split of sequence i for kv head h and the query heads of its group
// (bias_rope_kernel of step.cu, same arithmetic), then the cache write of that one new token for
// (i, h): quantise the group that ages out, if one does (every G-th step), move the scratch and
// append. One CTA per (kv head, sequence); the rows it appends are the ones it has just rotated.
template <class Shape>
__global__ void __launch_bounds__(kThreads) rope_write_kernel(const RopeParams rp, const WriteParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Shape g(p.geom);
    const int h = blockIdx.x, i = blockIdx.y;
    const int nh = p.geom.nh, nkv = p.geom.nkv, qpk = p.geom.qpk, hd = g.d, half_dim = hd >> 1;
    pdl_trigger();
    const __half* row = rp.qkv + (size_t)i * (nh + 2 * nkv) * hd;
    const int pos = rp.positions[i];
    // heads 0..qpk-1: the query heads of this kv head; head qpk: its key head
    for (int idx = threadIdx.x; idx < (qpk + 1) * half_dim; idx += kThreads) {
        const int hl = idx / half_dim, e = idx - hl * half_dim;
        const int head = hl < qpk ? h * qpk + hl : nh + h;            // position in the qkv row
        const __half* in = row + (size_t)head * hd;
        __half* out = hl < qpk ? rp.q + ((size_t)i * nh + head) * hd : rp.k + ((size_t)i * nkv + h) * hd;
        rope_pair(in[e], in[e + half_dim], rp.bias ? rp.bias + (size_t)head * hd : nullptr, e, hd, pos, rp.rope_base, out);
    }
    {   // value head: bias add only
        const size_t voff = (size_t)(nh + nkv + h) * hd;
        __half* out = rp.v + ((size_t)i * nkv + h) * hd;
        for (int e = threadIdx.x; e < hd; e += kThreads) out[e] = rp.bias ? __hadd(row[voff + e], rp.bias[voff + e]) : row[voff + e];
    }
    __threadfence();   // the rows just written are read back below, partly by asynchronous copies
    __syncthreads();
    const SeqWrite s = seq_write(p, i);
    const int ngroups = (s.next_old - s.prev_old) / g.g;
    for (int j = 0; j < ngroups; ++j) {
        pack_group(p, g, s, h, j, false, smem_raw);
        __syncthreads();
        pack_group(p, g, s, h, j, true, smem_raw);
        __syncthreads();
    }
    if (s.num_new > 0) scratch_update(p, s, h);
}

// Dynamic shared memory of the pack: the staged form holds the tile and its parameters, the register-tile
// form only what crosses lanes (keys: per-warp extremes and the channel parameters; values: the folded
// words of every warp and the group parameters).
template <class Shape>
size_t pack_smem_bytes(const Geom& g) {
    if constexpr (Shape::in_registers) {
        constexpr int WPR = Shape::d / 8, RPP = kThreads / WPR, NK = Shape::g / RPP, LPI = Shape::vg / 8;
        constexpr size_t keys = (size_t)(kThreads / 32) * WPR * 32 + 3 * Shape::d * sizeof(float) + 2 * Shape::d * sizeof(__half);
        constexpr size_t vals = (size_t)(kThreads / 32) * NK * 32 * 4 + (size_t)(kThreads / 32) * (32 / LPI) * NK * 32;
        constexpr size_t tile = (size_t)Shape::g * Shape::d * sizeof(__half);   // the rows of one group, as requested by request_tile
        return tile + (keys > vals ? keys : vals);
    } else {
        size_t params = (size_t)(g.d > g.g * g.hg ? g.d : g.g * g.hg);
        return (size_t)g.g * g.d * sizeof(__half) + (3 * params + 4 * kThreads) * sizeof(float);
    }
}

template <class Shape>
cudaError_t launch_pack(const WriteParams& p, dim3 grid, int per_cta, int with_scratch_update, cudaStream_t stream) {
    size_t smem = pack_smem_bytes<Shape>(p.geom);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(pack_groups_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(pack_groups_kernel<Shape>, grid, dim3(kThreads), smem, stream, p, per_cta, with_scratch_update);
}

template <int D, int G>
cudaError_t launch_pack_for_block(const WriteParams& p, dim3 grid, int per_cta, int with_scratch_update, cudaStream_t stream,
                                  bool* done) {
    *done = true;
    if (p.geom.b == 16) return launch_pack<StaticShape<D, G, 16>>(p, grid, per_cta, with_scratch_update, stream);
    if (p.geom.b == 32) return launch_pack<StaticShape<D, G, 32>>(p, grid, per_cta, with_scratch_update, stream);
    *done = false;
    return cudaSuccess;
}

template <class Shape>
cudaError_t launch_rope_write_shape(const RopeParams& rp, const WriteParams& p, cudaStream_t stream) {
    const size_t smem = pack_smem_bytes<Shape>(p.geom);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(rope_write_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    rope_write_kernel<Shape><<<dim3(p.geom.nkv, p.n), kThreads, smem, stream>>>(rp, p);
    return cudaGetLastError();
}

template <class Shape>
cudaError_t launch_append_shape(const WriteParams& p, cudaStream_t stream) {
    const size_t smem = pack_smem_bytes<Shape>(p.geom);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(append_write_kernel<Shape>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(append_write_kernel<Shape>, dim3(p.geom.nkv, p.n), dim3(kThreads), smem, stream, p);
}

template <int D, int G>
cudaError_t launch_append_for_block(const WriteParams& p, cudaStream_t stream, bool* done) {
    *done = true;
    if (p.geom.b == 16) return launch_append_shape<StaticShape<D, G, 16>>(p, stream);
    if (p.geom.b == 32) return launch_append_shape<StaticShape<D, G, 32>>(p, stream);
    *done = false;
    return cudaSuccess;
}

template <int D, int G>
cudaError_t launch_rope_write_for_block(const RopeParams& rp, const WriteParams& p, cudaStream_t stream, bool* done) {
    *done = true;
    if (p.geom.b == 16) return launch_rope_write_shape<StaticShape<D, G, 16>>(rp, p, stream);
    if (p.geom.b == 32) return launch_rope_write_shape<StaticShape<D, G, 32>>(rp, p, stream);
    *done = false;
    return cudaSuccess;
}

}  // namespace

// RoPE of one new token per sequence fused with its cache write. p.new_k / p.new_v must be rp.k / rp.v,
// one row per sequence (new_offsets == nullptr, num_new_scalar == 1).
cudaError_t launch_rope_write(const RopeParams& rp, const WriteParams& p, cudaStream_t stream) {
    const Geom& g = p.geom;
    if (p.n <= 0) return cudaSuccess;
    if (p.new_k != rp.k || p.new_v != rp.v || p.new_offsets || p.num_new_scalar != 1) return cudaErrorInvalidValue;
    bool done = false;
    cudaError_t e = cudaSuccess;
    if (g.d == 128 && g.g == 128) e = launch_rope_write_for_block<128, 128>(rp, p, stream, &done);
    else if (g.d == 128 && g.g == 64) e = launch_rope_write_for_block<128, 64>(rp, p, stream, &done);
    else if (g.d == 128 && g.g == 32) e = launch_rope_write_for_block<128, 32>(rp, p, stream, &done);
    else if (g.d == 64 && g.g == 128) e = launch_rope_write_for_block<64, 128>(rp, p, stream, &done);
    else if (g.d == 64 && g.g == 64) e = launch_rope_write_for_block<64, 64>(rp, p, stream, &done);
    else if (g.d == 64 && g.g == 32) e = launch_rope_write_for_block<64, 32>(rp, p, stream, &done);
    if (e != cudaSuccess) return e;
    if (!done) e = launch_rope_write_shape<DynamicShape>(rp, p, stream);
    return e;
}

// Chunks up to this many tokens per sequence are written by the one-launch form.
constexpr int kAppendMaxNew = 8;

cudaError_t launch_cache_write(const WriteParams& p, int max_new_per_seq, cudaStream_t stream) {
    const Geom& g = p.geom;
    if (p.n <= 0 || max_new_per_seq <= 0) return cudaSuccess;
    if (max_new_per_seq <= kAppendMaxNew) {
        bool done = false;
        cudaError_t e = cudaSuccess;
        if (g.d == 128 && g.g == 128) e = launch_append_for_block<128, 128>(p, stream, &done);
        else if (g.d == 128 && g.g == 64) e = launch_append_for_block<128, 64>(p, stream, &done);
        else if (g.d == 128 && g.g == 32) e = launch_append_for_block<128, 32>(p, stream, &done);
        else if (g.d == 64 && g.g == 128) e = launch_append_for_block<64, 128>(p, stream, &done);
        else if (g.d == 64 && g.g == 64) e = launch_append_for_block<64, 64>(p, stream, &done);
        else if (g.d == 64 && g.g == 32) e = launch_append_for_block<64, 32>(p, stream, &done);
        if (e != cudaSuccess) return e;
        return done ? cudaSuccess : launch_append_shape<DynamicShape>(p, stream);
    }
    // Quantise the groups that age out and move / append the scratch rows.
    // Compile-time shapes, one launch: a CTA takes a run of consecutive groups of one tensor (keys | values), so that
    // the next group's rows travel while the current one is packed; the CTA of the first run then also updates its
    // tensor's scratch rows, which only its own groups were read from: a run is at least as long as the groups the
    // scratch can hold, (R + G - 1) / G rounded up. Runs are as long as leaves about two CTAs per resident slot
    // (three per multiprocessor) -- with many sequences one CTA per (sequence, kv head, tensor), no CTA without a group.
    // KIVI_PACK_GROUPS_PER_CTA in the environment overrides the run length (for measurements).
    // Other geometries: one CTA per (group, tensor), then a second kernel for the scratch.
    const int max_groups = max_new_per_seq / g.g + 1;
    const int from_scratch = (g.r + g.g - 1 + g.g - 1) / g.g;
    static const int forced = [] { const char* e = getenv("KIVI_PACK_GROUPS_PER_CTA"); return e ? atoi(e) : 0; }();
    const int fuse = 1;
    const long long tensors = 2LL * g.nkv * p.n, want_ctas = 2LL * 3 * sm_count();
    const int lanes_wanted = (int)((want_ctas + tensors - 1) / tensors);
    int per_cta = forced > 0 ? forced : (max_groups + lanes_wanted - 1) / lanes_wanted;
    if (per_cta < from_scratch) per_cta = from_scratch;
    if (per_cta > max_groups) per_cta = max_groups;
    const int lanes = (max_groups + per_cta - 1) / per_cta;
    bool done = false;
    cudaError_t e = cudaSuccess;
    const dim3 run_grid(2 * lanes, g.nkv, p.n);   // (run of groups, keys | values)
    if (g.d == 128 && g.g == 128) e = launch_pack_for_block<128, 128>(p, run_grid, per_cta, fuse, stream, &done);
    else if (g.d == 128 && g.g == 64) e = launch_pack_for_block<128, 64>(p, run_grid, per_cta, fuse, stream, &done);
    else if (g.d == 128 && g.g == 32) e = launch_pack_for_block<128, 32>(p, run_grid, per_cta, fuse, stream, &done);
    else if (g.d == 64 && g.g == 128) e = launch_pack_for_block<64, 128>(p, run_grid, per_cta, fuse, stream, &done);
    else if (g.d == 64 && g.g == 64) e = launch_pack_for_block<64, 64>(p, run_grid, per_cta, fuse, stream, &done);
    else if (g.d == 64 && g.g == 32) e = launch_pack_for_block<64, 32>(p, run_grid, per_cta, fuse, stream, &done);
    if (e != cudaSuccess) return e;
    if (done && fuse) return cudaSuccess;
    // any other geometry: one CTA per (group, tensor)
    if (!done) e = launch_pack<DynamicShape>(p, dim3(2 * max_groups, g.nkv, p.n), 1, 0, stream);
    if (e != cudaSuccess) return e;
    return launch_pdl(scratch_update_kernel, dim3(g.nkv, p.n), dim3(kThreads), 0, stream, p);
}

}  // namespace kivi

extern "C" int kivi_b200_writer_rejected_indices(uint32_t* count) {
    if (!count) return KIVI_ERR_NULL_POINTER;
    return cudaMemcpyFromSymbol(count, kivi::g_writer_rejected, sizeof(uint32_t)) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}
