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
//   pack kernel    one CTA per (sequence, kv head, aged-out group): the G x D tile is staged in
//                  shared memory with 16-byte loads, min/max are reduced in parallel (min/max
//                  are order-independent, so the result is bit-identical to the serial scan) and
//                  codes leave as 32-bit words, 8 channels each, fully coalesced;
//   scratch kernel one CTA per (sequence, kv head): overlapping move-to-front through registers
//                  with a barrier per step, then the append of the rows that stay unquantised.
// A token at absolute position p comes from scratch row p - old_tokens when it predates the call,
// else from the new rows; that indirection is what lets one call cross several boundaries and
// still equal the token-by-token writer.
#include "kivi_common.cuh"

namespace kivi {
namespace {

constexpr int kThreads = 256;

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
__device__ __forceinline__ unsigned code_of(float x, float mn, float scale) {
    int c = __float2int_rn(__fdiv_rn(__fsub_rn(x, mn), scale));
    c = c < 0 ? 0 : c;
    return (unsigned)(c > 15 ? 15 : c);
}

__device__ __forceinline__ void stage_tile(const WriteParams& p, const SeqWrite& s, const __half* scratch,
                                           const __half* fresh, int h, int pos0, __half* tile) {
    const Geom& g = p.geom;
    const int chunks_per_row = g.d / 8;
    const int total = g.g * chunks_per_row;
    for (int c = threadIdx.x; c < total; c += kThreads) {
        int t = c / chunks_per_row, w = c - t * chunks_per_row;
        const uint4* src = reinterpret_cast<const uint4*>(token_row(p, s, scratch, fresh, h, pos0 + t));
        reinterpret_cast<uint4*>(tile)[c] = src[w];
    }
}

__global__ void __launch_bounds__(kThreads) pack_groups_kernel(const WriteParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geom& g = p.geom;
    const int i = blockIdx.z, h = blockIdx.y, j = blockIdx.x;
    const SeqWrite s = seq_write(p, i);
    const int ngroups = (s.next_old - s.prev_old) / g.g;
    if (j >= ngroups) return;

    __half* tile = reinterpret_cast<__half*>(smem_raw);                  // [G, D]
    float* p_min = reinterpret_cast<float*>(tile + (size_t)g.g * g.d);   // [max(D, G*HG)]
    float* p_scale = p_min + (g.d > g.g * g.hg ? g.d : g.g * g.hg);

    const int pos0 = s.prev_old + j * g.g;
    const int lp0 = pos0 / g.b;
    if (lp0 + g.pages_per_group > p.seq.bt_width) return;  // table too narrow: host validation failed
    const int words_per_row = g.d / 8;

    // ---------------- keys: per channel over the G tokens ----------------
    stage_tile(p, s, p.cache.k_scratch, p.new_k, h, pos0, tile);
    __syncthreads();
    for (int c = threadIdx.x; c < g.d; c += kThreads) {
        float mn = __half2float(tile[c]);
        float mx = mn;
        for (int t = 1; t < g.g; ++t) {
            float x = __half2float(tile[(size_t)t * g.d + c]);
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
        float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
        if (!(scale > 0.0f)) scale = 1.0f;
        p_min[c] = mn;
        p_scale[c] = scale;
        const __half hs = __float2half_rn(scale), hz = __float2half_rn(mn);
        for (int pi = 0; pi < g.pages_per_group; ++pi) {
            size_t page = (size_t)s.bt[lp0 + pi];
            p.cache.k_scale[(page * g.nkv + h) * g.d + c] = hs;
            p.cache.k_zero[(page * g.nkv + h) * g.d + c] = hz;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < g.g * words_per_row; idx += kThreads) {
        int t = idx / words_per_row, w = idx - t * words_per_row;
        const __half* row = tile + (size_t)t * g.d + w * 8;
        unsigned word = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int c = w * 8 + e;
            word |= code_of(__half2float(row[e]), p_min[c], p_scale[c]) << (4 * e);
        }
        size_t page = (size_t)s.bt[lp0 + t / g.b];
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.cache.k_code + ((page * g.nkv + h) * g.b + (t % g.b)) * (g.d / 2));
        dst[w] = word;
    }
    __syncthreads();

    // ---------------- values: per token over each channel group ----------------
    stage_tile(p, s, p.cache.v_scratch, p.new_v, h, pos0, tile);
    __syncthreads();
    // One thread per (token, channel group). fminf/fmaxf drop a NaN operand and order -0 below
    // +0, so the result does not depend on the scan order; each thread starts at a different
    // word to spread the shared-memory banks.
    for (int idx = threadIdx.x; idx < g.g * g.hg; idx += kThreads) {
        int t = idx / g.hg, cg = idx - t * g.hg;
        const int seg_words = g.vg / 2;
        const __half2* seg = reinterpret_cast<const __half2*>(tile + (size_t)t * g.d + cg * g.vg);
        float2 x0 = __half22float2(seg[t % seg_words]);
        float mn = fminf(x0.x, x0.y), mx = fmaxf(x0.x, x0.y);
        for (int k = 1; k < seg_words; ++k) {
            float2 x = __half22float2(seg[(k + t) % seg_words]);
            mn = fminf(mn, fminf(x.x, x.y));
            mx = fmaxf(mx, fmaxf(x.x, x.y));
        }
        p_min[idx] = mn;
        p_scale[idx] = mx;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < g.g * g.hg; idx += kThreads) {
        int t = idx / g.hg, cg = idx - t * g.hg;
        float mn = p_min[idx], mx = p_scale[idx];
        float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
        if (!(scale > 0.0f)) scale = 1.0f;
        p_scale[idx] = scale;
        size_t page = (size_t)s.bt[lp0 + t / g.b];
        size_t param = ((page * g.nkv + h) * g.b + (t % g.b)) * g.hg + cg;
        p.cache.v_scale[param] = __float2half_rn(scale);
        p.cache.v_zero[param] = __float2half_rn(mn);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < g.g * words_per_row; idx += kThreads) {
        int t = idx / words_per_row, w = idx - t * words_per_row;
        const __half* row = tile + (size_t)t * g.d + w * 8;
        const int cg = (w * 8) / g.vg;
        const float mn = p_min[t * g.hg + cg], scale = p_scale[t * g.hg + cg];
        unsigned word = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) word |= code_of(__half2float(row[e]), mn, scale) << (4 * e);
        size_t page = (size_t)s.bt[lp0 + t / g.b];
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.cache.v_code + ((page * g.nkv + h) * g.b + (t % g.b)) * (g.d / 2));
        dst[w] = word;
    }
}

// Move-to-front of the rows that stay in the scratch, then append of the new rows that stay.
__global__ void __launch_bounds__(kThreads) scratch_update_kernel(const WriteParams p) {
    const Geom& g = p.geom;
    const int i = blockIdx.y, h = blockIdx.x;
    const SeqWrite s = seq_write(p, i);
    if (s.num_new == 0) return;
    const int delta = s.next_old - s.prev_old;
    const int chunks_per_row = g.d / 8;
    uint4* ks = reinterpret_cast<uint4*>(p.cache.k_scratch + ((size_t)s.slot * g.nkv + h) * g.scratch_rows * g.d);
    uint4* vs = reinterpret_cast<uint4*>(p.cache.v_scratch + ((size_t)s.slot * g.nkv + h) * g.scratch_rows * g.d);

    if (delta > 0 && s.start > s.next_old) {
        // rows [delta, delta + keep) -> [0, keep); destination below source, ascending steps.
        const int keep = s.start - s.next_old;
        const int total = keep * chunks_per_row;
        const int shift = delta * chunks_per_row;
        for (int base = 0; base < total; base += kThreads) {
            int c = base + threadIdx.x;
            uint4 a = make_uint4(0, 0, 0, 0), b = a;
            if (c < total) { a = ks[c + shift]; b = vs[c + shift]; }
            __syncthreads();
            if (c < total) { ks[c] = a; vs[c] = b; }
        }
        __syncthreads();
    }
    // New rows whose absolute position is at or beyond next_old stay in the scratch.
    const int first = s.start > s.next_old ? s.start : s.next_old;
    const int rows = s.end - first;
    const int total = rows * chunks_per_row;
    for (int c = threadIdx.x; c < total; c += kThreads) {
        int t = c / chunks_per_row, w = c - t * chunks_per_row;
        int pos = first + t;
        size_t src = ((size_t)(s.new_row0 + pos - s.start) * g.nkv + h) * chunks_per_row + w;
        int dst = (pos - s.next_old) * chunks_per_row + w;
        ks[dst] = reinterpret_cast<const uint4*>(p.new_k)[src];
        vs[dst] = reinterpret_cast<const uint4*>(p.new_v)[src];
    }
}

size_t pack_smem_bytes(const Geom& g) {
    size_t params = (size_t)(g.d > g.g * g.hg ? g.d : g.g * g.hg);
    return (size_t)g.g * g.d * sizeof(__half) + 2 * params * sizeof(float);
}

}  // namespace

cudaError_t launch_cache_write(const WriteParams& p, int max_new_per_seq, cudaStream_t stream) {
    const Geom& g = p.geom;
    if (p.n <= 0 || max_new_per_seq <= 0) return cudaSuccess;
    const size_t smem = pack_smem_bytes(g);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(pack_groups_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int max_groups = max_new_per_seq / g.g + 1;
    pack_groups_kernel<<<dim3(max_groups, g.nkv, p.n), kThreads, smem, stream>>>(p);
    scratch_update_kernel<<<dim3(g.nkv, p.n), kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace kivi
