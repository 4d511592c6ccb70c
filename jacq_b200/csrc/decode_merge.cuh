// Split-context merge shared by both decode kernels. Each CTA of a (sequence, kv head) writes its
// partial (running max in log2 units, sum, unnormalised accumulator) per query head to the
// workspace; the CTA whose arrival completes the count combines them and writes O. No CTA waits
// for another, so there is nothing here that can spin.
#pragma once
#include "kivi_common.cuh"

namespace kivi {

// Effective scan bounds of one query: quantised tokens to walk (already reduced to the retained
// pages in sparse mode) and residual rows.
__device__ __forceinline__ DecodeBounds effective_bounds(const DecodeParams& p, int seq_len) {
    const Geom& g = p.geom;
    const bool sparse = p.retained_pages >= 0;
    DecodeBounds b = decode_bounds(seq_len, g.r, g.g, p.max_seq, sparse ? 0x3fffffff / g.b : p.seq.bt_width, g.b);
    if (sparse) {
        int dense_pages = b.old_valid / g.b;
        int rp = p.retained_pages < dense_pages ? p.retained_pages : dense_pages;
        if (rp > p.seq.bt_width) rp = p.seq.bt_width;
        b.old_valid = (rp < 0 ? 0 : rp) * g.b;
    }
    return b;
}

__device__ __forceinline__ int chunks_of(const DecodeParams& p, int old_valid) {
    return old_valid > 0 ? (old_valid + p.chunk_tokens - 1) / p.chunk_tokens : 1;
}

// Call with all threads of the CTA after the partials of this CTA were stored.
__device__ __forceinline__ void merge_when_last(const DecodeParams& p, int i, int kv, int nchunks) {
    const Geom& g = p.geom;
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    unsigned int* counter = p.ws_count + (size_t)i * g.nkv + kv;
    if (threadIdx.x == 0) {
        unsigned int prev = atomicAdd(counter, 1u);
        s_last = (prev == (unsigned int)(nchunks - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t base = ((size_t)i * g.nkv + kv) * p.max_chunks;
    for (int idx = threadIdx.x; idx < g.qpk * g.d; idx += blockDim.x) {
        const int hq = idx / g.d, d = idx - hq * g.d;
        float mx = -1.0e30f;
        for (int c = 0; c < nchunks; ++c) mx = fmaxf(mx, __ldcg(p.ws_ml + ((base + c) * g.qpk + hq) * 2));
        float l = 0.0f, acc = 0.0f;
        for (int c = 0; c < nchunks; ++c) {
            const size_t pi = (base + c) * g.qpk + hq;
            const float w = fast_exp2(__ldcg(p.ws_ml + pi * 2) - mx);
            l += w * __ldcg(p.ws_ml + pi * 2 + 1);
            acc += w * __ldcg(p.ws_o + pi * g.d + d);
        }
        store_out(p, ((size_t)i * g.nh + kv * g.qpk + hq) * g.d + d, acc / fmaxf(l, 1.0e-30f));
    }
    if (threadIdx.x == 0) *counter = 0u;  // leave the workspace ready for the next launch
}

}  // namespace kivi
