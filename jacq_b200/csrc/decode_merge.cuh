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

// Work of one CTA of a (sequence, kv head): quantised tokens [tok0, tok1) and, for one of them, the
// fp16 residual rows. When the quantised part is split over several CTAs the residual gets a CTA
// of its own, so that it is walked alongside the chunks and not after the last one.
struct ChunkWork { int nchunks, tok0, tok1; bool with_residual; };

__device__ __forceinline__ ChunkWork chunk_work(const DecodeParams& p, const DecodeBounds& b, int chunk) {
    ChunkWork w;
    const int qc = b.old_valid > 0 ? (b.old_valid + p.chunk_tokens - 1) / p.chunk_tokens : 0;
    const bool own = qc > 1 && b.res_valid > 0;
    w.nchunks = own ? qc + 1 : (qc > 0 ? qc : 1);
    if (own && chunk == qc) {
        w.tok0 = w.tok1 = b.old_valid;
        w.with_residual = true;
    } else {
        w.tok0 = chunk * p.chunk_tokens;
        w.tok1 = b.old_valid < w.tok0 + p.chunk_tokens ? b.old_valid : w.tok0 + p.chunk_tokens;
        w.with_residual = !own && chunk == w.nchunks - 1;
    }
    return w;
}

// Call with all threads of the CTA after the partials of this CTA were stored. `scratch` is shared
// memory the CTA no longer needs (or nullptr). With enough of it the merge runs in two parallel
// phases: one warp per query head turns the chunks' (max, sum) pairs into normalised weights, then
// every thread owns up to MAXI output elements as runs of four and keeps eight chunks of each in flight. Without
// scratch each output element walks the chunks on its own.
template <int MAXI>
__device__ __forceinline__ void merge_when_last(const DecodeParams& p, int i, int kv, int nchunks, float* scratch,
                                                int scratch_floats) {
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
    const int outputs = g.qpk * g.d;
    const size_t out0 = ((size_t)i * g.nh + (size_t)kv * g.qpk) * g.d;
    if (scratch && nchunks * g.qpk <= scratch_floats && outputs <= MAXI * (int)blockDim.x && g.d % 4 == 0) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
        for (int hq = warp; hq < g.qpk; hq += nwarps) {
            float mx = -1.0e30f;
            for (int c = lane; c < nchunks; c += 32) mx = fmaxf(mx, __ldcg(p.ws_ml + ((base + c) * g.qpk + hq) * 2));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float l = 0.0f;
            for (int c = lane; c < nchunks; c += 32) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + ((base + c) * g.qpk + hq) * 2));
                const float w = fast_exp2(ml.x - mx);
                scratch[c * g.qpk + hq] = w;
                l += w * ml.y;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
            const float inv = 1.0f / fmaxf(l, 1.0e-30f);
            __syncwarp();
            for (int c = lane; c < nchunks; c += 32) scratch[c * g.qpk + hq] *= inv;
        }
        __syncthreads();
        // every thread owns up to MAXI / 4 runs of four consecutive channels and keeps eight chunks of
        // each in flight as 16-byte loads
        constexpr int MAXQ = MAXI / 4 > 0 ? MAXI / 4 : 1;
        const int quads = outputs / 4;
        float4 acc[MAXQ];
        int hq_of[MAXQ], d_of[MAXQ];
#pragma unroll
        for (int k = 0; k < MAXQ; ++k) {
            const int qd = threadIdx.x + k * blockDim.x;
            acc[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            hq_of[k] = qd < quads ? (qd * 4) / g.d : -1;
            d_of[k] = qd < quads ? qd * 4 - hq_of[k] * g.d : 0;
        }
        for (int c = 0; c < nchunks; c += 8) {
            float4 v[8][MAXQ];
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int k = 0; k < MAXQ; ++k)
                    v[u][k] = (c + u < nchunks && hq_of[k] >= 0)
                                  ? __ldcg(reinterpret_cast<const float4*>(p.ws_o + ((base + c + u) * g.qpk + hq_of[k]) * g.d + d_of[k]))
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int k = 0; k < MAXQ; ++k)
                    if (c + u < nchunks && hq_of[k] >= 0) {
                        const float w = scratch[(c + u) * g.qpk + hq_of[k]];
                        acc[k].x += w * v[u][k].x; acc[k].y += w * v[u][k].y;
                        acc[k].z += w * v[u][k].z; acc[k].w += w * v[u][k].w;
                    }
        }
#pragma unroll
        for (int k = 0; k < MAXQ; ++k)
            if (hq_of[k] >= 0) {
                const size_t o = out0 + (size_t)hq_of[k] * g.d + d_of[k];
                store_out(p, o, acc[k].x); store_out(p, o + 1, acc[k].y);
                store_out(p, o + 2, acc[k].z); store_out(p, o + 3, acc[k].w);
            }
    } else {
        for (int idx = threadIdx.x; idx < outputs; idx += blockDim.x) {
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
            store_out(p, out0 + (size_t)hq * g.d + d, acc / fmaxf(l, 1.0e-30f));
        }
    }
    if (threadIdx.x == 0) *counter = 0u;  // leave the workspace ready for the next launch
}

}  // namespace kivi
