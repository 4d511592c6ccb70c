// Split-context plumbing shared by both decode kernels. Each CTA of a (sequence, kv head) writes its
// partial (running max in log2 units, sum, unnormalised accumulator) per query head to the
// workspace; a small merge kernel launched behind the decode kernel (decode_merge.cu) combines them
// and writes O. No CTA waits for another, so there is nothing here that can spin.
#pragma once
#include "kivi_common.cuh"

namespace kivi {

// Effective scan bounds of one query: quantised tokens to walk (already reduced to the retained
// pages in sparse mode) and residual rows.
__device__ __forceinline__ DecodeBounds effective_bounds(const DecodeParams& p, int seq_len, int i) {
    const Geom& g = p.geom;
    const bool sparse = p.retained_pages >= 0 || p.retained_dev != nullptr;
    DecodeBounds b = decode_bounds(seq_len, g.r, g.g, p.max_seq, sparse ? 0x3fffffff / g.b : p.seq.bt_width, g.b);
    if (sparse) {
        int dense_pages = b.old_valid / g.b;
        const int retained = p.retained_dev ? p.retained_dev[i] : p.retained_pages;
        int rp = retained < dense_pages ? retained : dense_pages;
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

// Launched behind a decode kernel whose launch plan splits the context (max_chunks > 1).
cudaError_t launch_decode_merge(const DecodeParams& p, cudaStream_t stream);

}  // namespace kivi
