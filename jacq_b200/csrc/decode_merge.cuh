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

// ---- jobs of the tensor-core kernel ------------------------------------------------------------------------
// A unit is one (sequence, kv head): its key groups, then its fp16 residual in 16-row tiles. An item weighs
// what it moves: a group of G tokens G/16, a tile kTileWeight (G D bytes of codes against 64 D bytes of fp16
// rows). Part c of k of a unit owns the items whose start offset lies in [share_begin(c), share_begin(c + 1))
// of the unit's weight. A unit that has no item at all weighs 1, so that somebody writes its all-zero output.
constexpr int kResTileRows = 16;
constexpr int kTileWeight = 4;

struct UnitShape { int ng, nres, res_valid, w; };   // key groups, residual tiles, residual rows, weight

__host__ __device__ inline UnitShape unit_shape_of(int old_valid, int res_valid, int group) {
    UnitShape u;
    u.ng = old_valid / group;
    u.res_valid = res_valid;
    u.nres = (res_valid + kResTileRows - 1) / kResTileRows;
    u.w = u.ng * (group / 16) + u.nres * kTileWeight;
    if (u.w == 0) u.w = 1;
    return u;
}
__device__ __forceinline__ UnitShape unit_shape(const DecodeParams& p, int i) {
    const DecodeBounds b = effective_bounds(p, seq_len_of(p.seq, i), i);
    return unit_shape_of(b.old_valid, b.res_valid, p.geom.g);
}

__host__ __device__ inline long long share_begin(long long total, int parts, int c) {
    return (total * c + parts - 1) / parts;
}

// Items of a unit whose start offset lies in [d_lo, d_hi) (offsets relative to the unit's start): key groups
// [g0, g1) and residual tiles [t0, t1). `complete`: the unit's every item, so the owner can write the output
// itself; otherwise it leaves a partial.
struct SegmentItems { int g0, g1, t0, t1; bool any, complete; };

__host__ __device__ inline SegmentItems segment_items(const UnitShape& u, int wg, int d_lo, int d_hi) {
    SegmentItems s;
    const int qw = u.ng * wg;
    auto lower = [](int a, int b) { return a < b ? a : b; };
    s.g0 = lower(u.ng, (d_lo + wg - 1) / wg);
    s.g1 = lower(u.ng, (d_hi + wg - 1) / wg);
    s.t0 = d_lo <= qw ? 0 : lower(u.nres, (d_lo - qw + kTileWeight - 1) / kTileWeight);
    s.t1 = d_hi <= qw ? 0 : lower(u.nres, (d_hi - qw + kTileWeight - 1) / kTileWeight);
    s.any = s.g1 > s.g0 || s.t1 > s.t0;
    s.complete = s.g0 == 0 && s.g1 == u.ng && s.t0 == 0 && s.t1 == u.nres;
    return s;
}

// Job j of a launch: which unit, which part of how many, and the partial slot it writes when parts > 1.
struct DecodeJob { int unit, part, parts, slot; };

__device__ __forceinline__ DecodeJob decode_job(const DecodeParams& p, int j) {
    const JobPlan& pl = p.plan;
    DecodeJob job;
    if (j < pl.jobs1()) {
        job.unit = j / pl.k1;
        job.part = j - job.unit * pl.k1;
        job.parts = pl.k1;
        job.slot = j;
    } else {
        const int jj = j - pl.jobs1();
        const int u = jj / pl.k2;
        job.unit = pl.units1 + u;
        job.part = jj - u * pl.k2;
        job.parts = pl.k2;
        job.slot = (pl.k1 > 1 ? pl.jobs1() : 0) + jj;
    }
    return job;
}

// Launched behind the tensor-core kernel: combines the partials of the units that were cut.
cudaError_t launch_decode_part_merge(const DecodeParams& p, cudaStream_t stream);

}  // namespace kivi
