// Merge of the split-context partials of the decode kernels.
//
// A decode launch whose plan cuts the context into chunks leaves, per (sequence, kv head, chunk,
// query head), a running maximum m (log2 units), a sum l and an unnormalised accumulator o[D] in the
// workspace. One CTA per (sequence, kv head, query head) combines them:
//     O = sum_c 2^(m_c - M) o_c / sum_c 2^(m_c - M) l_c,   M = max_c m_c.
// The partials were written by other SMs, so every read is an L2 round trip of the order of a
// microsecond; the kernel is organised so that each thread has all of its loads in flight at once
// (thread (lane of chunks, run of four channels) owns every LANES-th chunk), pays that latency once
// and finishes through shared memory.
#include "decode_merge.cuh"

namespace kivi {
namespace {

constexpr int kMergeThreads = 256;
constexpr int kMergeMaxLoads = 10;   // chunks per thread held in registers at once

__global__ void __launch_bounds__(kMergeThreads) decode_merge_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char merge_smem[];
    const Geom& g = p.geom;
    const int hq = blockIdx.x, kv = blockIdx.y, i = blockIdx.z;
    pdl_trigger();
    const int seq_len = seq_len_of(p.seq, i);
    const DecodeBounds bnd = effective_bounds(p, seq_len, i);
    const int nchunks = chunk_work(p, bnd, 0).nchunks;
    // Every CTA waits, also the ones with nothing to merge: a kernel launched behind this one only waits
    // for THIS grid, so a CTA that left early would let it overtake the decode kernel.
    pdl_wait();                 // the partials are complete and visible
    if (nchunks <= 1) return;   // the decode kernel wrote O itself

    const int quads = g.d / 4;                     // runs of four channels
    const int lanes = kMergeThreads / quads;       // chunk lanes
    const int cl = threadIdx.x / quads, dq = threadIdx.x - cl * quads;
    const size_t base = ((size_t)i * g.nkv + kv) * p.max_chunks;
    float2* ml = reinterpret_cast<float2*>(merge_smem);                  // [nchunks] (m, l) of this head
    float4* part = reinterpret_cast<float4*>(merge_smem + (((size_t)p.max_chunks * sizeof(float2) + 15) / 16) * 16);

    // all loads first: this thread's chunks of o, then the (m, l) pairs
    float4 v[kMergeMaxLoads];
    const bool active = cl < lanes;
#pragma unroll
    for (int k = 0; k < kMergeMaxLoads; ++k) {
        const int c = cl + k * lanes;
        v[k] = (active && c < nchunks)
                   ? __ldcg(reinterpret_cast<const float4*>(p.ws_o + ((base + c) * g.qpk + hq) * g.d) + dq)
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    for (int c = threadIdx.x; c < nchunks; c += kMergeThreads)
        ml[c] = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + ((base + c) * g.qpk + hq) * 2));
    __syncthreads();
    float mx = -1.0e30f;
    for (int c = 0; c < nchunks; ++c) mx = fmaxf(mx, ml[c].x);
    float l = 0.0f;
    for (int c = 0; c < nchunks; ++c) l += fast_exp2(ml[c].x - mx) * ml[c].y;

    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kMergeMaxLoads; ++k) {
        const int c = cl + k * lanes;
        if (active && c < nchunks) {
            const float w = fast_exp2(ml[c].x - mx);
            acc.x += w * v[k].x; acc.y += w * v[k].y; acc.z += w * v[k].z; acc.w += w * v[k].w;
        }
    }
    // contexts cut into more chunks than the registers hold: the rest in a plain loop
    if (active)
        for (int c = cl + kMergeMaxLoads * lanes; c < nchunks; c += lanes) {
            const float w = fast_exp2(ml[c].x - mx);
            const float4 o = __ldcg(reinterpret_cast<const float4*>(p.ws_o + ((base + c) * g.qpk + hq) * g.d) + dq);
            acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
        }
    if (active) part[cl * quads + dq] = acc;
    __syncthreads();
    if (threadIdx.x < quads) {
        float4 s = part[threadIdx.x];
        for (int k = 1; k < lanes; ++k) {
            const float4 o = part[k * quads + threadIdx.x];
            s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
        }
        const float inv = 1.0f / fmaxf(l, 1.0e-30f);
        const size_t out = ((size_t)i * g.nh + (size_t)kv * g.qpk + hq) * g.d + 4 * threadIdx.x;
        store_out(p, out, s.x * inv); store_out(p, out + 1, s.y * inv);
        store_out(p, out + 2, s.z * inv); store_out(p, out + 3, s.w * inv);
    }
}

// The same combination for the tensor-core kernel's jobs: one CTA per (query head, cut unit); the unit's k
// partials sit in consecutive slots. A part that held no item left a neutral slot (m = -1e30, zeros).
__global__ void __launch_bounds__(kMergeThreads) decode_part_merge_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char merge_smem[];
    const Geom& g = p.geom;
    const JobPlan& pl = p.plan;
    const int hq = blockIdx.x;
    pdl_trigger();
    pdl_wait();   // every CTA waits (see above); the partials are then complete and visible
    // blockIdx.y counts the cut units: those of the first class (when it is cut), then those of the second
    int unit, nparts, slot0;
    {
        const int cut1 = pl.k1 > 1 ? pl.units1 : 0;
        if ((int)blockIdx.y < cut1) {
            unit = blockIdx.y; nparts = pl.k1; slot0 = unit * pl.k1;
        } else {
            const int u = blockIdx.y - cut1;
            unit = pl.units1 + u; nparts = pl.k2; slot0 = (pl.k1 > 1 ? pl.jobs1() : 0) + u * pl.k2;
        }
    }
    const int i = unit / g.nkv, kv = unit - i * g.nkv;

    const int quads = g.d / 4;
    const int lanes = kMergeThreads / quads;
    const int cl = threadIdx.x / quads, dq = threadIdx.x - cl * quads;
    float2* ml = reinterpret_cast<float2*>(merge_smem);                  // [nparts] (m, l) of this head
    float4* part = reinterpret_cast<float4*>(merge_smem + (((size_t)nparts * sizeof(float2) + 15) / 16) * 16);

    // all loads first (a part that held no item left zeros and m = -1e30, so nothing needs checking)
    float4 v[kMergeMaxLoads];
    const bool active = cl < lanes;
#pragma unroll
    for (int k = 0; k < kMergeMaxLoads; ++k) {
        const int c = cl + k * lanes;
        v[k] = (active && c < nparts)
                   ? __ldcg(reinterpret_cast<const float4*>(p.ws_o + ((size_t)(slot0 + c) * g.qpk + hq) * g.d) + dq)
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    for (int k = threadIdx.x; k < nparts; k += kMergeThreads)
        ml[k] = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + ((size_t)(slot0 + k) * g.qpk + hq) * 2));
    __syncthreads();
    float mx = -1.0e30f;
    for (int c = 0; c < nparts; ++c) mx = fmaxf(mx, ml[c].x);
    float l = 0.0f;
    for (int c = 0; c < nparts; ++c) l += fast_exp2(ml[c].x - mx) * ml[c].y;

    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kMergeMaxLoads; ++k) {
        const int c = cl + k * lanes;
        if (active && c < nparts) {
            const float w = fast_exp2(ml[c].x - mx);
            acc.x += w * v[k].x; acc.y += w * v[k].y; acc.z += w * v[k].z; acc.w += w * v[k].w;
        }
    }
    if (active)
        for (int c = cl + kMergeMaxLoads * lanes; c < nparts; c += lanes) {
            const float w = fast_exp2(ml[c].x - mx);
            const float4 o = __ldcg(reinterpret_cast<const float4*>(p.ws_o + ((size_t)(slot0 + c) * g.qpk + hq) * g.d) + dq);
            acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
        }
    if (cl < lanes) part[cl * quads + dq] = acc;
    __syncthreads();
    if (threadIdx.x < quads) {
        float4 s = part[threadIdx.x];
        for (int k = 1; k < lanes; ++k) {
            const float4 o = part[k * quads + threadIdx.x];
            s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
        }
        const float inv = 1.0f / fmaxf(l, 1.0e-30f);
        const size_t out = ((size_t)i * g.nh + (size_t)kv * g.qpk + hq) * g.d + 4 * threadIdx.x;
        store_out(p, out, s.x * inv); store_out(p, out + 1, s.y * inv);
        store_out(p, out + 2, s.z * inv); store_out(p, out + 3, s.w * inv);
    }
}

}  // namespace

cudaError_t launch_decode_merge(const DecodeParams& p, cudaStream_t stream) {
    if (p.n <= 0 || p.max_chunks <= 1) return cudaSuccess;
    if (p.geom.d % 4 || p.geom.d / 4 > kMergeThreads) return cudaErrorInvalidValue;
    const size_t smem = (((size_t)p.max_chunks * sizeof(float2) + 15) / 16) * 16 + (size_t)kMergeThreads * sizeof(float4);
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    return launch_pdl(decode_merge_kernel, dim3(p.geom.qpk, p.geom.nkv, p.n), dim3(kMergeThreads), smem, stream, p);
}

}  // namespace kivi

namespace kivi {

cudaError_t launch_decode_part_merge(const DecodeParams& p, cudaStream_t stream) {
    const int cut = p.plan.cut_units();
    if (p.n <= 0 || cut <= 0) return cudaSuccess;
    if (p.geom.d % 4 || p.geom.d / 4 > kMergeThreads) return cudaErrorInvalidValue;
    const int kmax = p.plan.k1 > p.plan.k2 ? p.plan.k1 : p.plan.k2;
    const size_t smem = (((size_t)kmax * sizeof(float2) + 15) / 16) * 16 + (size_t)kMergeThreads * sizeof(float4);
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    return launch_pdl(decode_part_merge_kernel, dim3(p.geom.qpk, cut), dim3(kMergeThreads), smem, stream, p);
}

}  // namespace kivi
