// Generic paged KIVI decode attention: any geometry the layout allows (even head_dim up to 256,
// any query-group size, sparse-retained tables with group > block). It is the kernel for shapes
// the tensor-core kernel (decode_mma.cu) does not cover, not a CPU or library fallback.
//
// Arithmetic follows the reference kernel (crates/jac-codegen-cuda/src/variants.rs:2359-2431):
// per token, dequantise K with the page's per-channel scale/zero, dot with q, online softmax,
// dequantise V with the token's per-group scale/zero, accumulate; then the fp16 residual rows.
// Differences in schedule only: one CTA per (sequence, kv head, context chunk) with one warp per
// query head of the group, exp2 with log2(e) folded into the score scale, and a split over the
// context whose partial (max, sum, accumulator) triples are merged by the last CTA to arrive.
#include "kivi_common.cuh"
#include "decode_merge.cuh"

namespace kivi {
namespace {

constexpr int kMaxBytesPerLane = 4;  // head_dim <= 256
__device__ unsigned int g_generic_rejected;   // page / slot ids outside the pools, replaced by id 0

__global__ void __launch_bounds__(256) decode_generic_kernel(const DecodeParams p) {
    const Geom& g = p.geom;
    const int i = blockIdx.z, kv = blockIdx.y, chunk = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;

    const int seq_len = seq_len_of(p.seq, i);
    const DecodeBounds bnd = effective_bounds(p, seq_len, i);
    const int old_valid = bnd.old_valid;
    const ChunkWork work = chunk_work(p, bnd, chunk);
    const int nchunks = work.nchunks;
    if (chunk >= nchunks) return;
    const int t0 = work.tok0, t1 = work.tok1;
    const bool with_residual = work.with_residual;

    const int* bt = p.seq.block_tables + (size_t)i * p.seq.bt_stride;
    int slot = slot_of(p.seq, i);
    if (!index_in_pool(slot, p.cache.num_slots)) { slot = 0; if (threadIdx.x == 0) atomicAdd(&g_generic_rejected, 1u); }
    const int bytes_per_row = g.d / 2;
    const float score_scale = rsqrtf((float)g.d) * 1.4426950408889634f;

    for (int hq = warp; hq < g.qpk; hq += nwarps) {
        const int h = kv * g.qpk + hq;
        const __half* qh = p.q + ((size_t)i * g.nh + h) * g.d;
        float q0[kMaxBytesPerLane], q1[kMaxBytesPerLane];
        float a0[kMaxBytesPerLane], a1[kMaxBytesPerLane];
        float ks0[kMaxBytesPerLane], ks1[kMaxBytesPerLane], kz0[kMaxBytesPerLane], kz1[kMaxBytesPerLane];
#pragma unroll
        for (int k = 0; k < kMaxBytesPerLane; ++k) {
            int j = lane + 32 * k;
            bool on = j < bytes_per_row;
            q0[k] = on ? __half2float(qh[2 * j]) : 0.0f;
            q1[k] = on ? __half2float(qh[2 * j + 1]) : 0.0f;
            a0[k] = a1[k] = 0.0f;
            ks0[k] = ks1[k] = 1.0f;
            kz0[k] = kz1[k] = 0.0f;
        }
        float m = -1.0e30f, l = 0.0f;
        int cur_page = -1;

        for (int s = t0; s < t1; ++s) {
            const int lp = s / g.b, off = s - lp * g.b;
            int page = bt[lp];
            if (!index_in_pool(page, p.cache.num_blocks)) { page = 0; if (lane == 0 && off == 0) atomicAdd(&g_generic_rejected, 1u); }
            const size_t head_base = (size_t)page * g.nkv + kv;
            if (page != cur_page) {
                cur_page = page;
#pragma unroll
                for (int k = 0; k < kMaxBytesPerLane; ++k) {
                    int j = lane + 32 * k;
                    if (j < bytes_per_row) {
                        ks0[k] = __half2float(p.cache.k_scale[head_base * g.d + 2 * j]);
                        ks1[k] = __half2float(p.cache.k_scale[head_base * g.d + 2 * j + 1]);
                        kz0[k] = __half2float(p.cache.k_zero[head_base * g.d + 2 * j]);
                        kz1[k] = __half2float(p.cache.k_zero[head_base * g.d + 2 * j + 1]);
                    }
                }
            }
            const uint8_t* kc = p.cache.k_code + (head_base * g.b + off) * bytes_per_row;
            const uint8_t* vc = p.cache.v_code + (head_base * g.b + off) * bytes_per_row;
            const __half* vs = p.cache.v_scale + (head_base * g.b + off) * g.hg;
            const __half* vz = p.cache.v_zero + (head_base * g.b + off) * g.hg;
            float part = 0.0f;
#pragma unroll
            for (int k = 0; k < kMaxBytesPerLane; ++k) {
                int j = lane + 32 * k;
                if (j < bytes_per_row) {
                    unsigned byte = kc[j];
                    part += q0[k] * fmaf((float)(byte & 15u), ks0[k], kz0[k]);
                    part += q1[k] * fmaf((float)(byte >> 4), ks1[k], kz1[k]);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            const float score = part * score_scale;
            const float m_new = fmaxf(m, score);
            const float corr = fast_exp2(m - m_new);
            const float pr = fast_exp2(score - m_new);
            l = l * corr + pr;
#pragma unroll
            for (int k = 0; k < kMaxBytesPerLane; ++k) {
                int j = lane + 32 * k;
                if (j < bytes_per_row) {
                    unsigned byte = vc[j];
                    int cg = (2 * j) / g.vg;
                    float sc = __half2float(vs[cg]), zr = __half2float(vz[cg]);
                    a0[k] = a0[k] * corr + pr * fmaf((float)(byte & 15u), sc, zr);
                    a1[k] = a1[k] * corr + pr * fmaf((float)(byte >> 4), sc, zr);
                }
            }
            m = m_new;
        }

        if (with_residual) {
            const __half* kr = p.cache.k_scratch + ((size_t)slot * g.nkv + kv) * g.scratch_rows * g.d;
            const __half* vr = p.cache.v_scratch + ((size_t)slot * g.nkv + kv) * g.scratch_rows * g.d;
            for (int s = 0; s < bnd.res_valid; ++s) {
                float part = 0.0f;
#pragma unroll
                for (int k = 0; k < kMaxBytesPerLane; ++k) {
                    int j = lane + 32 * k;
                    if (j < bytes_per_row) {
                        float2 x = __half22float2(reinterpret_cast<const __half2*>(kr + (size_t)s * g.d)[j]);
                        part += q0[k] * x.x + q1[k] * x.y;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                const float score = part * score_scale;
                const float m_new = fmaxf(m, score);
                const float corr = fast_exp2(m - m_new);
                const float pr = fast_exp2(score - m_new);
                l = l * corr + pr;
#pragma unroll
                for (int k = 0; k < kMaxBytesPerLane; ++k) {
                    int j = lane + 32 * k;
                    if (j < bytes_per_row) {
                        float2 x = __half22float2(reinterpret_cast<const __half2*>(vr + (size_t)s * g.d)[j]);
                        a0[k] = a0[k] * corr + pr * x.x;
                        a1[k] = a1[k] * corr + pr * x.y;
                    }
                }
                m = m_new;
            }
        }

        if (nchunks == 1) {
            const float inv_l = 1.0f / fmaxf(l, 1.0e-30f);
            const size_t oh = ((size_t)i * g.nh + h) * g.d;
#pragma unroll
            for (int k = 0; k < kMaxBytesPerLane; ++k) {
                int j = lane + 32 * k;
                if (j < bytes_per_row) {
                    store_out(p, oh + 2 * j, a0[k] * inv_l);
                    store_out(p, oh + 2 * j + 1, a1[k] * inv_l);
                }
            }
        } else {
            const size_t part_idx = (((size_t)i * g.nkv + kv) * p.max_chunks + chunk) * g.qpk + hq;
            float* po = p.ws_o + part_idx * g.d;
#pragma unroll
            for (int k = 0; k < kMaxBytesPerLane; ++k) {
                int j = lane + 32 * k;
                if (j < bytes_per_row) {
                    po[2 * j] = a0[k];
                    po[2 * j + 1] = a1[k];
                }
            }
            if (lane == 0) {
                p.ws_ml[part_idx * 2] = m;
                p.ws_ml[part_idx * 2 + 1] = l;
            }
        }
    }
}

}  // namespace

cudaError_t decode_generic_rejected(unsigned int* count) {
    return cudaMemcpyFromSymbol(count, g_generic_rejected, sizeof(unsigned int));
}

cudaError_t launch_decode_generic(const DecodeParams& p, cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    int warps = p.geom.qpk < 8 ? p.geom.qpk : 8;
    decode_generic_kernel<<<dim3(p.max_chunks, p.geom.nkv, p.n), warps * 32, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace kivi
