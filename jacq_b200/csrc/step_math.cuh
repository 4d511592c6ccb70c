// Element-wise arithmetic of the decode step shared by the stand-alone kernels (step.cu) and the
// GEMV prologues (gemv.cu). Expressions and reduction order follow the reference kernels
// (crates/jac-codegen-cuda/src/templates/kernels.cu) so that both forms give the reference's bits.
#pragma once
#include "kivi_common.cuh"
#include "p2p.cuh"

namespace kivi {

constexpr int kNormThreads = 256;   // the RMSNorm reduction order of the reference depends on this value

// 1 / rms of a row held in shared memory as fp16, by a CTA of kNormThreads threads (all must
// call): thread t sums elements t, t + 256, ...; xor-shuffle tree; warp totals added in order;
// rsqrtf(sum / n + eps)   (kernels.cu:10-31). `warp_sums` is shared scratch of 32 floats.
__device__ __forceinline__ float rms_scale(const __half* row, int hidden, float eps, float* warp_sums) {
    const int tid = threadIdx.x;
    float local = 0.0f;
    for (int i = tid; i < hidden; i += kNormThreads) {
        const float v = __half2float(row[i]);
        local += v * v;
    }
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    __syncthreads();   // a previous call's readers are done with warp_sums
    if ((tid & 31) == 0) warp_sums[tid >> 5] = local;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += warp_sums[w];
    return rsqrtf(total / hidden + eps);
}

// (x * scale) * w for eight fp16 values (kernels.cu:32).
__device__ __forceinline__ uint4 norm_apply8(const uint4& a, const uint4& w, float scale) {
    const __half* ah = reinterpret_cast<const __half*>(&a);
    const __half* wh = reinterpret_cast<const __half*>(&w);
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) oh[k] = __float2half(__half2float(ah[k]) * scale * __half2float(wh[k]));
    return o;
}

__device__ __forceinline__ uint4 hadd8(uint4 a, const uint4& d) {
    __half2* ah = reinterpret_cast<__half2*>(&a);
    const __half2* dh = reinterpret_cast<const __half2*>(&d);
#pragma unroll
    for (int k = 0; k < 4; ++k) ah[k] = __hadd2(ah[k], dh[k]);
    return a;
}

// One rotated pair of RoPE after the optional bias add (kernels.cu:40-54, :163-166): elements i and
// i + hd/2 of a head at position pos; freq = 1 / powf(base, (2 i) / hd), angle = pos * freq.
__device__ __forceinline__ void rope_pair(__half h0, __half h1, const __half* bias_head, int i, int hd, int pos,
                                          float rope_base, __half* out_head) {
    const int half_dim = hd >> 1;
    const float freq = 1.0f / powf(rope_base, (2.0f * i) / hd);
    const float ang = pos * freq;
    const float c = cosf(ang), s = sinf(ang);
    if (bias_head) { h0 = __hadd(h0, bias_head[i]); h1 = __hadd(h1, bias_head[i + half_dim]); }
    const float x0 = __half2float(h0), x1 = __half2float(h1);
    out_head[i] = __float2half(x0 * c - x1 * s);
    out_head[i + half_dim] = __float2half(x1 * c + x0 * s);
}

// Input of the fused RoPE + cache-write kernel (cache_write.cu): one qkv row per sequence.
struct RopeParams {
    const __half* qkv;      // [n, (NH + 2 NKV) * D]
    const __half* bias;     // [(NH + 2 NKV) * D] or nullptr
    const int* positions;   // [n]
    __half* q;              // [n, NH, D]
    __half* k;              // [n, NKV, D]: the writer's new_k
    __half* v;              // [n, NKV, D]: the writer's new_v
    float rope_base;
};

// SiLU(gate) * up for one pair (kernels.cu:146-153).
__device__ __forceinline__ __half silu_mul1(__half g, __half u) {
    const float gv = __half2float(g);
    const float sv = gv / (1.0f + expf(-gv));
    return __float2half(sv * __half2float(u));
}

// SiLU(gate) * up for eight fp16 values: g / (1 + expf(-g)) * up   (kernels.cu:146-153).
__device__ __forceinline__ uint4 silu_mul8(const uint4& g, const uint4& u) {
    const __half* gh = reinterpret_cast<const __half*>(&g);
    const __half* uh = reinterpret_cast<const __half*>(&u);
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float gv = __half2float(gh[k]);
        const float sv = gv / (1.0f + expf(-gv));
        oh[k] = __float2half(sv * __half2float(uh[k]));
    }
    return o;
}

// What a GEMV does to its input rows before the product.
// kGemvAddNormSiluOut: the add+norm prologue with a SwiGLU epilogue for the fused gate|up matrix: the warp
// that owns gate row i also owns up row i (i + out_dim) and stores SiLU(gate_i) * up_i, so the product
// never exists unfused and the down projection reads its input as is.
enum GemvPrologueKind { kGemvPlain = 0, kGemvAddNorm = 1, kGemvAddNormSiluOut = 2 };
struct GemvPrologue {
    const __half* x;        // plain: [batch, in]; add+norm: residual rows (or a table with `tokens`)
    const int* tokens;      // add+norm: optional row gather (embedding lookup)
    const __half* delta;    // add+norm: optional [batch, in] added first
    P2pGather gather;       // add+norm: when gather.tp > 0 the delta is the sum of the ranks' slots of that site instead
    P2pPush push;           // any kind: when push.tp > 0 the result goes to every rank's slot of that site (fp16 pairs)
    const __half* weight;   // add+norm: [in]
    __half* x_out;          // add+norm: optional [batch, in], the updated residual rows (written once)
    float eps;
};

}  // namespace kivi
