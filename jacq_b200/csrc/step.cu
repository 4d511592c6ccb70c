// Decode step of the generated runtime around the KIVI cache: the element-wise kernels between
// the projections and the host loop that strings one step together.
//
// Reference: forward() in crates/jac-codegen-cuda/src/templates/runtime.cu:125-187 and its kernels
// in templates/kernels.cu. The reference runs one token per step with <<<1,256>>>-style launches;
// here a step carries `batch` sequences, every kernel takes one row per sequence, the residual add
// is fused into the RMSNorm that follows it, bias add and the q/k/v split into RoPE, and the fp16
// KV store plus three attention kernels are replaced by the int4-KIVI writer and paged decode.
//
// The arithmetic of each element keeps the reference's expression and order, so the results are
// bit-identical to the reference kernels on the same GPU (RoPE: up to a handful of elements per
// ten thousand one fp16 ulp away at positions in the thousands, where the reference's compile-time
// ROPE_BASE lets the compiler fold part of powf):
//   RMSNorm   thread t of 256 sums elements t, t+256, ...; xor-shuffle tree; warp totals added in
//             order; scale = rsqrtf(sum / n + eps); out = (x * scale) * w        (kernels.cu:10-33)
//   RoPE      freq = 1 / powf(base, (2 i) / HD); ang = pos * freq; rotate pair (i, i + HD/2)
//                                                                                (kernels.cu:40-54)
//   SiLU*up   g / (1 + expf(-g)) * up                                            (kernels.cu:146-153)
//   add, bias fp16 __hadd                                                        (kernels.cu:156-166)
#include "kivi_common.cuh"
#include "step_math.cuh"

namespace kivi {
namespace {

// x_out = x (+ delta); normed = RMSNorm(x_out) * weight. One CTA per row. `tokens` (optional)
// makes row i of x the embedding row tokens[i] (kernels.cu:4-7).
__global__ void __launch_bounds__(kNormThreads) residual_rmsnorm_kernel(
    const __half* __restrict__ x, const int* __restrict__ tokens, const __half* __restrict__ delta,
    const __half* __restrict__ weight, __half* __restrict__ x_out, __half* __restrict__ normed, int hidden, float eps,
    const P2pGather gather) {
    extern __shared__ __align__(16) unsigned char step_smem[];
    uint4* row = reinterpret_cast<uint4*>(step_smem);
    __shared__ float warp_sums[32];
    const int tid = threadIdx.x;
    pdl_trigger();
    const bool gathered = gather.tp > 0;
    P2pView view = {};
    if (gathered) view = p2p_view(gather);
    const size_t src_row = tokens ? (size_t)tokens[blockIdx.x] : (size_t)blockIdx.x;
    const uint4* xs = reinterpret_cast<const uint4*>(x + src_row * hidden);
    const uint4* ds = delta ? reinterpret_cast<const uint4*>(delta + (size_t)blockIdx.x * hidden) : nullptr;
    uint4* xo = x_out ? reinterpret_cast<uint4*>(x_out + (size_t)blockIdx.x * hidden) : nullptr;
    const int vecs = hidden >> 3;
    for (int v = tid; v < vecs; v += kNormThreads) {
        uint4 a = xs[v];
        if (gathered) a = hadd8(a, p2p_sum8<4>(view, (size_t)blockIdx.x * vecs + v));   // nothing else lives in registers here
        else if (ds) a = hadd8(a, ds[v]);
        if (xo) xo[v] = a;
        row[v] = a;
    }
    __syncthreads();
    const float scale = rms_scale(reinterpret_cast<const __half*>(row), hidden, eps, warp_sums);
    uint4* no = reinterpret_cast<uint4*>(normed + (size_t)blockIdx.x * hidden);
    const uint4* wv = reinterpret_cast<const uint4*>(weight);
    for (int v = tid; v < vecs; v += kNormThreads) no[v] = norm_apply8(row[v], wv[v], scale);
}

// qkv row [q heads | k heads | v heads] (+ bias) -> q and k rotated at positions[row], v copied.
// One CTA per (row, head), one thread per rotated pair, like the reference's launch
// (<<<NH + NKV, 64>>>, runtime.cu:159) with the value heads added.
__global__ void __launch_bounds__(128) bias_rope_kernel(
    const __half* __restrict__ qkv, const __half* __restrict__ bias, const int* __restrict__ positions,
    __half* __restrict__ q, __half* __restrict__ k, __half* __restrict__ v, int nh, int nkv, int hd, float rope_base) {
    const int rowi = blockIdx.y, h = blockIdx.x;
    const int half_dim = hd >> 1;
    pdl_trigger();
    pdl_wait();   // the projection that wrote qkv
    const __half* in = qkv + (size_t)rowi * (nh + 2 * nkv) * hd + (size_t)h * hd;
    const __half* bh = bias ? bias + (size_t)h * hd : nullptr;
    if (h >= nh + nkv) {   // a value head: bias add only
        __half* out = v + ((size_t)rowi * nkv + (h - nh - nkv)) * hd;
        for (int e = threadIdx.x; e < hd; e += blockDim.x) out[e] = bh ? __hadd(in[e], bh[e]) : in[e];
        return;
    }
    const int pos = positions[rowi];
    __half* out = h < nh ? q + ((size_t)rowi * nh + h) * hd : k + ((size_t)rowi * nkv + (h - nh)) * hd;
    for (int i = threadIdx.x; i < half_dim; i += blockDim.x) rope_pair(in[i], in[i + half_dim], bh, i, hd, pos, rope_base, out);
}

// out[row, i] = SiLU(gate_up[row, i]) * gate_up[row, ffn + i]; eight elements per thread.
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* __restrict__ gate_up, __half* __restrict__ out,
                                                        int ffn) {
    const int rowi = blockIdx.y;
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    if (v >= (ffn >> 3)) return;
    const uint4* row = reinterpret_cast<const uint4*>(gate_up + (size_t)rowi * 2 * ffn);
    reinterpret_cast<uint4*>(out + (size_t)rowi * ffn)[v] = silu_mul8(row[v], row[(ffn >> 3) + v]);
}

// Arg-max, first pass: block (chunk, row) scans its slice of the row. A candidate is (value, index);
// the larger value wins, the lower index on a tie, and nothing at or below -1e30 (or NaN) beats the
// initial (-1e30, 0) of kernels.cu:208-209.
constexpr int kArgmaxThreads = 256;
constexpr int kArgmaxChunk = 8192;

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(kArgmaxThreads) argmax_partial_kernel(
    const __half* __restrict__ logits, int n, int index_offset, float* __restrict__ part_val, int* __restrict__ part_idx) {
    __shared__ float s_val[kArgmaxThreads / 32];
    __shared__ int s_idx[kArgmaxThreads / 32];
    const int rowi = blockIdx.y;
    const __half* in = logits + (size_t)rowi * n;
    const int lo = blockIdx.x * kArgmaxChunk, hi = min(n, lo + kArgmaxChunk);
    float best = -1e30f;
    int best_i = 0;
    for (int i = lo + threadIdx.x; i < hi; i += kArgmaxThreads) {
        const float v = __half2float(in[i]);
        if (v > best) { best = v; best_i = i; }
    }
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kArgmaxThreads / 32; ++w)
            if (better(s_val[w], s_idx[w], best, best_i)) { best = s_val[w]; best_i = s_idx[w]; }
        part_val[(size_t)rowi * gridDim.x + blockIdx.x] = best;
        // a slice with no candidate above the floor reports global index 0, like the reference
        part_idx[(size_t)rowi * gridDim.x + blockIdx.x] = best > -1e30f ? best_i + index_offset : 0;
    }
}

// Second pass: one warp per row over the candidates of every rank. Rank r's candidates start at
// base + r * rank_stride: [rows][chunks] values, then at idx_off [rows][chunks] indices. With
// gather.tp > 0 the candidates are the ranks' slots of that exchange site (payload words in the same
// order, read through the exchange).
__global__ void argmax_merge_kernel(const unsigned char* __restrict__ base, size_t rank_stride, size_t idx_off, int chunks,
                                    int ranks, int rows, int* __restrict__ out, const P2pGather gather) {
    const bool gathered = gather.tp > 0;
    P2pView view = {};
    if (gathered) view = p2p_view(gather);
    const int rowi = blockIdx.x;
    float best = -1e30f;
    int best_i = 0;
    const int total = chunks * ranks;
    for (int e = threadIdx.x; e < total; e += 32) {
        const int rk = e / chunks, ch = e - rk * chunks;
        const size_t at = (size_t)rowi * chunks + ch;
        float v;
        int i;
        if (gathered) {
            const size_t wv = at, wi = idx_off / 4 + at;   // payload word numbers of the value and of the index
            const uint2 pv = p2p_read2(view, rk, wv >> 1), pi = p2p_read2(view, rk, wi >> 1);
            v = __uint_as_float((wv & 1) ? pv.y : pv.x);
            i = (int)((wi & 1) ? pi.y : pi.x);
        } else {
            const unsigned char* rb = base + (size_t)rk * rank_stride;
            v = __ldcg(reinterpret_cast<const float*>(rb) + at);
            i = __ldcg(reinterpret_cast<const int*>(rb + idx_off) + at);
        }
        if (better(v, i, best, best_i)) { best = v; best_i = i; }
    }
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) out[rowi] = best_i;
}

// Bookkeeping of a step: the decode sees the lengths after the append, the writer those before it.
__global__ void step_begin_kernel(const int* __restrict__ seq_lens, int* __restrict__ lens_after, int n,
                                  P2pHeader* header) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) lens_after[i] = seq_lens[i] + 1;
    if (header && i == 0) header->step_no += 1u;   // the exchanges of this step carry this number
}
__global__ void step_end_kernel(int* __restrict__ seq_lens, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) seq_lens[i] += 1;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
const __half* H(const kivi_f16* p) { return reinterpret_cast<const __half*>(p); }
__half* H(kivi_f16* p) { return reinterpret_cast<__half*>(p); }

int ok(cudaError_t e) { return e == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA; }

int launch_residual_rmsnorm(const __half* x, const int* tokens, const __half* delta, const __half* weight,
                            __half* x_out, __half* normed, int batch, int hidden, float eps, const P2pGather& gather,
                            cudaStream_t stream) {
    const size_t smem = (size_t)hidden * sizeof(__half);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(residual_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return KIVI_ERR_CUDA;
    }
    residual_rmsnorm_kernel<<<batch, kNormThreads, smem, stream>>>(x, tokens, delta, weight, x_out, normed, hidden, eps,
                                                                   gather);
    return ok(cudaGetLastError());
}

int launch_bias_rope(const __half* qkv, const __half* bias, const int* positions, __half* q, __half* k, __half* v,
                     int batch, int nh, int nkv, int hd, float rope_base, cudaStream_t stream) {
    const int threads = hd / 2 <= 32 ? 32 : (hd / 2 <= 64 ? 64 : 128);
    return ok(launch_pdl(bias_rope_kernel, dim3(nh + 2 * nkv, batch), dim3(threads), 0, stream, qkv, bias, positions, q, k, v,
                         nh, nkv, hd, rope_base));
}

int launch_silu_mul(const __half* gate_up, __half* out, int batch, int ffn, cudaStream_t stream) {
    silu_mul_kernel<<<dim3(((ffn >> 3) + 255) / 256, batch), 256, 0, stream>>>(gate_up, out, ffn);
    return ok(cudaGetLastError());
}

int argmax_chunks(int n) { return (n + kArgmaxChunk - 1) / kArgmaxChunk; }
size_t argmax_payload_bytes(int batch, int vocab) {
    return ((size_t)batch * argmax_chunks(vocab) * (sizeof(float) + sizeof(int)) + 15) / 16 * 16;
}

// Projection y[b, :] = W x[b, :]. `push` (tensor parallel over peer memory, may be nullptr): the result is
// a partial sum that every rank needs; the GEMV and the skinny GEMM deliver it from their own epilogue
// (the copy kernel covers shapes neither can).
int project(const __half* w, const __half* x, __half* y, int out_dim, int in_dim, int batch, cudaStream_t stream,
            const P2pPush* push = nullptr) {
    if (batch <= 4) {
        GemvPrologue pro = {};
        pro.x = x;
        if (push) pro.push = *push;
        return ok(launch_gemv_fused(w, kGemvPlain, pro, y, nullptr, out_dim, in_dim, batch, stream));
    }
    if (skinny_gemm_supports(in_dim, batch) && (!push || out_dim % 4 == 0))   // delivers from its own epilogue too
        return ok(launch_skinny_gemm(w, x, y, nullptr, out_dim, in_dim, batch, stream, push));
    int rc = skinny_gemm_supports(in_dim, batch) ? ok(launch_skinny_gemm(w, x, y, nullptr, out_dim, in_dim, batch, stream))
                                                 : ok(launch_gemv(w, x, y, nullptr, out_dim, in_dim, batch, stream));
    if (rc == KIVI_OK && push) rc = ok(launch_p2p_push(y, (size_t)batch * out_dim * sizeof(__half), *push, stream));
    return rc;
}

// KIVI_STEP_FUSED_WRITE=0 in the environment runs RoPE and the cache write as their three separate
// kernels instead of the fused one (a tuning switch; same results).
bool fused_rope_write() {
    static const bool on = [] { const char* e = getenv("KIVI_STEP_FUSED_WRITE"); return !e || atoi(e) != 0; }();
    return on;
}

// Up to four sequences: the step's element-wise kernels ride in the prologue of the GEMV that
// consumes them (one launch instead of two, and the weights start streaming before the input is
// ready). Larger batches run the stand-alone kernel and then the skinny GEMM.
bool fuse_prologues(int batch) { return batch <= 4; }

// y = W RMSNorm(x (+ delta)); the updated residual rows go to x_out.
// swiglu_rows > 0: w is a fused gate|up matrix of 2 * swiglu_rows rows and y receives SiLU(gate) * up
// [batch, swiglu_rows] (small batches only; the caller checks fuse_prologues()).
int project_add_norm(const __half* w, const __half* x, const int* tokens, const __half* delta, const P2pGather& gather,
                     const __half* weight, __half* x_out, __half* normed_scratch, __half* y, int out_dim, int hidden,
                     int batch, float eps, cudaStream_t stream, int swiglu_rows = 0) {
    if (fuse_prologues(batch)) {
        GemvPrologue pro = {};
        pro.x = x; pro.tokens = tokens; pro.delta = delta; pro.gather = gather; pro.weight = weight; pro.x_out = x_out;
        pro.eps = eps;
        if (swiglu_rows > 0)
            return ok(launch_gemv_fused(w, kGemvAddNormSiluOut, pro, y, nullptr, swiglu_rows, hidden, batch, stream));
        return ok(launch_gemv_fused(w, kGemvAddNorm, pro, y, nullptr, out_dim, hidden, batch, stream));
    }
    const int rc = launch_residual_rmsnorm(x, tokens, delta, weight, x_out, normed_scratch, batch, hidden, eps, gather,
                                           stream);
    return rc != KIVI_OK ? rc : project(w, normed_scratch, y, out_dim, hidden, batch, stream);
}

// y = W (SiLU(gate) * up) for rows [gate | up], larger batches: the stand-alone kernel, then the projection.
int project_silu_mul(const __half* w, const __half* gate_up, __half* mid_scratch, __half* y, int out_dim, int ffn,
                     int batch, cudaStream_t stream, const P2pPush* push = nullptr) {
    const int rc = launch_silu_mul(gate_up, mid_scratch, batch, ffn, stream);
    return rc != KIVI_OK ? rc : project(w, mid_scratch, y, out_dim, ffn, batch, stream, push);
}

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

struct StepLayout {
    size_t x0, x1, normed, qkv, q, k, v, attn, proj, gate_up, mid, logits, lens_after, parts, gathered, decode_ws, total;
    size_t decode_ws_bytes, parts_bytes;
};

int qkv_rows(const kivi_step_config& c) { return (c.num_q_heads + 2 * c.num_kv_heads) * c.head_dim; }

StepLayout step_layout(const kivi_step_config& c, const Geom& g, int batch, int max_seq_len) {
    StepLayout L;
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t o = at; at += up256(bytes); return o; };
    const size_t n = (size_t)batch, h2 = sizeof(__half);
    const int tp = c.tp_size > 1 ? c.tp_size : 1;
    L.decode_ws_bytes = decode_workspace_total(g, batch, split_old(max_seq_len, g.r, g.g));
    L.decode_ws = take(L.decode_ws_bytes);
    L.x0 = take(n * c.hidden * h2);
    L.x1 = take(n * c.hidden * h2);
    L.normed = take(n * c.hidden * h2);
    L.qkv = take(n * qkv_rows(c) * h2);
    L.q = take(n * c.num_q_heads * c.head_dim * h2);
    L.k = take(n * c.num_kv_heads * c.head_dim * h2);
    L.v = take(n * c.num_kv_heads * c.head_dim * h2);
    L.attn = take(n * c.num_q_heads * c.head_dim * h2);
    L.proj = take(n * c.hidden * h2);
    L.gate_up = take(n * 2 * c.ffn * h2);
    L.mid = take(n * c.ffn * h2);
    L.logits = take(n * c.vocab * h2);
    L.lens_after = take(n * sizeof(int));
    L.parts_bytes = argmax_payload_bytes(batch, c.vocab);   // [values | indices] of this rank's arg-max candidates
    L.parts = take(L.parts_bytes);
    L.gathered = take(L.parts_bytes * tp);
    L.total = at;
    return L;
}

// Largest payload one rank delivers at an exchange site: a projection [batch, H] or its arg-max candidates.
size_t step_exchange_payload(const kivi_step_config& c, int batch) {
    const size_t proj = (size_t)batch * c.hidden * sizeof(__half);
    const size_t cand = argmax_payload_bytes(batch, c.vocab);
    return proj > cand ? proj : cand;
}

int check_step_config(const kivi_step_config* c) {
    if (!c) return KIVI_ERR_NULL_POINTER;
    if (c->layers <= 0 || c->hidden <= 0 || c->num_q_heads <= 0 || c->num_kv_heads <= 0 || c->head_dim <= 0 ||
        c->ffn <= 0 || c->vocab <= 0 || c->vocab_offset < 0)
        return KIVI_ERR_GEOMETRY;
    if (c->hidden % 8 || c->ffn % 8 || c->head_dim % 8) return KIVI_ERR_GEOMETRY;   // 16-byte rows everywhere
    if (c->num_q_heads % c->num_kv_heads) return KIVI_ERR_GEOMETRY;
    if (c->head_dim / 2 > 256) return KIVI_ERR_GEOMETRY;
    if (c->tp_size < 1 || c->tp_rank < 0 || c->tp_rank >= c->tp_size) return KIVI_ERR_GEOMETRY;
    if (!(c->rope_base > 0.0f) || !(c->norm_eps >= 0.0f)) return KIVI_ERR_GEOMETRY;
    return KIVI_OK;
}

kivi_geometry step_geometry(const kivi_step_config& c) {
    kivi_geometry s = {c.num_q_heads, c.num_kv_heads, c.head_dim, c.block_size, c.group_size, c.residual};
    return s;
}

CachePtrs to_ptrs(const kivi_cache& c) {
    CachePtrs o;
    o.k_code = c.k_code_pages;
    o.k_scale = reinterpret_cast<__half*>(c.k_scale_pages);
    o.k_zero = reinterpret_cast<__half*>(c.k_zero_pages);
    o.v_code = c.v_code_pages;
    o.v_scale = reinterpret_cast<__half*>(c.v_scale_pages);
    o.v_zero = reinterpret_cast<__half*>(c.v_zero_pages);
    o.k_scratch = reinterpret_cast<__half*>(c.k_residual_scratch);
    o.v_scratch = reinterpret_cast<__half*>(c.v_residual_scratch);
    o.num_blocks = c.num_blocks; o.num_slots = c.num_slots;
    return o;
}

}  // namespace
}  // namespace kivi

using namespace kivi;

extern "C" size_t kivi_b200_decode_step_workspace_bytes(const kivi_step_config* cfg, int batch, int max_seq_len) {
    if (check_step_config(cfg) != KIVI_OK || batch <= 0 || batch > 64 || max_seq_len < 1) return 0;
    kivi_geometry gs = step_geometry(*cfg);
    if (kivi_b200_validate_geometry(&gs, nullptr) != KIVI_OK) return 0;
    return step_layout(*cfg, make_geom(gs), batch, max_seq_len).total;
}

extern "C" size_t kivi_b200_p2p_region_bytes(const kivi_step_config* cfg, int batch) {
    if (check_step_config(cfg) != KIVI_OK || batch <= 0 || batch > 64 || cfg->tp_size > kMaxTp) return 0;
    return p2p_layout(cfg->tp_size, 2 * cfg->layers + 1, step_exchange_payload(*cfg, batch)).total;
}

extern "C" int kivi_b200_decode_step(const kivi_step_config* cfg, const kivi_step_weights* weights,
                                     const kivi_step_state* state, const int32_t* tokens_in, int batch, int max_seq_len,
                                     int32_t* tokens_out, kivi_f16* logits_out, const kivi_step_comm* comm,
                                     cudaStream_t stream) {
    int rc = check_step_config(cfg);
    if (rc != KIVI_OK) return rc;
    if (!weights || !state || !tokens_in || !tokens_out) return KIVI_ERR_NULL_POINTER;
    if (!weights->embed || !weights->final_norm || !weights->lm_head || !weights->layers) return KIVI_ERR_NULL_POINTER;
    if (!state->caches || !state->block_tables || !state->seq_lens) return KIVI_ERR_NULL_POINTER;
    if (batch < 1 || batch > 64 || max_seq_len < 1 || max_seq_len > 0x3fffffff) return KIVI_ERR_RANGE;
    const kivi_step_config& c = *cfg;
    const bool tp = c.tp_size > 1;
    if (tp && !comm) return KIVI_ERR_NULL_POINTER;
    const bool p2p = tp && comm->peer_regions != nullptr;
    if (tp && !p2p && (!comm->allreduce_f16 || !comm->allgather)) return KIVI_ERR_NULL_POINTER;
    if (p2p && (c.tp_size > kMaxTp || c.hidden % 2)) return KIVI_ERR_GEOMETRY;
    kivi_geometry gs = step_geometry(c);
    rc = kivi_b200_validate_geometry(&gs, nullptr);
    if (rc != KIVI_OK) return rc;
    const Geom g = make_geom(gs);
    if ((long long)split_old(max_seq_len, g.r, g.g) > (long long)state->max_blocks_per_seq * g.b)
        return KIVI_ERR_BLOCK_TABLE;
    const StepLayout L = step_layout(c, g, batch, max_seq_len);
    if (!state->workspace || state->workspace_bytes < L.total) return KIVI_ERR_WORKSPACE;
    if (!aligned16(state->workspace)) return KIVI_ERR_ALIGNMENT;
    for (int l = 0; l < c.layers; ++l) {
        const kivi_layer_weights& lw = weights->layers[l];
        if (!lw.attn_norm || !lw.qkv || !lw.o || !lw.ffn_norm || !lw.gate_up || !lw.down) return KIVI_ERR_NULL_POINTER;
        if (c.attn_bias && !lw.qkv_bias) return KIVI_ERR_NULL_POINTER;
        if (!state->caches[l].k_code_pages || !state->caches[l].k_residual_scratch) return KIVI_ERR_NULL_POINTER;
        if (!state->slot_ids && batch > state->caches[l].num_slots) return KIVI_ERR_RANGE;
    }

    unsigned char* ws = static_cast<unsigned char*>(state->workspace);
    auto hp = [&](size_t off) { return reinterpret_cast<__half*>(ws + off); };
    __half *x_cur = hp(L.x0), *x_nxt = hp(L.x1);
    __half *normed = hp(L.normed), *qkv = hp(L.qkv), *q = hp(L.q), *k = hp(L.k), *v = hp(L.v), *attn = hp(L.attn);
    __half *proj = hp(L.proj), *gate_up = hp(L.gate_up), *mid = hp(L.mid);
    __half* logits = logits_out ? H(logits_out) : hp(L.logits);
    int* lens_after = reinterpret_cast<int*>(ws + L.lens_after);
    void* decode_ws = L.decode_ws_bytes ? ws + L.decode_ws : nullptr;
    const int q_dim = c.num_q_heads * c.head_dim;
    const int max_old = split_old(max_seq_len, g.r, g.g);

#define KIVI_STEP_TRY(expr) do { const int rc__ = (expr); if (rc__ != KIVI_OK) return rc__; } while (0)

    // ---- exchange between ranks: sites 2l (after o_proj), 2l + 1 (after down_proj), 2L (arg-max) ----
    const P2pLayout pl = p2p_layout(c.tp_size, 2 * c.layers + 1, step_exchange_payload(c, batch));
    unsigned char* own = p2p ? static_cast<unsigned char*>(comm->peer_regions[c.tp_rank]) : nullptr;
    if (p2p) {
        if (comm->region_bytes < pl.total) return KIVI_ERR_WORKSPACE;
        for (int r = 0; r < c.tp_size; ++r)
            if (!comm->peer_regions[r] || !aligned16(comm->peer_regions[r])) return KIVI_ERR_NULL_POINTER;
    }
    P2pHeader* header = reinterpret_cast<P2pHeader*>(own);
    const int sites = 2 * c.layers + 1;
    auto gather_at = [&](int site) {
        P2pGather ga = {};
        if (!p2p) return ga;            // tp = 0: the consumer reads its plain local input
        ga.header = header;
        ga.status = &header->status;
        ga.slots = own + pl.slots_off;
        ga.slot_bytes = pl.slot_bytes;
        ga.tp = c.tp_size;
        ga.site = site;
        ga.sites = sites;
        ga.spin_limit = comm->spin_limit ? comm->spin_limit : kP2pSpinLimit;
        return ga;
    };
    auto push_at = [&](int site) {
        P2pPush ps = {};
        for (int r = 0; r < c.tp_size; ++r)
            ps.slot[r] = static_cast<unsigned char*>(comm->peer_regions[r]) + pl.slots_off + (size_t)c.tp_rank * pl.slot_bytes;
        ps.header = header;
        ps.half_stride = (size_t)c.tp_size * pl.slot_bytes;
        ps.tp = c.tp_size;
        ps.site = site;
        ps.sites = sites;
        return ps;
    };
    // all-reduce through the hooks: in place, now (peer memory delivers from the projection itself and sums
    // in the consumer)
    auto allreduce_hook = [&](__half* buf, size_t bytes) -> int {
        if (!tp || p2p) return KIVI_OK;
        return comm->allreduce_f16(comm->user, reinterpret_cast<kivi_f16*>(buf), bytes / 2, stream) ? KIVI_ERR_CUDA : KIVI_OK;
    };
    const size_t proj_bytes = (size_t)batch * c.hidden * sizeof(__half);

    step_begin_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(state->seq_lens, lens_after, batch, p2p ? header : nullptr);
    KIVI_STEP_TRY(ok(cudaGetLastError()));

    SeqAddressing wa;   // writer: lengths before the append
    wa.seq_lens = state->seq_lens; wa.seq_len_scalar = 0;
    wa.block_tables = state->block_tables; wa.bt_stride = state->max_blocks_per_seq; wa.bt_width = state->max_blocks_per_seq;
    wa.slot_ids = state->slot_ids; wa.slot_shared = 0;
    SeqAddressing da = wa;   // decode: lengths after it
    da.seq_lens = lens_after;

    const __half* delta = nullptr;           // projection waiting to be added to the residual stream
    int delta_site = -1;                     // ... and, with peer memory, the exchange site its partials went to
    const int* embed_tokens = tokens_in;     // layer 0 reads its rows from the embedding table
    for (int l = 0; l < c.layers; ++l) {
        const kivi_layer_weights& lw = weights->layers[l];
        // attention block
        KIVI_STEP_TRY(project_add_norm(H(lw.qkv), embed_tokens ? H(weights->embed) : x_cur, embed_tokens, delta,
                                       delta_site >= 0 ? gather_at(delta_site) : P2pGather{}, H(lw.attn_norm), x_nxt,
                                       normed, qkv, qkv_rows(c), c.hidden, batch, c.norm_eps, stream));
        embed_tokens = nullptr;
        { __half* t = x_cur; x_cur = x_nxt; x_nxt = t; }
        // bias + RoPE + split and the cache write of the new token: one launch, one CTA per (kv head, sequence)
        WriteParams wp;
        wp.geom = g; wp.cache = to_ptrs(state->caches[l]); wp.seq = wa;
        wp.new_k = k; wp.new_v = v; wp.new_offsets = nullptr; wp.num_new_scalar = 1; wp.n = batch;   // row i = sequence i
        if (fused_rope_write()) {
            RopeParams rp = {qkv, c.attn_bias ? H(lw.qkv_bias) : nullptr, state->seq_lens, q, k, v, c.rope_base};
            KIVI_STEP_TRY(ok(launch_rope_write(rp, wp, stream)));
        } else {
            KIVI_STEP_TRY(launch_bias_rope(qkv, c.attn_bias ? H(lw.qkv_bias) : nullptr, state->seq_lens, q, k, v, batch,
                                           c.num_q_heads, c.num_kv_heads, c.head_dim, c.rope_base, stream));
            KIVI_STEP_TRY(ok(launch_cache_write(wp, 1, stream)));
        }
        KIVI_STEP_TRY(run_decode(g, wp.cache, da, q, nullptr, attn, batch, max_seq_len, max_old, -1, decode_ws,
                                 L.decode_ws_bytes, stream));
        P2pPush push_o = p2p ? push_at(2 * l) : P2pPush{};
        KIVI_STEP_TRY(project(H(lw.o), attn, proj, c.hidden, q_dim, batch, stream, p2p ? &push_o : nullptr));
        KIVI_STEP_TRY(allreduce_hook(proj, proj_bytes));
        // feed-forward block
        const bool swiglu_in_epilogue = fuse_prologues(batch);   // the gate_up GEMV then writes SiLU(gate) * up itself
        KIVI_STEP_TRY(project_add_norm(H(lw.gate_up), x_cur, nullptr, proj, gather_at(2 * l), H(lw.ffn_norm), x_nxt,
                                       normed, swiglu_in_epilogue ? mid : gate_up, 2 * c.ffn, c.hidden, batch, c.norm_eps,
                                       stream, swiglu_in_epilogue ? c.ffn : 0));
        { __half* t = x_cur; x_cur = x_nxt; x_nxt = t; }
        // the down projection must not overwrite `proj` while a gate_up CTA may still read it as delta:
        // it cannot, every gate_up CTA has finished its prologue before the first down CTA passes its wait
        P2pPush push_down = p2p ? push_at(2 * l + 1) : P2pPush{};
        if (swiglu_in_epilogue)
            KIVI_STEP_TRY(project(H(lw.down), mid, proj, c.hidden, c.ffn, batch, stream, p2p ? &push_down : nullptr));
        else
            KIVI_STEP_TRY(project_silu_mul(H(lw.down), gate_up, mid, proj, c.hidden, c.ffn, batch, stream,
                                           p2p ? &push_down : nullptr));
        KIVI_STEP_TRY(allreduce_hook(proj, proj_bytes));
        delta = proj;
        delta_site = p2p ? 2 * l + 1 : -1;
    }
    KIVI_STEP_TRY(project_add_norm(H(weights->lm_head), x_cur, nullptr, delta,
                                   delta_site >= 0 ? gather_at(delta_site) : P2pGather{}, H(weights->final_norm), x_nxt,
                                   normed, logits, c.vocab, c.hidden, batch, c.norm_eps, stream));

    // arg-max: candidates per 8192-entry slice on every rank, [values | indices]; the ranks' candidates meet
    // through the hook's all-gather or through the last exchange site, and every rank picks the same winner
    const int chunks = argmax_chunks(c.vocab);
    unsigned char* parts = ws + L.parts;
    const size_t idx_off = (size_t)batch * chunks * sizeof(float);
    argmax_partial_kernel<<<dim3(chunks, batch), kArgmaxThreads, 0, stream>>>(
        logits, c.vocab, c.vocab_offset, reinterpret_cast<float*>(parts), reinterpret_cast<int*>(parts + idx_off));
    KIVI_STEP_TRY(ok(cudaGetLastError()));
    const unsigned char* cand = parts;
    size_t rank_stride = 0;
    P2pGather cand_gather = {};
    if (p2p) {
        const P2pPush push_cand = push_at(2 * c.layers);
        KIVI_STEP_TRY(ok(launch_p2p_push(parts, L.parts_bytes, push_cand, stream)));
        cand_gather = gather_at(2 * c.layers);
        rank_stride = pl.slot_bytes;
    } else if (tp) {
        unsigned char* gathered = ws + L.gathered;
        if (comm->allgather(comm->user, parts, gathered, L.parts_bytes, stream)) return KIVI_ERR_CUDA;
        cand = gathered;
        rank_stride = L.parts_bytes;
    }
    argmax_merge_kernel<<<batch, 32, 0, stream>>>(cand, rank_stride, idx_off, chunks, tp ? c.tp_size : 1, batch, tokens_out,
                                                  cand_gather);
    KIVI_STEP_TRY(ok(cudaGetLastError()));
    step_end_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(state->seq_lens, batch);
    return ok(cudaGetLastError());
#undef KIVI_STEP_TRY
}

extern "C" int kivi_b200_residual_rmsnorm(const kivi_f16* x, const kivi_f16* delta, const kivi_f16* weight,
                                          kivi_f16* x_out, kivi_f16* normed, int batch, int hidden, float eps,
                                          cudaStream_t stream) {
    if (!x || !weight || !normed) return KIVI_ERR_NULL_POINTER;
    if (batch < 0 || hidden <= 0 || hidden % 8 || (size_t)hidden * 2 > 200 * 1024) return KIVI_ERR_RANGE;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(normed) || (delta && !aligned16(delta)) ||
        (x_out && !aligned16(x_out)))
        return KIVI_ERR_ALIGNMENT;
    if (batch == 0) return KIVI_OK;
    return launch_residual_rmsnorm(H(x), nullptr, delta ? H(delta) : nullptr, H(weight), x_out ? H(x_out) : nullptr,
                                   H(normed), batch, hidden, eps, P2pGather{}, stream);
}

extern "C" int kivi_b200_bias_rope(const kivi_f16* qkv, const kivi_f16* bias, const int32_t* positions, kivi_f16* q,
                                   kivi_f16* k, kivi_f16* v, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                   float rope_base, cudaStream_t stream) {
    if (!qkv || !positions || !q || !k || !v) return KIVI_ERR_NULL_POINTER;
    if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || head_dim % 2 || head_dim / 2 > 256)
        return KIVI_ERR_RANGE;
    if (batch == 0) return KIVI_OK;
    return launch_bias_rope(H(qkv), bias ? H(bias) : nullptr, positions, H(q), H(k), H(v), batch, num_q_heads,
                            num_kv_heads, head_dim, rope_base, stream);
}

extern "C" int kivi_b200_silu_mul(const kivi_f16* gate_up, kivi_f16* out, int batch, int ffn, cudaStream_t stream) {
    if (!gate_up || !out) return KIVI_ERR_NULL_POINTER;
    if (batch < 0 || ffn <= 0 || ffn % 8) return KIVI_ERR_RANGE;
    if (!aligned16(gate_up) || !aligned16(out)) return KIVI_ERR_ALIGNMENT;
    if (batch == 0) return KIVI_OK;
    return launch_silu_mul(H(gate_up), H(out), batch, ffn, stream);
}

extern "C" int kivi_b200_argmax(const kivi_f16* logits, int32_t* out_index, int batch, int n, void* workspace,
                                size_t workspace_bytes, cudaStream_t stream) {
    if (!logits || !out_index) return KIVI_ERR_NULL_POINTER;
    if (batch < 0 || n <= 0) return KIVI_ERR_RANGE;
    if (batch == 0) return KIVI_OK;
    const int chunks = argmax_chunks(n);
    const size_t need = (size_t)batch * chunks * (sizeof(float) + sizeof(int));
    if (!workspace || workspace_bytes < need) return KIVI_ERR_WORKSPACE;
    float* pv = static_cast<float*>(workspace);
    int* pi = reinterpret_cast<int*>(pv + (size_t)batch * chunks);
    argmax_partial_kernel<<<dim3(chunks, batch), kArgmaxThreads, 0, stream>>>(H(logits), n, 0, pv, pi);
    if (cudaGetLastError() != cudaSuccess) return KIVI_ERR_CUDA;
    argmax_merge_kernel<<<batch, 32, 0, stream>>>(reinterpret_cast<const unsigned char*>(pv), 0,
                                                  (size_t)batch * chunks * sizeof(float), chunks, 1, batch, out_index,
                                                  P2pGather{});
    return ok(cudaGetLastError());
}
