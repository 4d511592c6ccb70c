// Shared definitions of the B200 KIVI kernels: launch-parameter blocks, geometry helpers and the
// few PTX wrappers (mbarrier, bulk async copy, mma, movmatrix) the kernels use.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdlib>

#include "../../include/jacq_kivi_b200.h"

namespace kivi {

// Geometry as the kernels see it (all derived values precomputed on the host).
struct Geom {
    int nh, nkv, d, b, g, r;
    int qpk;           // query heads per kv head
    int hg;            // value channel groups, ceil(D / G)
    int vg;            // value channel-group width, min(G, D)
    int scratch_rows;  // R + G
    int pages_per_group;
    int log2b;         // log2(block) when the block size is a power of two, else -1
};

inline Geom make_geom(const kivi_geometry& s) {
    Geom g;
    g.nh = s.num_q_heads; g.nkv = s.num_kv_heads; g.d = s.head_dim;
    g.b = s.block_size; g.g = s.group_size; g.r = s.residual;
    g.qpk = g.nh / g.nkv;
    g.hg = (g.d + g.g - 1) / g.g;
    g.vg = g.g < g.d ? g.g : g.d;
    g.scratch_rows = g.r + g.g;
    g.pages_per_group = g.g / g.b;
    g.log2b = -1;
    for (int sh = 0; sh < 16; ++sh) if ((1 << sh) == g.b) g.log2b = sh;
    return g;
}

// split_old_tokens of the reference (integrations/vllm_kivi/source_patch.py:1655-1659) with the
// key group as the age-out unit.
__host__ __device__ inline int split_old(int seq_len, int residual, int group) {
    int q = seq_len - residual;
    if (q < 0) return 0;
    return (q / group) * group;
}

struct CachePtrs {
    uint8_t* k_code; __half* k_scale; __half* k_zero;
    uint8_t* v_code; __half* v_scale; __half* v_zero;
    __half* k_scratch; __half* v_scratch;
    // Pages in the pools and scratch slots, where the caller stated them (ABI v2); INT_MAX for the reference-lane
    // symbols, whose signatures carry no sizes. Page ids and slot ids read from device memory are held against them.
    int num_blocks, num_slots;
};

// A page or slot id read from device memory is used as an address only when it lies inside the pool. A block
// table entry that is stale or garbage would otherwise become an out-of-bounds access; ids that fail are counted
// (kivi_b200_rejected_indices) and the access is skipped (writer: the whole sequence's write) or redirected to
// id 0 (decode: the output of that sequence is then meaningless, but nothing outside the pool is touched).
__host__ __device__ inline bool index_in_pool(int id, int pool_size) { return (unsigned)id < (unsigned)pool_size; }

// How a launch finds each sequence's length, block-table row and scratch slot. The v1 symbols
// pass host scalars and one shared table; the v2 calls pass device arrays.
struct SeqAddressing {
    const int* seq_lens;      // device [n] or nullptr -> seq_len_scalar
    int seq_len_scalar;
    const int* block_tables;  // device
    int bt_stride;            // elements between rows; 0 = one shared table
    int bt_width;             // entries readable per row
    const int* slot_ids;      // device [n] or nullptr
    int slot_shared;          // with slot_ids == nullptr: 1 -> slot 0 for all, 0 -> slot i
};

__device__ __forceinline__ int seq_len_of(const SeqAddressing& a, int i) {
    return a.seq_lens ? a.seq_lens[i] : a.seq_len_scalar;
}
__device__ __forceinline__ int slot_of(const SeqAddressing& a, int i) {
    return a.slot_ids ? a.slot_ids[i] : (a.slot_shared ? 0 : i);
}

// Decode bounds of the reference kernel (crates/jac-codegen-cuda/src/variants.rs:2486-2495) for a
// runtime geometry: quantised tokens scanned and residual rows read. max_seq is the longest
// sequence the launch was planned for (the reference's LQ + RESIDUAL); longer lengths are clamped
// to it, as the reference does. max_seq < 0 = no cap.
struct DecodeBounds { int old_valid; int res_valid; };
__host__ __device__ inline DecodeBounds decode_bounds(int seq_len, int residual, int group, int max_seq,
                                                      int bt_width, int block) {
    int bounded = seq_len < 0 ? 0 : seq_len;
    if (max_seq >= 0 && bounded > max_seq) bounded = max_seq;
    int ov = split_old(bounded, residual, group);
    // never walk past the block table the caller gave us
    long long cover = (long long)bt_width * block;
    if (ov > cover) ov = (int)((cover / group) * group);
    int rv = bounded - ov;
    if (rv < 0) rv = 0;
    if (rv > residual + group) rv = residual + group;
    DecodeBounds b; b.old_valid = ov; b.res_valid = rv;
    return b;
}

// ---------------------------------------------------------------------------------------------
// Launch plan of the tensor-core decode kernel. Work units are the (sequence, kv head) pairs in order. A launch
// whose units do not fill whole waves of resident CTAs would end on a few CTAs running alone, so the first
// `units1` units are cut into k1 equal parts each and the rest into k2 >= k1 parts: CTAs start in index order,
// the large jobs first, and the small ones fill what would have been the partial wave. A unit cut into parts
// leaves one partial per part (slot numbers below) for the merge kernel; uncut units write their output themselves.
struct JobPlan {
    int units1, k1, units2, k2;
    __host__ __device__ int jobs1() const { return units1 * k1; }
    __host__ __device__ int jobs() const { return units1 * k1 + units2 * k2; }
    __host__ __device__ int slots() const { return (k1 > 1 ? units1 * k1 : 0) + (k2 > 1 ? units2 * k2 : 0); }
    __host__ __device__ int cut_units() const { return (k1 > 1 ? units1 : 0) + (k2 > 1 ? units2 : 0); }
};

// ---------------------------------------------------------------------------------------------
// Decode launch parameters shared by the generic and the tensor-core kernels.
struct DecodeParams {
    Geom geom;
    CachePtrs cache;
    SeqAddressing seq;
    const __half* q;      // [n, NH, D]
    float* out;           // [n, NH, D]
    __half* out_h;        // when set, the result is written here as fp16 instead of `out`
    int n;                // queries (sequences) in this launch
    int max_seq;          // longest sequence the launch is planned for (reference: LQ + RESIDUAL), or -1
    int retained_pages;   // sparse-retained: pages to scan from the compact table, else -1
    const int* retained_dev;  // sparse-retained with one count per sequence (device [n]); overrides retained_pages
    // Generic kernel: split over the context. Each CTA takes `chunk_tokens` quantised tokens, the fp16 residual of a
    // split context is a chunk of its own; partials go to the workspace and a second kernel merges them.
    int chunk_tokens;
    int max_chunks;
    float* ws_o;          // [n, NKV, max_chunks, QPK, D]
    float* ws_ml;         // [n, NKV, max_chunks, QPK, 2]  (running max in log2 units, sum)
    int* status;          // device status word (0 = ok), may be nullptr
    // Tensor-core kernel: how the units are cut into jobs (one CTA each); partials of cut units go to
    // ws_o [plan.slots(), QPK, D] / ws_ml [plan.slots(), QPK, 2].
    JobPlan plan;
};

__device__ __forceinline__ void store_out(const DecodeParams& p, size_t idx, float v) {
    if (p.out_h) p.out_h[idx] = __float2half(v);
    else p.out[idx] = v;
}

// Writer launch parameters.
struct WriteParams {
    Geom geom;
    CachePtrs cache;
    SeqAddressing seq;        // seq_lens = length BEFORE the new tokens
    const __half* new_k;      // [total_new, NKV, D]
    const __half* new_v;
    const int* new_offsets;   // device [n+1] or nullptr -> sequence i owns rows [i*num_new_scalar, ...)
    int num_new_scalar;
    int n;
};

// ---------------------------------------------------------------------------------------------
// PTX helpers.

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (each poll itself blocks for a hardware-defined time)
// and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int it = 0; it < (1 << 22); ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk asynchronous copy global -> shared (the TMA engine, no tensor map; the plain single-CTA form).
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// 16-byte asynchronous copy global -> shared (per-thread cp.async), and the arrive that lets an
// mbarrier track every cp.async this thread issued before it (.noinc: the arrival was counted at init).
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory access by 32-bit shared-window address: keeps the address arithmetic of the hot
// loops in one 32-bit add per access (constant parts fold into the instruction's immediate).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_half(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ void mbar_expect_tx32(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait32(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 22); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s32(uint32_t dst, const void* src_gmem, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src_gmem), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16_32(uint32_t dst, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc32(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_32(uint32_t (&r)[4], uint32_t a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void ldmatrix_x4_trans_32(uint32_t (&r)[4], uint32_t a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may start
// while its predecessor drains; it must call pdl_wait() before touching anything the predecessor
// wrote -- in EVERY CTA, also one that has nothing to do: the kernel after it waits only for this grid, and
// a grid whose CTAs left without waiting completes before its own predecessor has. pdl_trigger() lets
// the successor start early; it is harmless when nothing depends on it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The small kernels of the attention chain (RoPE + write, decode, merge) can be launched this way too
// (KIVI_PDL_CHAIN=1 in the environment), but that measured slower than ordinary launches inside a CUDA
// graph: 7.02 vs 6.01 ms per decode step with the merge kernel alone launched early. Early launch pays
// where there is something to do before the wait, as in the GEMVs, which prefetch their weights; a
// small kernel parked behind the decode kernel only takes resources from it. The kernels are correct
// either way.
inline bool pdl_chain_enabled() {
    static const bool on = [] { const char* e = getenv("KIVI_PDL_CHAIN"); return e && atoi(e) != 0; }();
    return on;
}

// Launch with programmatic stream serialisation allowed (the kernel must follow the pdl_wait rule above).
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_chain_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Transpose an 8x8 tile of 16-bit elements held one 32-bit register per lane (row lane/4,
// columns 2*(lane%4), +1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Multiprocessors of the current device, asked once per device (api.cu).
int sm_count();

// Host-side launchers implemented in the .cu files.
cudaError_t launch_cache_write(const WriteParams& p, int max_new_per_seq, cudaStream_t stream);
struct RopeParams;     // step_math.cuh
cudaError_t launch_rope_write(const RopeParams& rp, const WriteParams& p, cudaStream_t stream);
// Plans the split over the context, binds the workspace and launches the decode kernel; returns a
// kivi_status. `out_h` (fp16) replaces `out` (fp32) when non-null.
int run_decode(const Geom& g, const CachePtrs& cache, const SeqAddressing& seq, const __half* q, float* out,
               __half* out_h, int n, int max_seq_cap, int max_old_tokens, int retained_pages, void* ws,
               size_t ws_bytes, cudaStream_t stream, const int* retained_dev = nullptr);
size_t decode_workspace_total(const Geom& g, int n, int max_old_tokens);
cudaError_t launch_decode_generic(const DecodeParams& p, cudaStream_t stream);
cudaError_t decode_generic_rejected(unsigned int* count);
cudaError_t launch_decode_mma(const DecodeParams& p, cudaStream_t stream);
bool decode_mma_supports(const Geom& g, int retained_pages);
int decode_mma_ctas_per_sm();
cudaError_t launch_gemv(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim,
                        int batch, cudaStream_t stream);
struct GemvPrologue;   // step_math.cuh
cudaError_t launch_gemv_fused(const __half* w, int kind, const GemvPrologue& pro, __half* y16, float* y32, int out_dim,
                              int in_dim, int batch, cudaStream_t stream);
bool skinny_gemm_supports(int in_dim, int batch);
struct P2pPush;        // p2p.cuh
cudaError_t launch_skinny_gemm(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim,
                               int batch, cudaStream_t stream, const P2pPush* push_or_null = nullptr);

}  // namespace kivi
