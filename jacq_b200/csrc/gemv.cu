// fp16 GEMV / skinny GEMM of the generated decode runtime: y[b, o] = sum_i W[o, i] x[b, i].
//
// The reference calls cublasGemmEx with N = 1 (crates/jac-codegen-cuda/src/templates/runtime.cu:15-26);
// its kernel-DSL form is one thread per row with strided reads (variants.rs:318-329). The product
// is weight-bandwidth bound, so this kernel is a weight streamer: one warp owns two output rows at
// a time, every lane issues 16-byte loads of W (row-contiguous, 512 bytes per warp instruction),
// four k-steps are in flight per row, x sits in shared memory as fp16, products accumulate in fp32
// and a shuffle tree finishes each row. Up to four batch columns share one pass over W.
#include <cooperative_groups.h>
#include <cuda.h>

#include "kivi_common.cuh"
#include "step_math.cuh"

namespace kivi {
namespace {

constexpr int kGemvThreads = kNormThreads;   // the fused RMSNorm prologue needs exactly this many
constexpr int kGemvCtasPerSm = 3;
constexpr int kRowsPerWarp = 2;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <int BT>
__device__ __forceinline__ void fma_chunk(float (&acc)[BT], const uint4& w, const uint4* xs, int chunk,
                                          int chunks_per_x) {
    const __half2* wh = reinterpret_cast<const __half2*>(&w);
    float2 wf[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) wf[e] = __half22float2(wh[e]);
#pragma unroll
    for (int b = 0; b < BT; ++b) {
        const uint4 xv = xs[b * chunks_per_x + chunk];
        const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 xf = __half22float2(xh[e]);
            acc[b] = fmaf(wf[e].x, xf.x, acc[b]);
            acc[b] = fmaf(wf[e].y, xf.y, acc[b]);
        }
    }
}

// kGather: the add+norm prologue takes its delta from a peer exchange (pro.gather.tp > 0). A compile-time split, so
// that the kernels of a single GPU carry none of the exchange's code (their step measured 1.2 % faster for it).
template <int BT, int PRO, bool kGather>
__global__ void __launch_bounds__(kGemvThreads, kGemvCtasPerSm) gemv_kernel(const __half* __restrict__ w, const GemvPrologue pro,
                                                            __half* __restrict__ y16, float* __restrict__ y32,
                                                            int out_dim, int in_dim, int ldy) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float warp_sums[32];
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);  // [BT, in_dim / 8]
    const int chunks = in_dim / 8;
    uint4* ws = xs + BT * chunks;                    // [in_dim / 8] norm weight (add+norm prologues only)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kGemvThreads / 32);
    const int gwarp = blockIdx.x * (kGemvThreads / 32) + warp;
    // A warp owns two rows at a time: neighbours (2k, 2k + 1), or with the SwiGLU epilogue gate row k and up
    // row k + out_dim of a matrix with 2 * out_dim rows.
    constexpr bool kSiluOut = PRO == kGemvAddNormSiluOut;
    constexpr bool kNorm = PRO == kGemvAddNorm || kSiluOut;
    const int row_step = kSiluOut ? 1 : kRowsPerWarp;
    const int pair_stride = kSiluOut ? out_dim : 1;
    const int last_row = kSiluOut ? 2 * out_dim - 1 : out_dim - 1;
    pdl_trigger();

    // The weights do not depend on the kernel before this one: the first loads of W go out before
    // waiting for it, so they are in flight while the predecessor drains and the input is prepared.
    uint4 v[kRowsPerWarp][kUnroll];
    const int first_row = gwarp * row_step;
    bool have = false;
    if (first_row < out_dim && lane + 32 * (kUnroll - 1) < chunks) {
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int row = min(first_row + r * pair_stride, last_row);
            const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)row * in_dim);
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) v[r][u] = ld_stream(wr + lane + 32 * u);
        }
        have = true;
    }
    pdl_wait();

    if (PRO == kGemvPlain) {
        for (int c = threadIdx.x; c < BT * chunks; c += kGemvThreads) xs[c] = reinterpret_cast<const uint4*>(pro.x)[c];
        __syncthreads();
    } else if (kNorm) {
        constexpr bool gathered = kGather;
        P2pView view = {};
        if (gathered) view = p2p_view(pro.gather);
        for (int c = threadIdx.x; c < BT * chunks; c += kGemvThreads) {
            const int b = c / chunks, cc = c - b * chunks;
            const size_t src = pro.tokens ? (size_t)pro.tokens[b] : (size_t)b;
            uint4 a = reinterpret_cast<const uint4*>(pro.x + src * in_dim)[cc];
            if (gathered) a = hadd8(a, p2p_sum8(view, (size_t)c));   // polls until every rank's words have arrived
            else if (pro.delta) a = hadd8(a, reinterpret_cast<const uint4*>(pro.delta + (size_t)b * in_dim)[cc]);
            if (pro.x_out && blockIdx.x == 0) reinterpret_cast<uint4*>(pro.x_out + (size_t)b * in_dim)[cc] = a;
            xs[c] = a;
            if (b == 0) ws[cc] = reinterpret_cast<const uint4*>(pro.weight)[cc];   // needed after the reduction: fetch it now
        }
        __syncthreads();
        float scale[BT];
#pragma unroll
        for (int b = 0; b < BT; ++b)
            scale[b] = rms_scale(reinterpret_cast<const __half*>(xs + b * chunks), in_dim, pro.eps, warp_sums);
        __syncthreads();
        for (int c = threadIdx.x; c < BT * chunks; c += kGemvThreads) {
            const int b = c / chunks, cc = c - b * chunks;
            float sc = scale[0];
#pragma unroll
            for (int k = 1; k < BT; ++k) sc = b == k ? scale[k] : sc;
            xs[c] = norm_apply8(xs[c], ws[cc], sc);
        }
        __syncthreads();
    }

    P2pTarget target = {};
    if (pro.push.tp > 0) target = p2p_target(pro.push);
    for (int row0 = first_row; row0 < out_dim; row0 += warps_total * row_step) {
        float acc[kRowsPerWarp][BT];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[r][b] = 0.0f;
        const uint4* wr[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
            wr[r] = reinterpret_cast<const uint4*>(w + (size_t)min(row0 + r * pair_stride, last_row) * in_dim);
        int c = lane;
        for (; c + 32 * (kUnroll - 1) < chunks; c += 32 * kUnroll) {
            if (!have) {
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) v[r][u] = ld_stream(wr[r] + c + 32 * u);
            }
            have = false;
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) fma_chunk<BT>(acc[r], v[r][u], xs, c + 32 * u, chunks);
        }
        for (; c < chunks; c += 32) {
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                uint4 t = ld_stream(wr[r] + c);
                fma_chunk<BT>(acc[r], t, xs, c, chunks);
            }
        }
#pragma unroll
        for (int b = 0; b < BT; ++b) {
            float s[kRowsPerWarp];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                s[r] = acc[r][b];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s[r] += __shfl_xor_sync(0xffffffffu, s[r], o);
                if (!kSiluOut && lane == 0 && row0 + r < out_dim) {
                    if (y32) y32[(size_t)b * ldy + row0 + r] = s[r];
                    if (y16) y16[(size_t)b * ldy + row0 + r] = __float2half_rn(s[r]);
                }
            }
            // SwiGLU epilogue: gate and up pass through fp16 like the reference's gate_up buffer, then SiLU(g) * u
            if (kSiluOut && lane == 0)
                y16[(size_t)b * ldy + row0] = silu_mul1(__float2half_rn(s[0]), __float2half_rn(s[1]));
            // tensor parallel: the row pair goes straight into every rank's slot (out_dim is even)
            if (!kSiluOut && pro.push.tp > 0 && lane == 0 && row0 + 1 < out_dim)
                p2p_write1(pro.push, target, ((size_t)b * out_dim + row0) >> 1, pack_half2(s[0], s[1]));
        }
    }
}

template <int BT, int PRO, bool kGather>
cudaError_t launch_bt(const __half* w, const GemvPrologue& pro, __half* y16, float* y32, int out_dim, int in_dim,
                      cudaStream_t stream) {
    const bool norm = PRO == kGemvAddNorm || PRO == kGemvAddNormSiluOut;
    const size_t smem = (size_t)(BT + (norm ? 1 : 0)) * in_dim * sizeof(__half);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<BT, PRO, kGather>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    // Enough CTAs to fill the multiprocessors, never more warps than row pairs; all of them
    // resident at once, so a kernel launched behind this one can start as soon as they have.
    const int warps_needed = PRO == kGemvAddNormSiluOut ? out_dim : (out_dim + kRowsPerWarp - 1) / kRowsPerWarp;
    int blocks = (warps_needed + kGemvThreads / 32 - 1) / (kGemvThreads / 32);
    if (blocks > sm_count() * kGemvCtasPerSm) blocks = sm_count() * kGemvCtasPerSm;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_kernel<BT, PRO, kGather>, w, pro, y16, y32, out_dim, in_dim, out_dim);
}

template <int PRO>
cudaError_t launch_pro(const __half* w, const GemvPrologue& pro, __half* y16, float* y32, int out_dim, int in_dim,
                       int batch, cudaStream_t stream) {
    if constexpr (PRO != kGemvPlain) {
        if (pro.gather.tp > 0) {
            switch (batch) {
                case 1: return launch_bt<1, PRO, true>(w, pro, y16, y32, out_dim, in_dim, stream);
                case 2: return launch_bt<2, PRO, true>(w, pro, y16, y32, out_dim, in_dim, stream);
                case 3: return launch_bt<3, PRO, true>(w, pro, y16, y32, out_dim, in_dim, stream);
                default: return launch_bt<4, PRO, true>(w, pro, y16, y32, out_dim, in_dim, stream);
            }
        }
    }
    switch (batch) {
        case 1: return launch_bt<1, PRO, false>(w, pro, y16, y32, out_dim, in_dim, stream);
        case 2: return launch_bt<2, PRO, false>(w, pro, y16, y32, out_dim, in_dim, stream);
        case 3: return launch_bt<3, PRO, false>(w, pro, y16, y32, out_dim, in_dim, stream);
        default: return launch_bt<4, PRO, false>(w, pro, y16, y32, out_dim, in_dim, stream);
    }
}

}  // namespace

// y[b, :] = W prologue(x)[b, :] for 1 <= batch <= 4 in one pass over W.
cudaError_t launch_gemv_fused(const __half* w, int kind, const GemvPrologue& pro, __half* y16, float* y32, int out_dim,
                              int in_dim, int batch, cudaStream_t stream) {
    if (batch < 1 || batch > 4) return cudaErrorInvalidValue;
    if (kind == kGemvAddNorm) return launch_pro<kGemvAddNorm>(w, pro, y16, y32, out_dim, in_dim, batch, stream);
    if (kind == kGemvAddNormSiluOut) {   // out_dim = gate rows = up rows; fp16 output only
        if (!y16 || y32) return cudaErrorInvalidValue;
        return launch_pro<kGemvAddNormSiluOut>(w, pro, y16, y32, out_dim, in_dim, batch, stream);
    }
    return launch_pro<kGemvPlain>(w, pro, y16, y32, out_dim, in_dim, batch, stream);
}

cudaError_t launch_gemv(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim,
                        int batch, cudaStream_t stream) {
    int b = 0;
    while (b < batch) {   // groups of up to four columns share a pass over W
        const int take = batch - b >= 4 ? 4 : batch - b;
        GemvPrologue pro = {};
        pro.x = x + (size_t)b * in_dim;
        cudaError_t e = launch_gemv_fused(w, kGemvPlain, pro, y16 ? y16 + (size_t)b * out_dim : nullptr,
                                          y32 ? y32 + (size_t)b * out_dim : nullptr, out_dim, in_dim, take, stream);
        if (e != cudaSuccess) return e;
        b += take;
    }
    return cudaSuccess;
}

}  // namespace kivi

// ------------------------------------------------------------------------------------------------
// Skinny GEMM for 5..64 batch columns: y[b, o] = sum_i W[o, i] x[b, i] on the tensor cores. Two kernels: the
// tcgen05 + TMA kernel further down is the one that runs; the mma.sync kernel described here is what it
// replaced, kept behind KIVI_SKINNY_UMMA as the comparison (both share the split-K reduction).
//
// The product is still weight-bandwidth bound (every W byte is used once per batch column), so the
// kernel is a W streamer whose arithmetic happens to be MMAs. A CTA of four warps owns 128 output
// rows (32 per warp, so each x fragment read from shared memory feeds two row tiles) and one slice
// of the contraction; W tiles [128 x 64] and the matching x chunk [batch x 64] move through a
// 3-stage cp.async pipeline, so the x chunk is fetched once per CTA, not once per warp. Tile rows
// are 128 bytes with the two 64-byte halves swapped on odd rows, which makes both the 16-byte
// cp.async stores and the 16-byte fragment loads bank-conflict free. Fragments: lane (r, t) takes
// elements 8t..8t+7 of row r for both operands, which fixes the same permutation of the
// contraction on W and x. With few row blocks the contraction is split over the CTAs of a thread-block
// cluster (grid.y = cluster size <= 8): each CTA leaves its partial tile in its own shared memory,
// and after a cluster barrier every CTA adds up one slice of the tile across its peers through
// distributed shared memory and stores it. No workspace, no global round trip, a fixed summation
// order.
namespace kivi {
namespace {

constexpr int kSgRows = 128, kSgK = 64, kSgStages = 3, kSgThreads = 128, kSgCtasPerSm = 3;
constexpr int kSgRowBytes = kSgK * 2;
constexpr int kSgMaxSplits = 8;   // portable cluster size

__device__ __forceinline__ uint32_t sg_offset(int row, int chunk) {
    return (uint32_t)row * kSgRowBytes + (uint32_t)((chunk ^ ((row & 1) << 2)) << 4);
}

constexpr int kSgTileStride = kSgRows + 4;   // floats per batch column of a partial tile: 16-byte aligned, conflict-free stores

// Every CTA of the cluster has left its partial tile, [batch column][row] with stride kSgTileStride, at the same
// place of its shared memory. After a cluster barrier each CTA adds up one share of the tile across its peers
// through distributed shared memory, in rank order, and stores it (and delivers it to the tensor-parallel
// peers when push.tp > 0). Called by all kSgThreads threads of every CTA of the cluster.
__device__ __forceinline__ void sg_reduce_store(float* tile, int row0, int out_dim, int batch, int splits, __half* y16,
                                                float* y32, const P2pPush& push, const P2pTarget& target) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int TS = kSgTileStride;
    cluster.sync();
    const unsigned rank = cluster.block_rank();
    const int quads = batch * (kSgRows / 4);              // 4 consecutive rows of one column
    const int per = (quads + splits - 1) / splits;
    const int lo = (int)rank * per, hi = min(quads, lo + per);
    for (int u = lo + (int)threadIdx.x; u < hi; u += kSgThreads) {
        const int col = u / (kSgRows / 4), rr = (u - col * (kSgRows / 4)) * 4;
        // all remote loads are issued before the first one is used: their latencies overlap
        float4 part[kSgMaxSplits];
#pragma unroll
        for (int peer = 0; peer < kSgMaxSplits; ++peer)
            if (peer < splits) part[peer] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(tile, peer) + col * TS + rr);
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int peer = 0; peer < kSgMaxSplits; ++peer)
            if (peer < splits) { sum.x += part[peer].x; sum.y += part[peer].y; sum.z += part[peer].z; sum.w += part[peer].w; }
        const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int row = row0 + rr + k;
            if (row < out_dim) {
                if (y32) y32[(size_t)col * out_dim + row] = vals[k];
                if (y16) y16[(size_t)col * out_dim + row] = __float2half_rn(vals[k]);
            }
        }
        if (push.tp > 0 && row0 + rr + 3 < out_dim)
            p2p_write2(push, target, ((size_t)col * out_dim + row0 + rr) >> 2, pack_half2(vals[0], vals[1]),
                       pack_half2(vals[2], vals[3]));
    }
    cluster.sync();   // nobody leaves while a peer may still read its tile
}

template <int NT>   // batch columns padded to 8 * NT
__global__ void __launch_bounds__(kSgThreads, kSgCtasPerSm) skinny_gemm_kernel(
    const __half* __restrict__ w, const __half* __restrict__ x, __half* __restrict__ y16, float* __restrict__ y32,
    int out_dim, int in_dim, int batch, int chunks_per_split, const P2pPush push) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int XROWS = 8 * NT;
    constexpr int W_BYTES = kSgRows * kSgRowBytes, X_BYTES = XROWS * kSgRowBytes, STAGE = W_BYTES + X_BYTES;
    const uint32_t s32 = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * kSgRows;
    const int total_chunks = in_dim / kSgK;
    const int c0 = blockIdx.y * chunks_per_split;
    const int c1 = min(total_chunks, c0 + chunks_per_split);
    const int nchunks = c1 - c0;

    // rows of x beyond the batch are zero in every stage (they are never overwritten)
    for (int idx = threadIdx.x; idx < kSgStages * (XROWS - batch) * (kSgRowBytes / 4); idx += kSgThreads) {
        const int st = idx / ((XROWS - batch) * (kSgRowBytes / 4));
        const int rem = idx - st * ((XROWS - batch) * (kSgRowBytes / 4));
        reinterpret_cast<uint32_t*>(smem + st * STAGE + W_BYTES + batch * kSgRowBytes)[rem] = 0u;
    }

    // each thread always copies the same (row, 16-byte column) positions of a tile
    const int cp_row = threadIdx.x >> 3, cp_chunk = threadIdx.x & 7;   // rows cp_row + 16 k
    const uint32_t cp_dst = sg_offset(cp_row, cp_chunk);               // row parity is that of cp_row
    auto issue_w = [&](int c) {
        const uint32_t st = s32 + (uint32_t)(c % kSgStages) * STAGE;
        const size_t k0 = (size_t)(c0 + c) * kSgK;
#pragma unroll
        for (int k = 0; k < kSgRows / 16; ++k) {
            const int row = min(row0 + cp_row + 16 * k, out_dim - 1);
            cp_async16_32(st + cp_dst + (uint32_t)(16 * k) * kSgRowBytes, w + (size_t)row * in_dim + k0 + cp_chunk * 8);
        }
    };
    auto issue_x = [&](int c) {
        const uint32_t st = s32 + (uint32_t)(c % kSgStages) * STAGE;
        const size_t k0 = (size_t)(c0 + c) * kSgK;
#pragma unroll
        for (int k = 0; k < (XROWS + 15) / 16; ++k) {
            const int row = cp_row + 16 * k;
            if (row < batch)
                cp_async16_32(st + W_BYTES + cp_dst + (uint32_t)(16 * k) * kSgRowBytes,
                              x + (size_t)row * in_dim + k0 + cp_chunk * 8);
        }
    };
    auto issue = [&](int c) { issue_w(c); issue_x(c); };
    // The weights do not depend on the kernel before this one: the W tiles of the first stages are requested
    // before waiting for it (the kernel may have been launched early), the x chunks after.
    pdl_trigger();
    for (int c = 0; c < kSgStages - 1; ++c)
        if (c < nchunks) issue_w(c);
    pdl_wait();
    for (int c = 0; c < kSgStages - 1; ++c) {
        if (c < nchunks) issue_x(c);
        asm volatile("cp.async.commit_group;" ::: "memory");   // group c: x chunk c (and, in group 0, every early W tile)
    }

    float acc[2][NT][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.0f;

    // fragment addresses inside a stage: the lane's 16 bytes of the low half; ^64 gives the high half
    const uint32_t frag = (uint32_t)((t ^ ((r & 1) << 2)) << 4);
    const uint32_t wa0 = (uint32_t)(warp * 32 + r) * kSgRowBytes + frag;
    const uint32_t xa0 = W_BYTES + (uint32_t)r * kSgRowBytes + frag;

    for (int c = 0; c < nchunks; ++c) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kSgStages - 2) : "memory");
        __syncthreads();   // chunk c has landed for every thread; the stage refilled below is no longer read
        if (c + kSgStages - 1 < nchunks) issue(c + kSgStages - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const uint32_t st = s32 + (uint32_t)(c % kSgStages) * STAGE;
#pragma unroll
        for (int half = 0; half < 2; ++half) {   // 32 contraction elements per half: lane t holds 8t..8t+7
            const uint32_t wa = (st + wa0) ^ (64u * half), xa = (st + xa0) ^ (64u * half);
            uint4 a[2][2];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                a[m][0] = lds128(wa + (uint32_t)(16 * m) * kSgRowBytes);
                a[m][1] = lds128(wa + (uint32_t)(16 * m + 8) * kSgRowBytes);
            }
            // The MMA wants its four A registers as one aligned group: (row, k pair 0), (row + 8, pair 0), (row, pair 1),
            // (row + 8, pair 1). They come from two different 16-byte loads, so each group is put together once
            // here and then serves every column tile; the x fragments are fetched four tiles at a time to leave
            // the registers for that.
            uint32_t aq[2][2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                aq[m][0][0] = a[m][0].x; aq[m][0][1] = a[m][1].x; aq[m][0][2] = a[m][0].y; aq[m][0][3] = a[m][1].y;
                aq[m][1][0] = a[m][0].z; aq[m][1][1] = a[m][1].z; aq[m][1][2] = a[m][0].w; aq[m][1][3] = a[m][1].w;
            }
            constexpr int JB = NT < 4 ? NT : 4;
#pragma unroll
            for (int j0 = 0; j0 < NT; j0 += JB) {
                uint4 b[JB];
#pragma unroll
                for (int j = 0; j < JB; ++j)
                    if (j0 + j < NT) b[j] = lds128(xa + (uint32_t)(8 * (j0 + j)) * kSgRowBytes);
                // the two MMAs that update one accumulator are issued a sweep apart, so neither waits on the other
#pragma unroll
                for (int j = 0; j < JB; ++j)
#pragma unroll
                    for (int m = 0; m < 2; ++m)
                        if (j0 + j < NT)
                            mma16816(acc[m][j0 + j], aq[m][0][0], aq[m][0][1], aq[m][0][2], aq[m][0][3], b[j].x, b[j].y);
#pragma unroll
                for (int j = 0; j < JB; ++j)
#pragma unroll
                    for (int m = 0; m < 2; ++m)
                        if (j0 + j < NT)
                            mma16816(acc[m][j0 + j], aq[m][1][0], aq[m][1][1], aq[m][1][2], aq[m][1][3], b[j].z, b[j].w);
            }
        }
    }

    // tensor parallel (push.tp > 0, out_dim a multiple of 4): the result also goes straight into every
    // rank's exchange slot, two fp16 rows per 8-byte word
    const int splits = gridDim.y;
    P2pTarget target = {};
    if (push.tp > 0) target = p2p_target(push);
    if (splits == 1) {
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = row0 + warp * 32 + 16 * m + r + ((e & 2) ? 8 : 0), col = 8 * j + 2 * t + (e & 1);
                    if (row < out_dim && col < batch) {
                        if (y32) y32[(size_t)col * out_dim + row] = acc[m][j][e];
                        if (y16) y16[(size_t)col * out_dim + row] = __float2half_rn(acc[m][j][e]);
                    }
                    if (push.tp > 0) {   // the lane four up holds the next row of the same column
                        const float next = __shfl_xor_sync(0xffffffffu, acc[m][j][e], 4);
                        if ((r & 1) == 0 && row + 1 < out_dim && col < batch)
                            p2p_write1(push, target, ((size_t)col * out_dim + row) >> 1, pack_half2(acc[m][j][e], next));
                    }
                }
        return;
    }
    // Partial tile of this split, [batch column][row] with a padded column stride, in the (now idle)
    // pipeline buffers; the cluster then shares the reduction out by flat 4-float slices.
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    constexpr int TS = kSgTileStride;
    float* tile = reinterpret_cast<float*>(smem);
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                tile[(8 * j + 2 * t + (e & 1)) * TS + warp * 32 + 16 * m + r + ((e & 2) ? 8 : 0)] = acc[m][j][e];
    sg_reduce_store(tile, row0, out_dim, batch, splits, y16, y32, push, target);
}

// ------------------------------------------------------------------------------------------------
// The same product on the 5th-generation tensor cores (tcgen05 + TMA), the form taken by default: the legacy
// mma.sync path above is half busy at half the weight bandwidth once the batch reaches 64 columns, and its
// copies compete with the MMAs for issue slots. Per CTA: 128 output rows x N batch columns (N = 16, 32 or
// 64), accumulated in tensor memory (N fp32 columns of the 128 lanes). A [128 x 64] W tile is the A operand
// and the [N x 64] x chunk the B operand, both K-major in shared memory in the canonical 128-byte-swizzled
// form (row pitch 128 bytes, 16-byte chunk c of row r stored at chunk c ^ (r % 8), eight-row groups 1024
// bytes apart): that is what a tiled bulk copy with 128-byte swizzle writes and what the matrix
// descriptors below describe. Nothing in the main loop is done by the CTA as a whole. One thread of warp 0
// requests, per chunk, the W tile and the x chunk as two tiled bulk copies (cp.async.bulk.tensor; rows
// beyond out_dim or the batch arrive as zeros) into a ring of four to six stages and arms the stage's `full` barrier with
// the byte count; one thread of warp 1 waits for `full`, issues the four tcgen05.mma (K = 16 each) of the
// chunk and commits them to the stage's `empty` barrier, which the requesting thread waits for before it
// reuses the stage. The other threads sleep on `all_done` until the last MMA has completed; then every warp
// reads its accumulators with tcgen05.ld (warp w owns lanes 32 w .. 32 w + 31, one output row per thread)
// into the partial tile and the split-K reduction is the one of the mma.sync kernel.
// Every mbarrier wait is bounded; a wait that gives up is counted in g_umma_wait_failures and the kernel
// runs to its end (tensor memory freed, cluster barriers met) with a meaningless result.
__device__ unsigned g_umma_wait_failures = 0;

constexpr int kUmControlBytes = 1024;   // mbarriers and the tensor-memory address, ahead of the 1024-byte aligned stages

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile whose rows are 128 bytes: start
// address, leading-dimension offset 16 bytes (unused by this layout), stride between 8-row groups 1024
// bytes, descriptor version 1, layout type 2 (128-byte swizzle). All offsets in units of 16 bytes.
__device__ __forceinline__ uint64_t um_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate (bit 4), fp16 A and B (formats 0), both K-major, N >> 3
// at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t um_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kSgRows >> 4) << 24);
}
__device__ __forceinline__ void um_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void um_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void um_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void um_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 16 consecutive fp32 columns of the thread's lane
__device__ __forceinline__ void um_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

constexpr int kUmTmaCtasPerSm = 2;
// Stages of the ring: as many as two CTAs per multiprocessor leave room for (a stage is 16 KB of W plus 2, 4 or 8 KB
// of x). With 16 columns six stages measured 3 % faster than four on the Qwen2.5-14B projections.
__host__ __device__ constexpr int um_tma_stages(int n) { return n <= 16 ? 6 : (n <= 32 ? 5 : 4); }
// The cluster reduction moves splits x N x 128 partial sums through distributed shared memory, whose throughput is
// far below the load path's: with N = 64, seven splits cost 10-15 us per launch, four cost a third of that and
// still leave enough CTAs (each with four 24 KB stages in flight at 64 columns) to stream at full rate.
constexpr int kUmTmaMaxSplits = 4;
__host__ __device__ constexpr int um_tma_smem_bytes(int n) {   // 1024 bytes of slack to align the stages
    return 1024 + kUmControlBytes + um_tma_stages(n) * (kSgRows + n) * kSgRowBytes;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

template <int N>   // batch columns padded to N
__global__ void __launch_bounds__(kSgThreads, kUmTmaCtasPerSm) umma_tma_gemm_kernel(
    const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, __half* __restrict__ y16,
    float* __restrict__ y32, int out_dim, int in_dim, int batch, int chunks_per_split, const P2pPush push) {
    extern __shared__ __align__(128) unsigned char smem_unaligned[];
    constexpr int S = um_tma_stages(N);
    constexpr int W_BYTES = kSgRows * kSgRowBytes, X_BYTES = N * kSgRowBytes, STAGE = W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = N < 32 ? 32 : N;
    static_assert(N == 16 || N == 32 || N == 64, "batch columns per tile");
    static_assert(STAGE % 1024 == 0 && W_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
    const uint32_t base = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
    unsigned char* smem = smem_unaligned + (base - smem_u32(smem_unaligned));
    const uint32_t full0 = base, empty0 = base + 8u * S, all_done = base + 16u * S;   // mbarriers
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 16 * S + 8);
    const uint32_t stages = base + kUmControlBytes;
    unsigned char* stage_ptr = smem + kUmControlBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kSgRows;
    const int total_chunks = in_dim / kSgK;
    const int c0 = blockIdx.y * chunks_per_split;
    const int c1 = min(total_chunks, c0 + chunks_per_split);
    const int nchunks = max(c1 - c0, 0);

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * S + 1; ++i) mbar_init(reinterpret_cast<uint64_t*>(smem) + i, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    um_fence_before();
    __syncthreads();
    um_fence_after();
    const uint32_t tmem_d = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    bool failed = false;
    pdl_trigger();
    if (threadIdx.x == 0) {
        // The weights do not depend on the kernel before this one: the W tiles of the first stages are requested
        // before waiting for it (the kernel may have been launched early), the x chunks after.
        const int pre = min(S, nchunks);
        for (int c = 0; c < pre; ++c) {
            mbar_expect_tx32(full0 + 8u * c, STAGE);
            tma_load_2d(stages + (uint32_t)c * STAGE, &wmap, (c0 + c) * kSgK, row0, full0 + 8u * c);
        }
        pdl_wait();
        for (int c = 0; c < pre; ++c)
            tma_load_2d(stages + (uint32_t)c * STAGE + W_BYTES, &xmap, (c0 + c) * kSgK, 0, full0 + 8u * c);
        for (int c = pre; c < nchunks; ++c) {
            const int st = c % S;
            // the MMAs of chunk c - S, the stage's previous tenant, have read their operands
            if (!mbar_wait32(empty0 + 8u * st, (uint32_t)(c / S - 1) & 1u)) failed = true;
            mbar_expect_tx32(full0 + 8u * st, STAGE);
            tma_load_2d(stages + (uint32_t)st * STAGE, &wmap, (c0 + c) * kSgK, row0, full0 + 8u * st);
            tma_load_2d(stages + (uint32_t)st * STAGE + W_BYTES, &xmap, (c0 + c) * kSgK, 0, full0 + 8u * st);
        }
    } else {
        pdl_wait();
        if (threadIdx.x == 32) {
            constexpr uint32_t idesc = um_idesc(N);
            for (int c = 0; c < nchunks; ++c) {
                const int st = c % S;
                if (!mbar_wait32(full0 + 8u * st, (uint32_t)(c / S) & 1u)) failed = true;
                um_fence_after();
                const uint64_t adesc = um_desc(stages + (uint32_t)st * STAGE), bdesc = um_desc(stages + (uint32_t)st * STAGE + W_BYTES);
#pragma unroll
                for (int k = 0; k < kSgK / 16; ++k)   // 16 contraction elements = 32 bytes further along the swizzled row
                    um_mma(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (c > 0 || k > 0) ? 1u : 0u);
                um_commit(empty0 + 8u * st);
            }
            if (nchunks > 0) um_commit(all_done);   // every MMA of this CTA has completed when this arrives
        }
    }
    __syncwarp();
    if (nchunks > 0 && !mbar_wait32(all_done, 0u)) failed = true;
    um_fence_after();

    // accumulators: lane (= output row) 32 warp + lane, N columns
    float acc[N];
    if (nchunks > 0) {
#pragma unroll
        for (int j = 0; j < N; j += 16) um_ld16(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)j, acc + j);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = 0.0f;
    }
    um_fence_before();
    const bool cta_failed = __syncthreads_or(failed);   // all warps have their accumulators
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(TMEM_COLS) : "memory");
    if (cta_failed && threadIdx.x == 0) atomicAdd(&g_umma_wait_failures, 1u);

    constexpr int TS = kSgTileStride;
    float* tile = reinterpret_cast<float*>(stage_ptr);   // the stages are idle
#pragma unroll
    for (int j = 0; j < N; ++j) tile[j * TS + warp * 32 + lane] = acc[j];
    P2pTarget target = {};
    if (push.tp > 0) target = p2p_target(push);
    sg_reduce_store(tile, row0, out_dim, batch, (int)gridDim.y, y16, y32, push, target);
}

struct SkinnyPlan { int row_blocks, splits, chunks_per_split, nt; };

SkinnyPlan plan_skinny(int out_dim, int in_dim, int batch, int ctas_per_sm = kSgCtasPerSm, int split_cap = kSgMaxSplits) {
    SkinnyPlan p;
    p.nt = (batch + 7) / 8;
    p.row_blocks = (out_dim + kSgRows - 1) / kSgRows;
    const int chunks = in_dim / kSgK;
    int splits = ctas_per_sm * sm_count() / p.row_blocks;               // at most one wave of resident CTAs
    const int max_splits = chunks / 8 > 0 ? chunks / 8 : 1;      // at least 8 chunks (512 elements) per CTA
    if (splits > max_splits) splits = max_splits;
    if (splits > split_cap) splits = split_cap;
    if (splits < 1) splits = 1;
    p.chunks_per_split = (chunks + splits - 1) / splits;
    p.splits = splits;   // a trailing split may get fewer chunks, or none: it still joins the reduction
    return p;
}

// KIVI_SKINNY_EARLY=0 in the environment launches the skinny GEMM the ordinary way (tuning switch).
inline bool skinny_early_launch() {
    static const bool on = [] { const char* e = getenv("KIVI_SKINNY_EARLY"); return !e || atoi(e) != 0; }();
    return on;
}

template <int NT>
cudaError_t launch_skinny_nt(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim, int batch,
                             const SkinnyPlan& p, const P2pPush& push, cudaStream_t stream) {
    const int smem = kSgStages * (kSgRows + 8 * NT) * kSgRowBytes;
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.row_blocks, p.splits, 1);
    cfg.blockDim = dim3(kSgThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = skinny_early_launch() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<NT>, w, x, y16, y32, out_dim, in_dim, batch, p.chunks_per_split, push);
}

// KIVI_SKINNY_UMMA in the environment: the smallest batch that takes the tcgen05 kernel (tuning switch; above 64:
// never, every batch then runs on the mma.sync kernel).
inline int umma_min_batch() {
    static const int v = [] { const char* e = getenv("KIVI_SKINNY_UMMA"); return e ? atoi(e) : 5; }();
    return v;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: the library does not link libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled() {
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map of a row-major fp16 matrix [rows, cols] read in boxes of box_rows x 64 columns, 128-byte swizzle,
// out-of-range elements as zeros. base 16-byte aligned, cols a multiple of 8.
inline bool make_tile_map(CUtensorMap* map, const __half* base, int rows, int cols, int box_rows) {
    const EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(__half)};
    const cuuint32_t box[2] = {(cuuint32_t)kSgK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int N>
cudaError_t launch_umma_tma_n(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim, int batch,
                              const P2pPush& push, cudaStream_t stream) {
    const SkinnyPlan p = plan_skinny(out_dim, in_dim, batch, kUmTmaCtasPerSm, kUmTmaMaxSplits);
    CUtensorMap wmap, xmap;
    if (!make_tile_map(&wmap, w, out_dim, in_dim, kSgRows) || !make_tile_map(&xmap, x, batch, in_dim, N))
        return cudaErrorInvalidValue;
    const int smem = um_tma_smem_bytes(N);
    cudaError_t e = cudaFuncSetAttribute(umma_tma_gemm_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.row_blocks, p.splits, 1);
    cfg.blockDim = dim3(kSgThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = skinny_early_launch() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, umma_tma_gemm_kernel<N>, wmap, xmap, y16, y32, out_dim, in_dim, batch, p.chunks_per_split, push);
}

}  // namespace

bool skinny_gemm_supports(int in_dim, int batch) { return batch > 4 && batch <= 64 && in_dim % kSgK == 0; }

// push (may be nullptr): deliver the fp16 result into every rank's exchange slot as well; needs out_dim % 4 == 0.
cudaError_t launch_skinny_gemm(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim,
                               int batch, cudaStream_t stream, const P2pPush* push_or_null) {
    if (push_or_null && out_dim % 4) return cudaErrorInvalidValue;
    const P2pPush push = push_or_null ? *push_or_null : P2pPush{};
    const SkinnyPlan p = plan_skinny(out_dim, in_dim, batch);
    if (batch >= umma_min_batch()) {
        if (batch <= 16) return launch_umma_tma_n<16>(w, x, y16, y32, out_dim, in_dim, batch, push, stream);
        if (batch <= 32) return launch_umma_tma_n<32>(w, x, y16, y32, out_dim, in_dim, batch, push, stream);
        return launch_umma_tma_n<64>(w, x, y16, y32, out_dim, in_dim, batch, push, stream);
    }
    switch (p.nt) {
        case 1: return launch_skinny_nt<1>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        case 2: return launch_skinny_nt<2>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        case 3: return launch_skinny_nt<3>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        case 4: return launch_skinny_nt<4>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        case 5: return launch_skinny_nt<5>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        case 6: return launch_skinny_nt<6>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        case 7: return launch_skinny_nt<7>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
        default: return launch_skinny_nt<8>(w, x, y16, y32, out_dim, in_dim, batch, p, push, stream);
    }
}

}  // namespace kivi

extern "C" int kivi_b200_gemm_wait_failures(uint32_t* failures_out) {
    if (!failures_out) return KIVI_ERR_NULL_POINTER;
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, kivi::g_umma_wait_failures, sizeof(v)) != cudaSuccess) return KIVI_ERR_CUDA;
    *failures_out = v;
    return KIVI_OK;
}
