// fp16 GEMV / skinny GEMM of the generated decode runtime: y[b, o] = sum_i W[o, i] x[b, i].
//
// The reference calls cublasGemmEx with N = 1 (crates/jac-codegen-cuda/src/templates/runtime.cu:15-26);
// its kernel-DSL form is one thread per row with strided reads (variants.rs:318-329). The product
// is weight-bandwidth bound, so this kernel is a weight streamer: one warp owns two output rows at
// a time, every lane issues 16-byte loads of W (row-contiguous, 512 bytes per warp instruction),
// four k-steps are in flight per row, x sits in shared memory as fp16, products accumulate in fp32
// and a shuffle tree finishes each row. Up to four batch columns share one pass over W.
#include "kivi_common.cuh"

namespace kivi {
namespace {

constexpr int kGemvThreads = 256;
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

template <int BT>
__global__ void __launch_bounds__(kGemvThreads) gemv_kernel(const __half* __restrict__ w, const __half* __restrict__ x,
                                                            __half* __restrict__ y16, float* __restrict__ y32,
                                                            int out_dim, int in_dim, int ldy) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);  // [BT, in_dim / 8]
    const int chunks = in_dim / 8;
    for (int c = threadIdx.x; c < BT * chunks; c += kGemvThreads) xs[c] = reinterpret_cast<const uint4*>(x)[c];
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kGemvThreads / 32);
    const int gwarp = blockIdx.x * (kGemvThreads / 32) + warp;

    for (int row0 = gwarp * kRowsPerWarp; row0 < out_dim; row0 += warps_total * kRowsPerWarp) {
        float acc[kRowsPerWarp][BT];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[r][b] = 0.0f;
        const uint4* wr[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            int row = row0 + r < out_dim ? row0 + r : out_dim - 1;
            wr[r] = reinterpret_cast<const uint4*>(w + (size_t)row * in_dim);
        }
        int c = lane;
        for (; c + 32 * (kUnroll - 1) < chunks; c += 32 * kUnroll) {
            uint4 v[kRowsPerWarp][kUnroll];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) v[r][u] = ld_stream(wr[r] + c + 32 * u);
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) fma_chunk<BT>(acc[r], v[r][u], xs, c + 32 * u, chunks);
        }
        for (; c < chunks; c += 32) {
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                uint4 v = ld_stream(wr[r] + c);
                fma_chunk<BT>(acc[r], v, xs, c, chunks);
            }
        }
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                float s = acc[r][b];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0 && row0 + r < out_dim) {
                    if (y32) y32[(size_t)b * ldy + row0 + r] = s;
                    if (y16) y16[(size_t)b * ldy + row0 + r] = __float2half_rn(s);
                }
            }
    }
}

template <int BT>
cudaError_t launch_bt(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim,
                      cudaStream_t stream) {
    const size_t smem = (size_t)BT * in_dim * sizeof(__half);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    // Enough CTAs to fill the 148 SMs a few times over, never more warps than row pairs.
    const int warps_needed = (out_dim + kRowsPerWarp - 1) / kRowsPerWarp;
    int blocks = (warps_needed + kGemvThreads / 32 - 1) / (kGemvThreads / 32);
    if (blocks > 148 * 4) blocks = 148 * 4;
    gemv_kernel<BT><<<blocks, kGemvThreads, smem, stream>>>(w, x, y16, y32, out_dim, in_dim, out_dim);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemv(const __half* w, const __half* x, __half* y16, float* y32, int out_dim, int in_dim,
                        int batch, cudaStream_t stream) {
    int b = 0;
    while (b < batch) {
        const int left = batch - b;
        const __half* xb = x + (size_t)b * in_dim;
        __half* y16b = y16 ? y16 + (size_t)b * out_dim : nullptr;
        float* y32b = y32 ? y32 + (size_t)b * out_dim : nullptr;
        cudaError_t e;
        if (left >= 4) { e = launch_bt<4>(w, xb, y16b, y32b, out_dim, in_dim, stream); b += 4; }
        else if (left >= 2) { e = launch_bt<2>(w, xb, y16b, y32b, out_dim, in_dim, stream); b += 2; }
        else { e = launch_bt<1>(w, xb, y16b, y32b, out_dim, in_dim, stream); b += 1; }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace kivi
