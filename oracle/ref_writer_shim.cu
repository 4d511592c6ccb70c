// TEST INFRASTRUCTURE ONLY. Gives the reference's hand-CUDA cache writer (C++ linkage in the
// reference, integrations/vllm_kivi/source_patch.py:1661-1666 and :1737-1742) and its cuBLAS
// gemv() call (crates/jac-codegen-cuda/src/templates/runtime.cu:15-26) C entry points so the
// tests can drive them through ctypes. The writer source is dumped, unmodified, from the
// reference's Python string into oracle/_ref/ by build_ref.py and included here.
#include "kivi_cache_write_hand.cu"

#include <cublas_v2.h>

extern "C" void ref_kivi_cache_write_launch(
    unsigned char* K_CODE_PAGES, __half* K_SCALE_PAGES, __half* K_ZERO_PAGES,
    unsigned char* V_CODE_PAGES, __half* V_SCALE_PAGES, __half* V_ZERO_PAGES,
    __half* K_RESIDUAL_SCRATCH, __half* V_RESIDUAL_SCRATCH,
    const __half* NEW_K, const __half* NEW_V, const int64_t* SLOT_MAPPING,
    const int* BLOCK_TABLE, int seq_len, int NKV_RUNTIME, cudaStream_t stream) {
  kivi_cache_write_launch(K_CODE_PAGES, K_SCALE_PAGES, K_ZERO_PAGES, V_CODE_PAGES, V_SCALE_PAGES,
                          V_ZERO_PAGES, K_RESIDUAL_SCRATCH, V_RESIDUAL_SCRATCH, NEW_K, NEW_V,
                          SLOT_MAPPING, BLOCK_TABLE, seq_len, NKV_RUNTIME, stream);
}

extern "C" void ref_kivi_cache_write_batched_launch(
    unsigned char* K_CODE_PAGES, __half* K_SCALE_PAGES, __half* K_ZERO_PAGES,
    unsigned char* V_CODE_PAGES, __half* V_SCALE_PAGES, __half* V_ZERO_PAGES,
    __half* K_RESIDUAL_SCRATCH, __half* V_RESIDUAL_SCRATCH,
    const __half* NEW_K, const __half* NEW_V, const int64_t* SLOT_MAPPING,
    const int* BLOCK_TABLE, int START_SEQ_LEN, int NUM_NEW, int NKV_RUNTIME, cudaStream_t stream) {
  kivi_cache_write_batched_launch(K_CODE_PAGES, K_SCALE_PAGES, K_ZERO_PAGES, V_CODE_PAGES,
                                  V_SCALE_PAGES, V_ZERO_PAGES, K_RESIDUAL_SCRATCH,
                                  V_RESIDUAL_SCRATCH, NEW_K, NEW_V, SLOT_MAPPING, BLOCK_TABLE,
                                  START_SEQ_LEN, NUM_NEW, NKV_RUNTIME, stream);
}

// The generated runtime's gemv(): cublasGemmEx with the reference's exact arguments.
extern "C" int ref_gemv_cublas(const __half* W, const __half* x, __half* y, int in_dim, int out_dim,
                               cudaStream_t stream) {
  static cublasHandle_t handle = nullptr;
  if (!handle && cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
  cublasSetStream(handle, stream);
  const float alpha = 1.0f, beta = 0.0f;
  cublasStatus_t st = cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, out_dim, 1, in_dim, &alpha,
                                   W, CUDA_R_16F, in_dim, x, CUDA_R_16F, in_dim, &beta,
                                   y, CUDA_R_16F, out_dim, CUBLAS_COMPUTE_32F,
                                   CUBLAS_GEMM_DEFAULT_TENSOR_OP);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 2;
}
