// TEST INFRASTRUCTURE ONLY. C entry points over the reference's generated-runtime templates
// (crates/jac-codegen-cuda/src/templates/kernels.cu and runtime.cu), compiled where they lie in the
// reference checkout for two model configurations:
//   tiny   2 layers, hidden 256, 4 q / 2 kv heads, head_dim 64, FFN 512, vocab 1024 (parity tests)
//   q14b   the Qwen2.5-14B shape, MAX_SEQ 32768 (timing of the reference's own decode step)
// The element-wise kernels do not depend on the configuration except RoPE (heads, head_dim, base).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cublas_v2.h>
#include <cstdio>
#include <cstdlib>
#include <cmath>

#define REF_NS tiny
#define REF_H 256
#define REF_L 2
#define REF_NH 4
#define REF_NKV 2
#define REF_HD 64
#define REF_FFN 512
#define REF_VOCAB 1024
#define REF_MAX_SEQ 512
#define REF_ROPE_BASE 10000.0f
#define REF_NORM_EPS 1e-5f
#define REF_ATTN_BIAS true
#include "ref_runtime_ns.inc"
#undef REF_NS
#undef REF_H
#undef REF_L
#undef REF_NH
#undef REF_NKV
#undef REF_HD
#undef REF_FFN
#undef REF_VOCAB
#undef REF_MAX_SEQ
#undef REF_ROPE_BASE
#undef REF_NORM_EPS
#undef REF_ATTN_BIAS

#define REF_NS q14b
#define REF_H 5120
#define REF_L 48
#define REF_NH 40
#define REF_NKV 8
#define REF_HD 128
#define REF_FFN 13824
#define REF_VOCAB 152064
#define REF_MAX_SEQ 32768
#define REF_ROPE_BASE 1000000.0f
#define REF_NORM_EPS 1e-6f
#define REF_ATTN_BIAS true
#include "ref_runtime_ns.inc"

extern "C" {

int ref_tiny_set_weights(const __half* embed, const __half* final_norm, const __half* lm_head,
                         const __half* const* layer_ptrs) {
    return tiny::set_weights(embed, final_norm, lm_head, layer_ptrs);
}
int ref_tiny_step(int token, int pos, __half* logits_host) { return tiny::step(token, pos, logits_host); }
void ref_tiny_rope(__half* q, __half* k, int pos) { tiny::rope(q, k, pos); }

int ref_q14b_set_weights(const __half* embed, const __half* final_norm, const __half* lm_head,
                         const __half* const* layer_ptrs) {
    return q14b::set_weights(embed, final_norm, lm_head, layer_ptrs);
}
int ref_q14b_step(int token, int pos, __half* logits_host) { return q14b::step(token, pos, logits_host); }
float ref_q14b_time_steps(int token, int pos, int steps) { return q14b::time_steps(token, pos, steps); }
void ref_q14b_rope(__half* q, __half* k, int pos) { q14b::rope(q, k, pos); }

// Configuration-independent kernels, launched as the reference's forward() launches them
// (runtime.cu:141-185): one row per call.
void ref_rmsnorm(__half* out, const __half* x, const __half* weight, int n, float eps) {
    tiny::rmsnorm_kernel<<<1, 256>>>(out, x, weight, n, eps);
}
void ref_vadd(__half* out, const __half* a, const __half* b, int n) {
    tiny::vadd_kernel<<<(n + 255) / 256, 256>>>(out, a, b, n);
}
void ref_bias_add(__half* y, const __half* bias, int n) { tiny::bias_add_kernel<<<(n + 255) / 256, 256>>>(y, bias, n); }
void ref_silu_mul(__half* out, const __half* gate, const __half* up, int n) {
    tiny::silu_mul_kernel<<<(n + 255) / 256, 256>>>(out, gate, up, n);
}
void ref_argmax(int* out_idx, const __half* logits, int n) { tiny::argmax_kernel<<<1, 256>>>(out_idx, logits, n); }

}  // extern "C"
