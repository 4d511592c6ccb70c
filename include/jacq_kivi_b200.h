/*
 * jacq_kivi_b200 -- C launch contract of the B200-native int4-KIVI paged KV-cache path.
 *
 * One shared library (libjacq_kivi_b200.so) exports two families of entry points:
 *
 *  1. The reference's versioned launch contract, ABI v1 (docs/ABI.md of ImpossibleComputing/jacq):
 *     the exact `extern "C"` symbols the reference's torch-op binding declares
 *     (integrations/vllm_kivi/source_patch.py:570-658), compiled for the reference lane geometry
 *     (NH/NKV 40/8 or 20/4 for the `_tp2_local` symbols, head_dim 128, block = group = 32,
 *     residual 128, at most 124 old pages). They are drop-in: same argument order, same in-place
 *     mutation, asynchronous on the caller's stream, print-and-exit on a launch error.
 *
 *  2. ABI v2: runtime geometry, many sequences per launch, device-resident sequence lengths (no host
 *     synchronisation, usable under CUDA graph capture once the workspace exists), `int` status
 *     instead of exit(). The reference has no such call; it loops over requests and tokens in
 *     Python (integrations/vllm_kivi/source_patch.py:3105-3288).
 *
 * Every pointer below is a DEVICE pointer unless it says "host". fp16 tensors are passed as
 * `kivi_f16*` (raw IEEE binary16 bits). Nothing here allocates device memory unless stated.
 *
 * Tensor layout (reference: integrations/vllm_kivi/bindings.py:105-118), for geometry
 * NH query heads, NKV kv heads, D head_dim, B page tokens, G key group, R residual tokens,
 * HG = ceil(D / G) value channel groups of width min(G, D):
 *
 *   K_CODE_PAGES, V_CODE_PAGES   u8  [num_blocks, NKV, B, D/2]  byte j = channel 2j (low nibble),
 *                                                               channel 2j+1 (high nibble)
 *   K_SCALE_PAGES, K_ZERO_PAGES  f16 [num_blocks, NKV, D]       per channel, over the G tokens of
 *                                                               the group; when G > B the same
 *                                                               values are stored in every page of
 *                                                               the group
 *   V_SCALE_PAGES, V_ZERO_PAGES  f16 [num_blocks, NKV, B, HG]   per token, per channel group
 *   K/V_RESIDUAL_SCRATCH         f16 [num_slots, NKV, R+G, D]   row 0 = oldest unquantised token
 *   BLOCK_TABLE                  i32 [>= T_old / B]             logical page -> physical page
 *   Q f16 [NH, D],  O f32 [NH, D]
 *
 *   T_old = floor(max(T - R, 0) / G) * G tokens are quantised; the remaining T - T_old live in
 *   scratch rows [0, T - T_old).
 */
#ifndef JACQ_KIVI_B200_H_
#define JACQ_KIVI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __CUDA_RUNTIME_H__
typedef struct CUstream_st* cudaStream_t;
#endif

typedef uint16_t kivi_f16;

/* Same value as JACQ_KIVI_ABI_VERSION would take after the v2 additions (the reference's rule:
 * bump on any tensor-shape, launch-order or constant change; integrations/vllm_kivi/abi.py:35-36). */
#define JACQ_KIVI_B200_ABI_VERSION 2

enum kivi_status {
    KIVI_OK = 0,
    KIVI_ERR_NULL_POINTER = 1,     /* a required pointer is NULL */
    KIVI_ERR_GEOMETRY = 2,         /* unsupported or inconsistent geometry */
    KIVI_ERR_RANGE = 3,            /* batch / length / count out of range */
    KIVI_ERR_ALIGNMENT = 4,        /* a tensor base is not 16-byte aligned */
    KIVI_ERR_WORKSPACE = 5,        /* workspace missing or too small */
    KIVI_ERR_CUDA = 6,             /* the CUDA runtime reported an error on launch */
    KIVI_ERR_BLOCK_TABLE = 7       /* block table too narrow for the stated lengths */
};

/* Runtime geometry. The reference fixes these per translation unit as `static constexpr`
 * (crates/jac-codegen-cuda/src/variants.rs:2577-2587). */
typedef struct kivi_geometry {
    int32_t num_q_heads;   /* NH */
    int32_t num_kv_heads;  /* NKV; NH % NKV == 0 */
    int32_t head_dim;      /* D; 64 or 128 on the tensor-core path, any even value otherwise */
    int32_t block_size;    /* B, tokens per page */
    int32_t group_size;    /* G, tokens per key group; G % B == 0 */
    int32_t residual;      /* R, fp16 residual window */
} kivi_geometry;

/* One layer's page pool and residual scratch slots. */
typedef struct kivi_cache {
    uint8_t* k_code_pages;
    kivi_f16* k_scale_pages;
    kivi_f16* k_zero_pages;
    uint8_t* v_code_pages;
    kivi_f16* v_scale_pages;
    kivi_f16* v_zero_pages;
    kivi_f16* k_residual_scratch;
    kivi_f16* v_residual_scratch;
    int32_t num_blocks;
    int32_t num_slots;
} kivi_cache;

/* ------------------------------------------------------------------ ABI v2 ------------------ */

int kivi_b200_abi_version(void);
const char* kivi_b200_status_string(int status);

/* KIVI_OK if the geometry is usable at all; *fast_path (may be NULL) receives 1 when the
 * tensor-core decode kernel covers it, 0 when the generic kernel runs instead. */
int kivi_b200_validate_geometry(const kivi_geometry* geom, int* fast_path);

/* Cache writer for `batch` sequences in one call. Sequence i appends the rows
 * new_offsets[i] .. new_offsets[i+1]-1 of NEW_K / NEW_V ([total_new, NKV, D], token-major) to a
 * cache that held start_seq_lens[i] tokens, ageing out as many key groups as that crosses.
 * The result equals the reference's single-token writer applied token by token
 * (integrations/vllm_kivi/source_patch.py:1661-1697; batched form :1737-1775, which needs the
 * Python planner :504-553 to stay within one age-out per call -- not needed here).
 *   block_tables   i32 [batch, max_blocks_per_seq]
 *   start_seq_lens i32 [batch], new_offsets i32 [batch+1]   (device)
 *   slot_ids       i32 [batch] scratch slot of each sequence, or NULL for slot i = i
 *   max_new_per_seq  host upper bound of new_offsets[i+1]-new_offsets[i] (sizes the launch)
 *   max_start_seq_len host upper bound of start_seq_lens (checks the block-table width) */
int kivi_b200_cache_write(const kivi_geometry* geom, const kivi_cache* cache,
                          const kivi_f16* new_k, const kivi_f16* new_v,
                          const int32_t* block_tables, int max_blocks_per_seq,
                          const int32_t* start_seq_lens, const int32_t* new_offsets,
                          const int32_t* slot_ids, int batch, int max_new_per_seq,
                          int max_start_seq_len, cudaStream_t stream);

/* Bytes of caller-owned workspace the decode needs for this batch and longest sequence. */
size_t kivi_b200_decode_workspace_bytes(const kivi_geometry* geom, int batch, int max_seq_len);

/* Zero the workspace. Kept for callers of earlier versions: the decode reads only what the same call
 * wrote, so the workspace needs no initial contents. */
int kivi_b200_decode_workspace_init(void* workspace, size_t workspace_bytes, cudaStream_t stream);

/* Paged decode attention for `batch` independent sequences, one query token each
 * (the reference's jac_launch applied per sequence: crates/jac-codegen-cuda/src/variants.rs:2441-2509,
 * :2593-2601). q f16 [batch, NH, D]; out f32 [batch, NH, D]; seq_lens i32 [batch] on the device;
 * max_seq_len is a host upper bound used to size the launch and check the block-table width. */
int kivi_b200_decode(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                     const int32_t* block_tables, int max_blocks_per_seq, const int32_t* seq_lens,
                     const int32_t* slot_ids, int batch, int max_seq_len, float* out,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream);

/* The same call with the result stored as fp16 (out f16 [batch, NH, D]): what a serving engine hands to the
 * O projection, and half the bytes when the result leaves the device. Accumulation and normalisation are in
 * fp32 as above; only the final store rounds. The reference's launch contract has fp32 output only
 * (integrations/vllm_kivi/bindings.py:117), so this form has no counterpart there. */
int kivi_b200_decode_f16(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                     const int32_t* block_tables, int max_blocks_per_seq, const int32_t* seq_lens,
                     const int32_t* slot_ids, int batch, int max_seq_len, kivi_f16* out,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream);

/* Sparse-retained decode for `batch` sequences (the reference's jac_launch_sparse_retained applied per
 * sequence: crates/jac-codegen-cuda/src/variants.rs:2620-2691, :2737-2742; tables built by the page-aware
 * allocator, integrations/vllm_kivi/source_patch.py:1839-1900). Row i of retained_block_tables is sequence
 * i's COMPACT table: its first retained_pages[i] entries are the old pages still kept, in their original
 * order; a sequence scans min(retained_pages[i], its dense old pages, max_blocks_per_seq) of them and then
 * its fp16 residual, whose bounds still follow the dense seq_lens[i]. retained_pages is a device array, so a
 * batch can mix sequences that dropped pages with dense ones (give those their dense table and a count at
 * least as large as their dense page count). The tensor-core kernel covers group_size == block_size; other
 * geometries run the generic kernel. Everything else as kivi_b200_decode. */
int kivi_b200_decode_sparse(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                            const int32_t* retained_block_tables, int max_blocks_per_seq,
                            const int32_t* seq_lens, const int32_t* retained_pages, const int32_t* slot_ids,
                            int batch, int max_seq_len, float* out, void* workspace, size_t workspace_bytes,
                            cudaStream_t stream);

/* Decode for callers that cannot allocate device memory. Some hosts of this library hand it
 * buffers but have no allocator of their own to ask for a workspace: a serving runtime whose memory
 * pool was sized and frozen at start-up, a plugin running inside someone else's captured step, a
 * C caller with no CUDA allocation rights in its sandbox. This entry point (no counterpart in the
 * reference, which never splits the context and so needs no scratch) is kivi_b200_decode with the
 * split-context scratch taken from a fixed array inside the library instead of from the caller:
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine;
 *   - the array is KIVI_B200_NOALLOC_SCRATCH_BYTES long and every GPU that loads the library holds
 *     it until the process exits; a (batch, max_seq_len) whose launch plan needs more is refused
 *     with KIVI_ERR_WORKSPACE and nothing is launched (kivi_b200_decode_workspace_bytes tells the
 *     need in advance);
 *   - the first call on each device, made with that device current, looks the array's device
 *     address up (once per device, safe against two threads calling first at the same time; the address
 *     is kept until the process exits, so do not cudaDeviceReset between calls); make that first call
 *     before any stream capture begins;
 *   - every call uses the same array: two calls whose kernels can overlap on the GPU (different
 *     streams, different host threads) race on it. Calls on one stream are safe back to back;
 *     nothing in the array has to be cleared between them (a call reads only partials it wrote).
 * Arguments and results are those of kivi_b200_decode. */
#define KIVI_B200_NOALLOC_SCRATCH_BYTES (1u << 20)
int kivi_b200_decode_noalloc(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                             const int32_t* block_tables, int max_blocks_per_seq, const int32_t* seq_lens,
                             const int32_t* slot_ids, int batch, int max_seq_len, float* out,
                             cudaStream_t stream);

/* How kivi_b200_decode would cut a launch of `batch` sequences of at most max_seq_len tokens into jobs (one
 * CTA each), for callers and tests that want to see the plan: plan_out = {units1, k1, units2, k2}: the first
 * units1 (sequence, kv head) units are cut into k1 parts each, the other units2 into k2 parts; parts of a cut
 * unit leave partials in the workspace that a second kernel merges. Pure host arithmetic. No counterpart in
 * the reference, which runs one warp per query head over the whole context. */
int kivi_b200_decode_plan(const kivi_geometry* geom, int batch, int max_seq_len, int32_t plan_out[4]);

/* What part `part` of `parts` of a sequence of seq_len tokens holds under that plan: items_out = {g0, g1, t0, t1},
 * the key groups [g0, g1) and the 16-row tiles [t0, t1) of the fp16 residual. Over part = 0 .. parts - 1 these
 * ranges tile the sequence's groups and tiles exactly once. The arithmetic the kernel itself runs, exported
 * for tests. No counterpart in the reference. */
int kivi_b200_decode_part_items(const kivi_geometry* geom, int seq_len, int part, int parts, int32_t items_out[4]);

/* Page ids (block tables) and slot ids are read from device memory and become addresses. The v2 calls hold them
 * against kivi_cache.num_blocks / num_slots inside the kernels: the writer leaves a sequence untouched when its
 * slot or one of the pages the write would pack into lies outside the pool; the decode reads page / slot 0
 * instead (that sequence's output is then meaningless) -- nothing outside the pools is accessed either way.
 * These report how many such sequences (writer) and ids (decode) were met since the library was loaded on the
 * current device; 0 in any healthy run. The reference checks neither (its signatures carry no pool sizes, and
 * the reference-lane symbols here cannot check for the same reason). Synchronise the device. */
int kivi_b200_writer_rejected_indices(uint32_t* count_out);
int kivi_b200_decode_rejected_indices(uint32_t* count_out);

/* The tensor-core decode kernel waits on shared-memory barriers for its staged pages; every such wait is
 * bounded. A CTA whose wait gave up drains its copies, counts itself here and leaves (the launch's output is
 * then undefined). Writes the number of such CTAs since the library was loaded on the current device (0 in
 * any healthy run) to *failures_out; synchronises the device. No counterpart in the reference, whose kernels
 * have no asynchronous staging. */
int kivi_b200_decode_wait_failures(uint32_t* failures_out);

/* fp16 GEMV / skinny GEMM of the generated decode runtime: y[b, o] = sum_i W[o, i] * x[b, i],
 * W row-major [out_dim, in_dim], fp32 accumulation (reference: gemv(),
 * crates/jac-codegen-cuda/src/templates/runtime.cu:15-26, a cublasGemmEx call). 1 <= batch <= 64.
 * in_dim % 8 == 0. Exactly one of y_f16 / y_f32 may be NULL; y_f32 is the kernel-DSL form
 * (crates/jac-codegen-cuda/src/variants.rs:318-329). Batches of 5..64 columns with in_dim % 64 == 0
 * run as a tensor-core skinny GEMM (tcgen05, tiles moved by TMA, accumulators in tensor memory) that
 * splits the contraction over a thread-block cluster and reduces through distributed shared memory;
 * w and x must then be 16-byte aligned. No call of this entry point allocates. */
int kivi_b200_gemv_f16(const kivi_f16* w, const kivi_f16* x, kivi_f16* y_f16, float* y_f32,
                       int out_dim, int in_dim, int batch, cudaStream_t stream);

/* The skinny GEMM waits on shared-memory barriers for its copies and tensor-core operations; every such
 * wait is bounded, and a CTA whose wait gave up runs to its end (result undefined) and counts itself
 * here. Writes the number of such CTAs since the library was loaded on the current device (0 in any
 * healthy run) to *failures_out; synchronises the device. */
int kivi_b200_gemm_wait_failures(uint32_t* failures_out);

/* ------------------------------------------------------------------ ABI v1 (reference lane) -- */

/* ---------------------------------------------------------------------------------------------
 * Decode step of the generated runtime around the KIVI cache.
 *
 * forward() of crates/jac-codegen-cuda/src/templates/runtime.cu:125-187 runs one token through
 * embed -> L x [RMSNorm, fused QKV projection (+bias), RoPE, KV store, attention, O projection,
 * residual add, RMSNorm, fused gate|up projection, SiLU(gate)*up, down projection, residual add]
 * -> RMSNorm -> lm_head, with the kernels of templates/kernels.cu:4-227 between cuBLAS GEMVs and
 * an fp16 KV cache [L, NKV, MAX_SEQ, HD]. kivi_b200_decode_step is that step for `batch`
 * sequences at once with the fp16 cache replaced by the int4-KIVI paged cache (one kivi_cache per
 * layer; all layers share the block tables, the sequence lengths and the scratch slot ids) and
 * the arg-max of kernels.cu:203-227 at the end. Arithmetic follows the reference kernels
 * (fp16 storage of every intermediate, fp32 inside a kernel; RMSNorm, SiLU, bias and residual add
 * are bit-identical to the reference kernels on the same GPU, RoPE too up to rare one-ulp
 * differences at large positions; the projections are fp32-accumulated like the cuBLAS call they
 * replace, in a different summation order).
 *
 * Weights use the reference's file layout (templates/export.py:69-92, loader runtime.cu:59-97):
 * row-major [out, in]; qkv = q|k|v rows fused; gate_up = gate|up rows fused.
 *
 * Tensor parallelism over KV heads (no counterpart in the reference): rank r of tp_size holds the
 * query/key/value rows of its KV heads, the matching columns of `o`, FFN/tp_size gate and up rows,
 * the matching columns of `down` and VOCAB/tp_size rows of lm_head; the head, FFN and vocabulary
 * counts in kivi_step_config are those LOCAL sizes. The two partial projections per layer are
 * summed across ranks, and the per-rank arg-max candidates gathered, through kivi_step_comm.
 * --------------------------------------------------------------------------------------------- */
typedef struct kivi_step_config {
    int32_t layers;
    int32_t hidden;        /* H (global) */
    int32_t num_q_heads;   /* local NH */
    int32_t num_kv_heads;  /* local NKV */
    int32_t head_dim;
    int32_t ffn;           /* local FFN rows of gate and of up */
    int32_t vocab;         /* local lm_head rows */
    int32_t vocab_offset;  /* global id of local row 0 */
    int32_t attn_bias;     /* 1: qkv_bias is added after the QKV projection (Config::ATTN_BIAS) */
    float rope_base;       /* Config::ROPE_BASE */
    float norm_eps;        /* Config::NORM_EPS */
    int32_t block_size;    /* KIVI page geometry, as in kivi_geometry */
    int32_t group_size;
    int32_t residual;
    int32_t tp_size;       /* 1 = no tensor parallelism */
    int32_t tp_rank;
} kivi_step_config;

typedef struct kivi_layer_weights {
    const kivi_f16* attn_norm;  /* [H] */
    const kivi_f16* qkv;        /* [(NH + 2 NKV) * D, H] */
    const kivi_f16* qkv_bias;   /* [(NH + 2 NKV) * D] or NULL */
    const kivi_f16* o;          /* [H, NH * D] */
    const kivi_f16* ffn_norm;   /* [H] */
    const kivi_f16* gate_up;    /* [2 * FFN, H] */
    const kivi_f16* down;       /* [H, FFN] */
} kivi_layer_weights;

typedef struct kivi_step_weights {
    const kivi_f16* embed;               /* [VOCAB_GLOBAL, H], replicated on every rank */
    const kivi_f16* final_norm;          /* [H] */
    const kivi_f16* lm_head;             /* [VOCAB, H] */
    const kivi_layer_weights* layers;    /* host array [layers] of device pointers */
} kivi_step_weights;

typedef struct kivi_step_state {
    const kivi_cache* caches;        /* host array [layers] */
    const int32_t* block_tables;     /* device [batch, max_blocks_per_seq] */
    int32_t max_blocks_per_seq;
    int32_t* seq_lens;               /* device [batch]: tokens already cached; the step adds one to each */
    const int32_t* slot_ids;         /* device [batch] or NULL (slot i for sequence i) */
    void* workspace;                 /* device, kivi_b200_decode_step_workspace_bytes, zeroed once */
    size_t workspace_bytes;
} kivi_step_state;

/* Collectives for tp_size > 1, one of two forms.
 *
 * Hooks: the caller's all-reduce (fp16 sum, in place) and all-gather, run on `stream`, 0 on success
 * (an NCCL communicator, torch.distributed, ...).
 *
 * Peer memory (peer_regions != NULL; the hooks are then unused): the library's own exchange over
 * NVLink. Every rank creates one region of kivi_b200_p2p_region_bytes() bytes with
 * kivi_b200_p2p_region_create(), hands the returned handle to the other ranks (any host channel),
 * opens theirs with kivi_b200_p2p_region_open() and passes the tp_size pointers, own region at
 * index tp_rank, in rank order. A rank pushes its partial projection into its slot in every
 * region with plain peer stores of 8-byte words, each carrying 32 bits of data and the 32-bit sequence
 * number of the exchange, so a word is entirely old or entirely new and there is no separate flag; the
 * kernel that consumes the sum (residual add + RMSNorm) polls the words of the tp_size slots until they
 * carry the current number and adds them up in rank order in fp32, so every
 * rank gets the same bits and the reduction has no launch of its own. Waits are bounded: a rank
 * that never delivers ends the wait after about a second and sets its bit in the region's status
 * word (kivi_b200_p2p_status), the step's result is then undefined but nothing hangs. All ranks
 * must have opened all regions before the first step, and must step in lockstep (same batch). */
typedef int (*kivi_allreduce_f16_fn)(void* user, kivi_f16* buf, size_t count, cudaStream_t stream);
typedef int (*kivi_allgather_fn)(void* user, const void* send, void* recv, size_t bytes_per_rank,
                                 cudaStream_t stream);
typedef struct kivi_step_comm {
    kivi_allreduce_f16_fn allreduce_f16;
    kivi_allgather_fn allgather;
    void* user;
    void* const* peer_regions;   /* host array [tp_size] of device pointers, or NULL for the hooks */
    size_t region_bytes;         /* size every region was created with */
    uint32_t spin_limit;         /* polls before a wait gives up; 0 = the library's default */
} kivi_step_comm;

#define KIVI_B200_P2P_HANDLE_BYTES 64
size_t kivi_b200_p2p_region_bytes(const kivi_step_config* cfg, int batch);
/* cudaMalloc + zero fill on the current device; handle_out receives KIVI_B200_P2P_HANDLE_BYTES bytes. */
int kivi_b200_p2p_region_create(size_t bytes, void** region, unsigned char* handle_out);
int kivi_b200_p2p_region_open(const unsigned char* handle, void** peer_region);
int kivi_b200_p2p_region_close(void* peer_region);
int kivi_b200_p2p_region_destroy(void* region);
/* Copies the region's status word to the host (synchronises `stream`): 0 = every wait was served. */
int kivi_b200_p2p_status(const void* region, uint32_t* status_out, cudaStream_t stream);

size_t kivi_b200_decode_step_workspace_bytes(const kivi_step_config* cfg, int batch, int max_seq_len);

/* One decode step. tokens_in / tokens_out: device int32 [batch] (global token ids; they may alias).
 * logits_out: optional device fp16 [batch, vocab] (local rows). max_seq_len bounds every sequence
 * length AFTER the step (launch planning; a captured graph stays valid while the bound holds).
 * The whole step is stream-ordered and allocation-free, so it can be captured in a CUDA graph. */
int kivi_b200_decode_step(const kivi_step_config* cfg, const kivi_step_weights* weights,
                          const kivi_step_state* state, const int32_t* tokens_in, int batch,
                          int max_seq_len, int32_t* tokens_out, kivi_f16* logits_out,
                          const kivi_step_comm* comm, cudaStream_t stream);

/* The step's element-wise kernels on their own (parity tests against the reference kernels):
 * rows of `hidden` (resp. heads, `n`) fp16 values, `batch` rows.
 *   residual_rmsnorm: x_out = x + delta (delta may be NULL); normed = RMSNorm(x_out) * weight
 *                     (kernels.cu:10-33 after vadd, :156-159)
 *   bias_rope:        qkv (+bias) -> RoPE on q and k heads at positions[b] (kernels.cu:40-54, :163-166)
 *                     written split as q [batch, NH*D], k and v [batch, NKV*D]
 *   silu_mul:         out = SiLU(gate) * up for gate_up rows [gate | up] (kernels.cu:146-153)
 *   argmax:           first index of the row maximum (kernels.cu:203-227) */
int kivi_b200_residual_rmsnorm(const kivi_f16* x, const kivi_f16* delta, const kivi_f16* weight,
                               kivi_f16* x_out, kivi_f16* normed, int batch, int hidden, float eps,
                               cudaStream_t stream);
int kivi_b200_bias_rope(const kivi_f16* qkv, const kivi_f16* bias, const int32_t* positions,
                        kivi_f16* q, kivi_f16* k, kivi_f16* v, int batch, int num_q_heads,
                        int num_kv_heads, int head_dim, float rope_base, cudaStream_t stream);
int kivi_b200_silu_mul(const kivi_f16* gate_up, kivi_f16* out, int batch, int ffn, cudaStream_t stream);
int kivi_b200_argmax(const kivi_f16* logits, int32_t* out_index, int batch, int n, void* workspace,
                     size_t workspace_bytes, cudaStream_t stream);


/* Replaces the emitted `jac_launch` of decode_attention_kivi_paged
 * (crates/jac-codegen-cuda/src/variants.rs:2593-2601; declared by the binding at
 * integrations/vllm_kivi/source_patch.py:570-576). One sequence, NH = 40 query heads. */
void jac_launch(const kivi_f16* Q, const int* BLOCK_TABLE,
                const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,
                const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,
                const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH,
                int SEQ_LEN, float* O, cudaStream_t stream);

/* TP=2 rank-local clone, NH/NKV 20/4 (integrations/vllm_kivi/dsl_decode.py:267-319;
 * source_patch.py:578-584). */
void jac_launch_tp2_local(const kivi_f16* Q, const int* BLOCK_TABLE,
                          const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,
                          const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,
                          const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH,
                          int SEQ_LEN, float* O, cudaStream_t stream);

/* Replaces `jac_launch_batched` (variants.rs:2891-2896; source_patch.py:609-615): NUM_QUERIES
 * (<= 160) queries of ONE sequence sharing BLOCK_TABLE and scratch, each with its own SEQ_LENS[i]. */
void jac_launch_batched(const kivi_f16* Q, const int* SEQ_LENS, const int* BLOCK_TABLE,
                        const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,
                        const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,
                        const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH,
                        int NUM_QUERIES, float* O, cudaStream_t stream);

void jac_launch_batched_tp2_local(const kivi_f16* Q, const int* SEQ_LENS, const int* BLOCK_TABLE,
                                  const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,
                                  const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,
                                  const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH,
                                  int NUM_QUERIES, float* O, cudaStream_t stream);

/* Replaces `jac_launch_sparse_retained` (variants.rs:2737-2742; source_patch.py:590-596): scans
 * NUM_RETAINED_PAGES pages of a compact table; the residual bound still comes from SEQ_LEN. */
void jac_launch_sparse_retained(const kivi_f16* Q, const int* RETAINED_BLOCK_TABLE,
                                const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,
                                const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,
                                const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH,
                                int SEQ_LEN, int NUM_RETAINED_PAGES, float* O, cudaStream_t stream);

void jac_launch_sparse_retained_tp2_local(const kivi_f16* Q, const int* RETAINED_BLOCK_TABLE,
                                          const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,
                                          const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,
                                          const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH,
                                          int SEQ_LEN, int NUM_RETAINED_PAGES, float* O, cudaStream_t stream);

/* Replaces `jac_launch_cache_write` (variants.rs:3226-3253; source_patch.py:645-650). SEQ_LEN is
 * the length after the new token. NKV = 8. */
void jac_launch_cache_write(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES, kivi_f16* K_ZERO_PAGES,
                            unsigned char* V_CODE_PAGES, kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                            kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                            const kivi_f16* NEW_K, const kivi_f16* NEW_V,
                            const int* BLOCK_TABLE, int SEQ_LEN, cudaStream_t stream);

/* Replaces `jac_launch_cache_write_batched` (variants.rs:3135-3167; source_patch.py:655-660).
 * NUM_NEW outside [1, 160] prints and exits like the reference; unlike the reference a chunk that
 * crosses several age-out boundaries is handled in the one call. */
void jac_launch_cache_write_batched(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES, kivi_f16* K_ZERO_PAGES,
                                    unsigned char* V_CODE_PAGES, kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                    kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                    const kivi_f16* NEW_K, const kivi_f16* NEW_V,
                                    const int* BLOCK_TABLE, int START_SEQ_LEN, int NUM_NEW, cudaStream_t stream);

/* C-callable forms of the reference's C++-linkage hand-CUDA writer
 * (kivi_cache_write_launch / kivi_cache_write_batched_launch, source_patch.py:624-637,
 * :1661-1666, :1737-1742). The library also exports those two names with C++ linkage and the
 * reference's exact parameter lists, so the reference's binding links against it unchanged.
 * NKV_RUNTIME is 8 or 4; SLOT_MAPPING is accepted and ignored, as in the reference. */
void kivi_b200_cache_write_launch(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES, kivi_f16* K_ZERO_PAGES,
                                  unsigned char* V_CODE_PAGES, kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                  kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                  const kivi_f16* NEW_K, const kivi_f16* NEW_V, const int64_t* SLOT_MAPPING,
                                  const int* BLOCK_TABLE, int seq_len, int NKV_RUNTIME, cudaStream_t stream);

void kivi_b200_cache_write_batched_launch(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES, kivi_f16* K_ZERO_PAGES,
                                          unsigned char* V_CODE_PAGES, kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                          kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                          const kivi_f16* NEW_K, const kivi_f16* NEW_V, const int64_t* SLOT_MAPPING,
                                          const int* BLOCK_TABLE, int START_SEQ_LEN, int NUM_NEW, int NKV_RUNTIME,
                                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* JACQ_KIVI_B200_H_ */
