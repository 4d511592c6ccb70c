/*
 * TEST INFRASTRUCTURE ONLY -- scalar CPU restatement of the int4-KIVI paged KV-cache path.
 *
 * This file is the checker for the CUDA library, never part of the product: only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may build, load or call it.
 *
 * It restates, for a runtime geometry, the arithmetic of the reference implementation
 * (ImpossibleComputing/jacq). Each function names the reference lines it follows:
 *
 *   writer  : integrations/vllm_kivi/source_patch.py:1517-1697 (hand-CUDA writer), which the
 *             reference asserts equal to crates/jac-codegen-cuda/src/variants.rs:2936-3067,
 *             :3226-3253 (DSL writer); batched form source_patch.py:1705-1775,
 *             planner source_patch.py:488-553.
 *   decode  : crates/jac-codegen-cuda/src/variants.rs:2316-2327 (unpack), :2338-2351 (page
 *             gather), :2359-2431 (recurrence), :2463-2502 (prologue/epilogue);
 *             snapshot tests/snapshots/kernels/decode_attention_kivi_paged_library_flash.cu.
 *   gemv    : crates/jac-codegen-cuda/src/templates/runtime.cu:15-26, variants.rs:318-329.
 *
 * Parity pin: the reference holds no numerical golden vectors for this path. This oracle is
 * pinned against outputs of the reference's own CUDA (compiled unmodified into oracle/_ref and
 * run on a B200); the vectors are committed under tests/golden/ with the script that made them.
 *
 * Generalisation beyond the reference lane (block == group == 32, head_dim 128), reducing to
 * it exactly when block == group:
 *   - age-out unit = one key group = G tokens = G/B pages; split_old = floor((T-R)/G)*G;
 *     scratch capacity R+G rows;
 *   - the key scale/zero of a group are stored in the [NKV, D] slot of every page of the group;
 *   - value channel-group width = min(G, D), HD_GROUPS = ceil(D / G).
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int32_t nh;   /* query heads */
    int32_t nkv;  /* kv heads */
    int32_t d;    /* head_dim */
    int32_t b;    /* page (block) tokens */
    int32_t g;    /* KIVI group */
    int32_t r;    /* fp16 residual window */
} kivi_geom;

/* ---------------------------------------------------------------- fp16 <-> fp32 ---------- */

/* IEEE binary16 -> binary32, exact. NaN maps to the canonical quiet NaN like cvt.f32.f16. */
static float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = man ? 0x7fffffffu : (sign | 0x7f800000u);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even; NaN -> 0x7fff (what __float2half produces). */
static uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return 0x7fffu;
    if (ax >= 0x477ff000u) {            /* >= 65520 rounds to inf; inf stays inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) {             /* <= 2^-25 rounds to zero (ties to even -> 0) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) {                      /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    return (uint16_t)(sign | (base + q));  /* carry into the exponent is the right answer */
}

/* min/max as the GPU's min.f32/max.f32: a NaN operand is dropped, -0 orders below +0. */
static float gmin(float a, float b) {
    if (a != a) return b;
    if (b != b) return a;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? a : b;
    return a < b ? a : b;
}
static float gmax(float a, float b) {
    if (a != a) return b;
    if (b != b) return a;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? b : a;
    return a > b ? a : b;
}

/* clamp_code of the reference (source_patch.py:1517-1522): int(rintf(x)) clamped to [0,15].
 * The float->int conversion saturates on the GPU and maps NaN to 0; written out here because
 * both are undefined in C. */
static int clamp_code(float x) {
    if (x != x) return 0;
    float r = rintf(x);
    if (r < 0.0f) return 0;
    if (r > 15.0f) return 15;
    return (int)r;
}

static inline uint8_t pack_codes(int lo, int hi) {
    return (uint8_t)((lo & 0x0f) | ((hi & 0x0f) << 4));
}

/* ---------------------------------------------------------------- geometry --------------- */

static int hd_groups(const kivi_geom* gm) { return (gm->d + gm->g - 1) / gm->g; }
static int vgroup_width(const kivi_geom* gm) { return gm->g < gm->d ? gm->g : gm->d; }

int kivi_oracle_validate(const kivi_geom* gm) {
    if (gm->nh <= 0 || gm->nkv <= 0 || gm->d <= 0 || gm->b <= 0 || gm->g <= 0 || gm->r < 0) return 1;
    if (gm->nh % gm->nkv) return 2;
    if (gm->d % 2) return 3;
    if (gm->g % gm->b) return 4;
    if (gm->d % vgroup_width(gm)) return 5;
    return 0;
}

/* split_old_tokens (source_patch.py:1655-1659), with the group as the age-out unit. */
int kivi_oracle_split_old(const kivi_geom* gm, int seq_len) {
    int q = seq_len - gm->r;
    if (q < 0) return 0;
    return (q / gm->g) * gm->g;
}

/* ---------------------------------------------------------------- writer ----------------- */

typedef struct {
    uint8_t* k_code;   /* [num_blocks, NKV, B, D/2] */
    uint16_t* k_scale; /* [num_blocks, NKV, D] */
    uint16_t* k_zero;
    uint8_t* v_code;
    uint16_t* v_scale; /* [num_blocks, NKV, B, HD_GROUPS] */
    uint16_t* v_zero;
} kivi_pages;

/* pack_key_age_out_page_kernel (source_patch.py:1532-1581): per (head, channel) min/max over the
 * group's G scratch rows, scale = (max-min)/15, zero = min, codes from the unrounded fp32
 * scale/zero; params replicated into each of the group's G/B pages. */
static void age_out_keys(const kivi_geom* gm, const kivi_pages* pg, const uint16_t* k_scratch,
                         const int32_t* block_table, int first_logical_page) {
    const int D = gm->d, B = gm->b, G = gm->g, NKV = gm->nkv, RS = gm->r + gm->g;
    const int pages = G / B;
    for (int h = 0; h < NKV; ++h) {
        for (int d = 0; d < D; ++d) {
            float mn = h2f(k_scratch[((size_t)h * RS) * D + d]);
            float mx = mn;
            for (int t = 1; t < G; ++t) {
                float x = h2f(k_scratch[((size_t)h * RS + t) * D + d]);
                mn = gmin(mn, x);
                mx = gmax(mx, x);
            }
            float scale = (mx - mn) / 15.0f;
            if (!(scale > 0.0f)) scale = 1.0f;
            for (int p = 0; p < pages; ++p) {
                size_t page = (size_t)block_table[first_logical_page + p];
                pg->k_scale[(page * NKV + h) * D + d] = f2h(scale);
                pg->k_zero[(page * NKV + h) * D + d] = f2h(mn);
            }
            for (int t = 0; t < G; ++t) {
                float x = h2f(k_scratch[((size_t)h * RS + t) * D + d]);
                int code = clamp_code((x - mn) / scale);
                size_t page = (size_t)block_table[first_logical_page + t / B];
                uint8_t* byte = &pg->k_code[((page * NKV + h) * B + (t % B)) * (D / 2) + d / 2];
                if (d & 1) *byte = (uint8_t)((*byte & 0x0f) | ((code & 0x0f) << 4));
                else       *byte = (uint8_t)((*byte & 0xf0) | (code & 0x0f));
            }
        }
    }
}

/* pack_value_age_out_page_kernel (source_patch.py:1583-1620): per (head, token, channel group)
 * min/max over the group's channels. */
static void age_out_values(const kivi_geom* gm, const kivi_pages* pg, const uint16_t* v_scratch,
                           const int32_t* block_table, int first_logical_page) {
    const int D = gm->d, B = gm->b, G = gm->g, NKV = gm->nkv, RS = gm->r + gm->g;
    const int HG = hd_groups(gm), VG = vgroup_width(gm);
    for (int h = 0; h < NKV; ++h) {
        for (int t = 0; t < G; ++t) {
            size_t page = (size_t)block_table[first_logical_page + t / B];
            int off = t % B;
            const uint16_t* row = v_scratch + ((size_t)h * RS + t) * D;
            for (int cg = 0; cg < HG; ++cg) {
                int d_base = cg * VG;
                float mn = h2f(row[d_base]);
                float mx = mn;
                for (int c = 1; c < VG; ++c) {
                    float x = h2f(row[d_base + c]);
                    mn = gmin(mn, x);
                    mx = gmax(mx, x);
                }
                float scale = (mx - mn) / 15.0f;
                if (!(scale > 0.0f)) scale = 1.0f;
                size_t param = ((page * NKV + h) * B + off) * HG + cg;
                pg->v_scale[param] = f2h(scale);
                pg->v_zero[param] = f2h(mn);
                for (int c = 0; c < VG; c += 2) {
                    int d0 = d_base + c;
                    int c0 = clamp_code((h2f(row[d0]) - mn) / scale);
                    int c1 = clamp_code((h2f(row[d0 + 1]) - mn) / scale);
                    pg->v_code[((page * NKV + h) * B + off) * (D / 2) + d0 / 2] = pack_codes(c0, c1);
                }
            }
        }
    }
}

/* shift_scratch_after_age_out_kernel (source_patch.py:1635-1648): rows [G, G+len) -> [0, len). */
static void shift_scratch(const kivi_geom* gm, uint16_t* k_scratch, uint16_t* v_scratch, int len) {
    const int D = gm->d, G = gm->g, NKV = gm->nkv, RS = gm->r + gm->g;
    for (int h = 0; h < NKV; ++h) {
        for (int r = 0; r < len; ++r) {
            memmove(k_scratch + ((size_t)h * RS + r) * D, k_scratch + ((size_t)h * RS + r + G) * D, (size_t)D * 2);
            memmove(v_scratch + ((size_t)h * RS + r) * D, v_scratch + ((size_t)h * RS + r + G) * D, (size_t)D * 2);
        }
    }
}

static void append_rows(const kivi_geom* gm, uint16_t* k_scratch, uint16_t* v_scratch,
                        const uint16_t* new_k, const uint16_t* new_v, int row0, int n) {
    const int D = gm->d, NKV = gm->nkv, RS = gm->r + gm->g;
    for (int t = 0; t < n; ++t)
        for (int h = 0; h < NKV; ++h) {
            memcpy(k_scratch + ((size_t)h * RS + row0 + t) * D, new_k + ((size_t)t * NKV + h) * D, (size_t)D * 2);
            memcpy(v_scratch + ((size_t)h * RS + row0 + t) * D, new_v + ((size_t)t * NKV + h) * D, (size_t)D * 2);
        }
}

/* kivi_cache_write_batched_launch (source_patch.py:1737-1775): append num_new rows, then at most
 * one age-out. The caller keeps start..start+num_new within one boundary (plan_batched_write).
 * Returns 0, or 1 if the chunk would overflow the scratch or cross more than one boundary. */
int kivi_oracle_write_batched(const kivi_geom* gm, kivi_pages* pg, uint16_t* k_scratch, uint16_t* v_scratch,
                              const uint16_t* new_k, const uint16_t* new_v, const int32_t* block_table,
                              int start_seq_len, int num_new) {
    int prev_old = kivi_oracle_split_old(gm, start_seq_len);
    int prev_res = start_seq_len - prev_old;
    int end = start_seq_len + num_new;
    int next_old = kivi_oracle_split_old(gm, end);
    if (num_new < 1 || prev_res + num_new > gm->r + gm->g) return 1;
    if (next_old - prev_old > gm->g) return 1;
    append_rows(gm, k_scratch, v_scratch, new_k, new_v, prev_res, num_new);
    if (next_old > prev_old) {
        int lp = prev_old / gm->b;
        age_out_keys(gm, pg, k_scratch, block_table, lp);
        age_out_values(gm, pg, v_scratch, block_table, lp);
        shift_scratch(gm, k_scratch, v_scratch, end - next_old);
    }
    return 0;
}

/* kivi_cache_write_launch (source_patch.py:1661-1697): seq_len is the length AFTER the token. */
int kivi_oracle_write_token(const kivi_geom* gm, kivi_pages* pg, uint16_t* k_scratch, uint16_t* v_scratch,
                            const uint16_t* new_k, const uint16_t* new_v, const int32_t* block_table,
                            int seq_len) {
    return kivi_oracle_write_batched(gm, pg, k_scratch, v_scratch, new_k, new_v, block_table, seq_len - 1, 1);
}

/* A chunk of any length == the single-token writer applied token by token. */
int kivi_oracle_write_tokens(const kivi_geom* gm, kivi_pages* pg, uint16_t* k_scratch, uint16_t* v_scratch,
                             const uint16_t* new_k, const uint16_t* new_v, const int32_t* block_table,
                             int start_seq_len, int num_new) {
    const size_t per_tok = (size_t)gm->nkv * gm->d;
    for (int t = 0; t < num_new; ++t) {
        int rc = kivi_oracle_write_token(gm, pg, k_scratch, v_scratch, new_k + t * per_tok, new_v + t * per_tok,
                                         block_table, start_seq_len + t + 1);
        if (rc) return rc;
    }
    return 0;
}

/* plan_batched_write (source_patch.py:504-553): cut a chunk so each piece crosses at most one
 * age-out boundary. Writes up to max_out (start, num_new) pairs; returns the number of pieces
 * or -1 on bad arguments / overflow of max_out. */
int kivi_oracle_plan_batched_write(const kivi_geom* gm, int start_seq_len, int num_new,
                                   int32_t* out_start, int32_t* out_num, int max_out) {
    if (start_seq_len < 0 || num_new < 1) return -1;
    int cap = gm->r + gm->g, seq = start_seq_len, remaining = num_new, n = 0;
    while (remaining > 0) {
        int prev_res = seq - kivi_oracle_split_old(gm, seq);
        int take = cap - prev_res;
        if (take > remaining) take = remaining;
        if (take <= 0 || n >= max_out) return -1;
        out_start[n] = seq;
        out_num[n] = take;
        ++n;
        seq += take;
        remaining -= take;
    }
    return n;
}

/* ---------------------------------------------------------------- decode ----------------- */

/* Bounds of variants.rs:2486-2495 for a runtime geometry. max_old_tokens is the reference's LQ
 * cap (pass a negative value for "no cap"). */
static void decode_bounds(const kivi_geom* gm, int seq_len, int max_old_tokens, int* old_valid, int* res_valid) {
    int bounded = seq_len < 0 ? 0 : seq_len;
    if (max_old_tokens >= 0 && bounded > max_old_tokens + gm->r) bounded = max_old_tokens + gm->r;
    int ov = kivi_oracle_split_old(gm, bounded);
    if (max_old_tokens >= 0 && ov > max_old_tokens) ov = max_old_tokens;
    int rv = bounded - ov;
    if (rv < 0) rv = 0;
    if (rv > gm->r + gm->g) rv = gm->r + gm->g;
    *old_valid = ov;
    *res_valid = rv;
}

/* One (sequence, query head). mode 0: the reference's single-pass online softmax in token order,
 * fp32 with fmaf dequant (variants.rs:2359-2431). mode 1: independent two-pass softmax over
 * fp32-dequantised K/V with double accumulation (pattern of specs/kernels/paged_attn/reference.cu).
 * num_retained_pages >= 0 selects the sparse-retained form (variants.rs:2620-2691): scan that
 * many pages of a compact table, residual bound from the dense seq_len. */
static void decode_head(const kivi_geom* gm, const kivi_pages* pg, const uint16_t* q, const int32_t* block_table,
                        const uint16_t* k_scratch, const uint16_t* v_scratch, int seq_len, int max_old_tokens,
                        int num_retained_pages, int h, int mode, float* out) {
    const int D = gm->d, B = gm->b, NKV = gm->nkv, RS = gm->r + gm->g;
    const int HG = hd_groups(gm), VG = vgroup_width(gm);
    const int kv = h / (gm->nh / gm->nkv);
    int old_valid, res_valid;
    decode_bounds(gm, seq_len, max_old_tokens, &old_valid, &res_valid);
    if (num_retained_pages >= 0) {
        int dense_pages = old_valid / B;
        int rp = num_retained_pages > dense_pages ? dense_pages : num_retained_pages;
        old_valid = rp * B;
    }
    const float scale_attn = 1.0f / sqrtf((float)D);
    const int total = old_valid + res_valid;
    float* kd = (float*)malloc(sizeof(float) * D);
    float* vd = (float*)malloc(sizeof(float) * D);
    float* scores = mode ? (float*)malloc(sizeof(float) * (total > 0 ? total : 1)) : NULL;
    double* acc_d = mode ? (double*)calloc(D, sizeof(double)) : NULL;
    float m = -1.0e30f, l = 0.0f;
    float* acc = (float*)calloc(D, sizeof(float));
    double mx = -1.0e30, denom = 0.0;

    for (int pass = 0; pass < (mode ? 2 : 1); ++pass) {
        if (mode && pass == 1) {
            for (int s = 0; s < total; ++s) if (scores[s] > mx) mx = scores[s];
        }
        for (int s = 0; s < total; ++s) {
            if (s < old_valid) {
                int lp = s / B, off = s - lp * B;
                size_t page = (size_t)block_table[lp];
                const uint16_t* ks = pg->k_scale + (page * NKV + kv) * D;
                const uint16_t* kz = pg->k_zero + (page * NKV + kv) * D;
                const uint8_t* kc = pg->k_code + ((page * NKV + kv) * B + off) * (D / 2);
                const uint8_t* vc = pg->v_code + ((page * NKV + kv) * B + off) * (D / 2);
                const uint16_t* vs = pg->v_scale + ((page * NKV + kv) * B + off) * HG;
                const uint16_t* vz = pg->v_zero + ((page * NKV + kv) * B + off) * HG;
                for (int d = 0; d < D; ++d) {
                    int kcode = (d & 1) ? (kc[d / 2] >> 4) : (kc[d / 2] & 0x0f);
                    int vcode = (d & 1) ? (vc[d / 2] >> 4) : (vc[d / 2] & 0x0f);
                    kd[d] = fmaf((float)kcode, h2f(ks[d]), h2f(kz[d]));
                    vd[d] = fmaf((float)vcode, h2f(vs[d / VG]), h2f(vz[d / VG]));
                }
            } else {
                int r = s - old_valid;
                for (int d = 0; d < D; ++d) {
                    kd[d] = h2f(k_scratch[((size_t)kv * RS + r) * D + d]);
                    vd[d] = h2f(v_scratch[((size_t)kv * RS + r) * D + d]);
                }
            }
            if (!mode) {
                float part = 0.0f;
                for (int d = 0; d < D; ++d) part += h2f(q[(size_t)h * D + d]) * kd[d];
                float score = part * scale_attn;
                float m_new = m > score ? m : score;
                float corr = expf(m - m_new);
                float p = expf(score - m_new);
                l = l * corr + p;
                for (int d = 0; d < D; ++d) acc[d] = acc[d] * corr + p * vd[d];
                m = m_new;
            } else if (pass == 0) {
                double part = 0.0;
                for (int d = 0; d < D; ++d) part += (double)h2f(q[(size_t)h * D + d]) * (double)kd[d];
                scores[s] = (float)(part * (double)scale_attn);
            } else {
                double p = exp((double)scores[s] - mx);
                denom += p;
                for (int d = 0; d < D; ++d) acc_d[d] += p * (double)vd[d];
            }
        }
    }
    if (!mode) {
        float inv_l = 1.0f / (l > 1.0e-30f ? l : 1.0e-30f);
        for (int d = 0; d < D; ++d) out[(size_t)h * D + d] = acc[d] * inv_l;
    } else {
        double inv = 1.0 / (denom > 1.0e-30 ? denom : 1.0e-30);
        for (int d = 0; d < D; ++d) out[(size_t)h * D + d] = (float)(acc_d[d] * inv);
    }
    free(kd); free(vd); free(acc);
    if (scores) free(scores);
    if (acc_d) free(acc_d);
}

/* jac_launch of the paged decode (variants.rs:2593-2601): one sequence, all NH heads. */
void kivi_oracle_decode(const kivi_geom* gm, const kivi_pages* pg, const uint16_t* q, const int32_t* block_table,
                        const uint16_t* k_scratch, const uint16_t* v_scratch, int seq_len, int max_old_tokens,
                        int num_retained_pages, int mode, float* out) {
    for (int h = 0; h < gm->nh; ++h)
        decode_head(gm, pg, q, block_table, k_scratch, v_scratch, seq_len, max_old_tokens, num_retained_pages, h, mode, out);
}

/* Multi-sequence form: sequence i has its own block-table row, scratch slot and seq_len; this is
 * the reference applied independently per sequence (source_patch.py:3105-3288). Parallel over
 * (sequence, query head) with OpenMP when nthreads > 1; also the timed CPU baseline. */
void kivi_oracle_decode_batch(const kivi_geom* gm, const kivi_pages* pg, const uint16_t* q,
                              const int32_t* block_tables, int bt_stride, const int32_t* seq_lens,
                              const int32_t* slot_ids, const uint16_t* k_scratch, const uint16_t* v_scratch,
                              int batch, int max_old_tokens, int mode, int nthreads, float* out) {
    const size_t slot_elems = (size_t)gm->nkv * (gm->r + gm->g) * gm->d;
    const int items = batch * gm->nh;
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
    for (int it = 0; it < items; ++it) {
        int i = it / gm->nh, h = it % gm->nh;
        int slot = slot_ids ? slot_ids[i] : i;
        decode_head(gm, pg, q + (size_t)i * gm->nh * gm->d, block_tables + (size_t)i * bt_stride,
                    k_scratch + slot * slot_elems, v_scratch + slot * slot_elems, seq_lens[i], max_old_tokens, -1,
                    h, mode, out + (size_t)i * gm->nh * gm->d);
    }
}

/* Multi-sequence writer: sequence i appends new rows [offsets[i], offsets[i+1]) of new_k/new_v
 * starting from start_seq_lens[i], token by token. */
int kivi_oracle_write_batch(const kivi_geom* gm, kivi_pages* pg, uint16_t* k_scratch, uint16_t* v_scratch,
                            const uint16_t* new_k, const uint16_t* new_v, const int32_t* block_tables, int bt_stride,
                            const int32_t* start_seq_lens, const int32_t* offsets, const int32_t* slot_ids,
                            int batch, int nthreads) {
    const size_t slot_elems = (size_t)gm->nkv * (gm->r + gm->g) * gm->d;
    const size_t per_tok = (size_t)gm->nkv * gm->d;
    int bad = 0;
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads) reduction(| : bad)
    for (int i = 0; i < batch; ++i) {
        int slot = slot_ids ? slot_ids[i] : i;
        bad |= kivi_oracle_write_tokens(gm, pg, k_scratch + slot * slot_elems, v_scratch + slot * slot_elems,
                                        new_k + offsets[i] * per_tok, new_v + offsets[i] * per_tok,
                                        block_tables + (size_t)i * bt_stride, start_seq_lens[i],
                                        offsets[i + 1] - offsets[i]);
    }
    return bad;
}

/* ---------------------------------------------------------------- gemv ------------------- */

/* gemv() of the generated runtime (templates/runtime.cu:15-26): y = W x, W row-major [out, in],
 * fp16 operands, fp32 accumulation. y_f16 and/or y_f32 may be NULL; the fp32 result is the
 * kernel-DSL form (variants.rs:318-329). Batched: x [batch, in], y [batch, out]. */
void kivi_oracle_gemv(const uint16_t* w, const uint16_t* x, uint16_t* y_f16, float* y_f32,
                      int out_dim, int in_dim, int batch, int nthreads) {
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(static) num_threads(nthreads)
    for (int o = 0; o < out_dim; ++o) {
        for (int bi = 0; bi < batch; ++bi) {
            float acc = 0.0f;
            for (int i = 0; i < in_dim; ++i)
                acc += h2f(w[(size_t)o * in_dim + i]) * h2f(x[(size_t)bi * in_dim + i]);
            if (y_f32) y_f32[(size_t)bi * out_dim + o] = acc;
            if (y_f16) y_f16[(size_t)bi * out_dim + o] = f2h(acc);
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * Element-wise kernels of the generated decode runtime (templates/kernels.cu), restated per row
 * for a batch of rows. Each keeps the reference's fp32 expression and, for the RMSNorm sum, its
 * reduction order, so the only differences from the reference on a GPU are those of the device
 * math library (rsqrtf, powf, cosf, sinf, expf are not correctly rounded there).
 * --------------------------------------------------------------------------------------------- */

/* __hadd: the exact sum of two fp16 values fits a double, so one rounding to fp16 follows. */
static uint16_t hadd(uint16_t a, uint16_t b) {
    _Float16 r = (_Float16)((double)h2f(a) + (double)h2f(b));
    uint16_t bits;
    memcpy(&bits, &r, 2);
    return bits;
}

/* vadd (kernels.cu:156-159) then rmsnorm_kernel<<<1,256>>> (kernels.cu:10-33): thread t sums
 * elements t, t+256, ...; a xor-shuffle tree adds the 32 lanes of a warp (every lane ends with
 * the same value because fp32 addition commutes); thread 0 adds the warp totals in order.
 * delta and x_out may be NULL. */
void kivi_oracle_residual_rmsnorm(const uint16_t* x, const uint16_t* delta, const uint16_t* weight,
                                  uint16_t* x_out, uint16_t* normed, int batch, int hidden, float eps) {
    enum { THREADS = 256 };
    uint16_t* row = (uint16_t*)malloc((size_t)hidden * sizeof(uint16_t));
    for (int b = 0; b < batch; ++b) {
        for (int i = 0; i < hidden; ++i) {
            uint16_t v = x[(size_t)b * hidden + i];
            if (delta) v = hadd(v, delta[(size_t)b * hidden + i]);
            row[i] = v;
            if (x_out) x_out[(size_t)b * hidden + i] = v;
        }
        float lane[THREADS];
        for (int t = 0; t < THREADS; ++t) {
            float local = 0.0f;
            for (int i = t; i < hidden; i += THREADS) {
                float v = h2f(row[i]);
                local += v * v;
            }
            lane[t] = local;
        }
        float total = 0.0f;
        for (int w = 0; w < THREADS / 32; ++w) {
            float* l = lane + 32 * w;
            for (int off = 16; off > 0; off >>= 1) {
                float next[32];
                for (int k = 0; k < 32; ++k) next[k] = l[k] + l[k ^ off];
                memcpy(l, next, sizeof(next));
            }
            total += l[0];
        }
        float scale = 1.0f / sqrtf(total / hidden + eps);
        for (int i = 0; i < hidden; ++i)
            normed[(size_t)b * hidden + i] = f2h(h2f(row[i]) * scale * h2f(weight[i]));
    }
    free(row);
}

/* bias_add_kernel (kernels.cu:163-166) then rope_qk_kernel (kernels.cu:40-54) at positions[b];
 * q, k and v are written split: q [batch, NH*HD], k and v [batch, NKV*HD]. bias may be NULL. */
void kivi_oracle_bias_rope(const uint16_t* qkv, const uint16_t* bias, const int* positions, uint16_t* q,
                           uint16_t* k, uint16_t* v, int batch, int nh, int nkv, int hd, float rope_base) {
    const int half = hd / 2, qkv_out = (nh + 2 * nkv) * hd;
    for (int b = 0; b < batch; ++b) {
        const uint16_t* in = qkv + (size_t)b * qkv_out;
        const int pos = positions[b];
        for (int h = 0; h < nh + nkv; ++h) {
            uint16_t* out = h < nh ? q + ((size_t)b * nh + h) * hd : k + ((size_t)b * nkv + (h - nh)) * hd;
            for (int i = 0; i < half; ++i) {
                float freq = 1.0f / powf(rope_base, (2.0f * i) / hd);
                float ang = pos * freq;
                float c = cosf(ang), s = sinf(ang);
                uint16_t h0 = in[h * hd + i], h1 = in[h * hd + i + half];
                if (bias) { h0 = hadd(h0, bias[h * hd + i]); h1 = hadd(h1, bias[h * hd + i + half]); }
                float x0 = h2f(h0), x1 = h2f(h1);
                out[i] = f2h(x0 * c - x1 * s);
                out[i + half] = f2h(x1 * c + x0 * s);
            }
        }
        for (int e = 0; e < nkv * hd; ++e) {
            uint16_t val = in[(nh + nkv) * hd + e];
            if (bias) val = hadd(val, bias[(nh + nkv) * hd + e]);
            v[(size_t)b * nkv * hd + e] = val;
        }
    }
}

/* silu_mul_kernel (kernels.cu:146-153) on rows [gate | up]. */
void kivi_oracle_silu_mul(const uint16_t* gate_up, uint16_t* out, int batch, int ffn) {
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < ffn; ++i) {
            float g = h2f(gate_up[(size_t)b * 2 * ffn + i]);
            float s = g / (1.0f + expf(-g));
            out[(size_t)b * ffn + i] = f2h(s * h2f(gate_up[(size_t)b * 2 * ffn + ffn + i]));
        }
}

/* argmax_kernel (kernels.cu:203-227): start from (-1e30, 0), replace on a strictly larger value.
 * The reference's choice among equal maxima depends on its thread layout; here the lowest index
 * wins. */
void kivi_oracle_argmax(const uint16_t* logits, int* out, int batch, int n) {
    for (int b = 0; b < batch; ++b) {
        float best = -1e30f;
        int best_i = 0;
        for (int i = 0; i < n; ++i) {
            float v = h2f(logits[(size_t)b * n + i]);
            if (v > best) { best = v; best_i = i; }
        }
        out[b] = best_i;
    }
}

/* Exposed for the tests of the conversion helpers. */
float kivi_oracle_h2f(uint16_t h) { return h2f(h); }
uint16_t kivi_oracle_f2h(float f) { return f2h(f); }
