// Paged int4-KIVI decode attention for B200: asynchronously staged pages, in-register int4 unpack,
// tensor-core QK^T and PV over the GQA query group, warp-shuffle softmax, split over the context.
//
// What it computes is the reference kernel's recurrence (crates/jac-codegen-cuda/src/variants.rs:
// 2359-2431, prologue/epilogue :2463-2502): softmax(q . dequant(K) / sqrt(D)) . dequant(V) over the
// quantised pages named by the block table, then over the fp16 residual rows. The reference runs
// one warp per query head and re-reads every K/V byte once per query head of the group; here one
// CTA serves all query heads of a kv head, so each byte is read once.
//
// Work split: one CTA per job. A job is a (sequence, kv head) unit or, where the host's launch plan cuts units,
// one of the k parts of a unit (JobPlan in kivi_common.cuh; the plan and the measurements behind it are in
// api.cu). A part owns a run of the unit's key groups and/or of the 16-row tiles of its fp16 residual, chosen by
// weight so that parts move equal bytes (decode_merge.cuh). A CTA's key groups go round-robin to its warps, its
// residual tiles to the least loaded warps; each warp keeps its own online-softmax state and the states are
// merged in shared memory at the end. A whole unit then writes its output; a part leaves a partial
// (maximum, sum, accumulator) in the workspace and a second, small kernel (decode_merge.cu) combines the
// parts of every cut unit. No CTA ever waits for another.
//
// Data movement: every warp owns a small ring of shared-memory slots of 64 tokens each (codes of
// K and V, the value scale/zero of those tokens, and with the first slot of a group its key
// scale/zero). Everything arrives by 16-byte cp.async, one warp instruction per 512 contiguous bytes of a
// page (1-D bulk copies were measured slower here: a page is only 1 KB per kv head, and every bulk copy
// costs about ten issue slots of address and uniform-register work), completing on the slot's mbarrier.
// Value codes are stored with their 16-byte columns swizzled so that ldmatrix reads them without bank
// conflicts. A warp fills its own slots and is the only one to wait on them: after draining a slot it
// issues the copies of the slot-count-th next one into it, so there is no "empty" barrier and no
// cross-warp synchronisation until the final merge, every warp keeps several slots in flight, and no
// registers are spent on staging. Every wait is bounded; a CTA whose wait ran out drains its copies, counts
// itself (kivi_b200_decode_wait_failures) and leaves.
//
// Arithmetic on codes: a 32-bit word holds 8 channels of one token. Masking a word with
// 0x000f000f / 0x00f000f0 leaves two nibbles in fp16 *subnormal* position: the pair (n_i, n_i+4)
// scaled by 2^-24, or (n_i+1, n_i+5) scaled by 2^-20 -- exact fp16 values the tensor core
// multiplies as they are. So unpacking costs 5 integer ops per 8 codes and no conversion:
//   QK^T:  sum_c q_c (s_c n_c + z_c) = sum_c (q_c s_c) n_c + sum_c q_c z_c. Per key group the
//          query fragment is pre-multiplied by the channel scales (odd channels by a further 2^-4
//          to even out the two nibble positions) and the zero-point term is one extra MMA set.
//          Channels are contracted, so the odd pairing (i, i+4) only permutes the contraction.
//   PV:    sum_s p_s (vs_s n_sd + vz_s) = sum_s (p_s vs_s) n_sd + sum_s p_s vz_s. Tokens are
//          contracted, so the A fragment wants the same 16-bit word of two consecutive tokens side by side:
//          ldmatrix.trans over the token rows delivers exactly that; the 2^-24 / 2^-20 factors land on
//          output channels and are undone in the epilogue.
// MMA shape m16n8k16 (fp16 in, fp32 accumulate): M = 16 tokens (QK^T) or 16 channels (PV),
// N = 8 query heads of the group (up to 8 used), so the tensor work wasted on padding is at most
// 2x for a group of 4. The score tile comes out token-major and is turned head-major for PV by
// movmatrix. tcgen05 does not fit: its M >= 64 would need the dequantised operand in shared memory
// or TMEM, i.e. a 4x expanded fp16 copy of every code written by CUDA cores.
//
// The running maximum is only raised (and the accumulators rescaled) when a tile exceeds it by
// more than 2^8: probabilities then stay below 256, far inside fp16/fp32 range, and the 36
// multiplies of a rescale are paid a handful of times per sequence instead of on every new maximum.
#include "kivi_common.cuh"
#include "decode_merge.cuh"

namespace kivi {
namespace {

constexpr int kResTile = kResTileRows;
#ifndef KIVI_SUB
#define KIVI_SUB 64
#endif
constexpr int kSubMax = KIVI_SUB;        // tokens per ring slot (never more than a key group)
constexpr int kBarBytes = 512;           // room for 64 mbarriers
// Bounded waits that ran out, over the life of the process (kivi_b200_decode_wait_failures reads it).
__device__ unsigned int g_decode_wait_failures;
// Page or slot ids outside the pools that this kernel met and replaced by id 0 (kivi_b200_decode_rejected_indices).
__device__ unsigned int g_decode_rejected;
constexpr int kMaxSlotsPerWarp = 8;    // small slots (32-token groups of 64 channels) need this many in flight to cover the latency
constexpr int kBarArrivals = 33;         // lane 0's expect_tx arrive + one cp.async arrive per lane
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleSlack = 8.0f;    // log2 units

template <int D, int G>
struct Cfg {
    static constexpr int VG = G < D ? G : D;   // value channel-group width
    static constexpr int HG = D / VG;          // value channel groups
    static constexpr int WPR = D / 8;          // 32-bit code words per token row
    static constexpr int KW = D / 32;          // key words per lane per token
    static constexpr int NMMA = D / 16;        // MMAs per 16-token tile, QK^T and PV each
    static constexpr int SUB = G < kSubMax ? G : kSubMax;   // tokens per ring slot
    static constexpr int SUBS = G / SUB;       // ring slots per key group
    static constexpr int VCOLS = D / 32;       // 16-byte chunks (32 channels) per token row of value codes
    static constexpr int VSW_SHIFT = VCOLS == 4 ? 1 : 2;   // token bits that swizzle the chunk column (see below)
    // slot layout (bytes)
    static constexpr int KC = 0;
    static constexpr int VC = KC + SUB * D / 2;
    static constexpr int VS = VC + SUB * D / 2;
    static constexpr int VZ = VS + SUB * HG * 2;
    // Key scale/zero of a group are read once, when its first slot is consumed. With one slot per
    // group they ride in the slot; otherwise they go to a small per-warp area (KP_BUFS buffers,
    // enough that the copy for a later group never lands before the current one was read).
    static constexpr int KP_BUFS = SUBS >= 4 ? 1 : (SUBS >= 2 ? 2 : 0);
    static constexpr int KP_BYTES = 4 * D;             // scale [D] then zero [D], fp16
    static constexpr int KS = KP_BUFS ? 0 : VZ + SUB * HG * 2;
    static constexpr int KZ = KS + D * 2;
    static constexpr int QUANT_BYTES = VZ + SUB * HG * 2 + (KP_BUFS ? 0 : KP_BYTES);
    static constexpr int CODE_BYTES = SUB * D;        // K + V codes of one slot
    static constexpr int RES_STRIDE = 2 * D + 16;      // padded fp16 row: ldmatrix rows hit distinct banks
    static constexpr int RES_BYTES = kResTile * RES_STRIDE;   // 16 key rows OR 16 value rows
    static constexpr int SLOT = ((QUANT_BYTES > RES_BYTES ? QUANT_BYTES : RES_BYTES) + 127) / 128 * 128;
    static constexpr int Q_BYTES = KW * 32 * 16;       // permuted query fragments of all lanes
    static constexpr int STATE_FLOATS = 8 * D + 16;    // per warp: O[8][D], m[8], l[8]
    static_assert(G % SUB == 0, "a key group must be whole slots");
    static_assert(VCOLS == 2 || VCOLS == 4, "value rows of 32 or 64 bytes");
    static_assert(NMMA == 2 * VCOLS, "two PV MMAs per 32-channel chunk column");
    static_assert(VG % 32 == 0, "a chunk column lies inside one value channel group");
};

#ifdef KIVI_DECODE_TRACE
// Debug builds only: per-CTA time stamps (globaltimer, ns) of the kernel's phases, read back by a
// tuning script through kivi_debug_decode_trace(). Not compiled into the product library.
__device__ unsigned long long g_decode_trace[4096 * 8];
__device__ __forceinline__ void trace_mark(int slot) {
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        if (cta < 4096) g_decode_trace[cta * 8 + slot] = t;
    }
}
#define KIVI_TRACE(slot) trace_mark(slot)
#else
#define KIVI_TRACE(slot)
#endif

// MMA row rho (0..7) of a 16-token tile holds token rho ^ ((rho >> 1) & 1); rows 8..15 add 8.
// With this pair swap the 16-byte key loads of a quarter warp touch rows of both parities.
__device__ __forceinline__ int row_token(int rho) { return rho ^ ((rho >> 1) & 1); }

// Split query fragment: q*scale is rounded to fp16 once (hi); lo = q*scale - hi is exact in an fp16
// FMA, and a second MMA set over the same code registers adds it back. It costs about a tenth of
// the kernel's throughput and cuts the output error by an order of magnitude. KIVI_QK_SPLIT:
// 0 = never, 1 = always, 2 (default) = for head_dim 64 only, whose short dot products with
// outlier channels otherwise come within a factor of two of the 1e-2 tolerance.
#ifndef KIVI_QK_SPLIT
#define KIVI_QK_SPLIT 2
#endif
__device__ __forceinline__ uint32_t hfma2_residual_u32(uint32_t a, uint32_t b, uint32_t hi) {
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b),
                        __hneg2(*reinterpret_cast<__half2*>(&hi)));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
// w >> 8 (a multiply-high by 2^24 on the FMA pipe was measured slower than the ALU shift).
__device__ __forceinline__ uint32_t shr8(uint32_t w) { return w >> 8; }
// (x0,x1),(x2,x3),(x4,x5),(x6,x7) -> (x0,x4),(x1,x5),(x2,x6),(x3,x7): the pairing the nibble masks give.
__device__ __forceinline__ void pair_by_four(const uint4& v, uint32_t (&o)[4]) {
    o[0] = __byte_perm(v.x, v.z, 0x5410);
    o[1] = __byte_perm(v.x, v.z, 0x7632);
    o[2] = __byte_perm(v.y, v.w, 0x5410);
    o[3] = __byte_perm(v.y, v.w, 0x7632);
}

template <int D, int G, int LOGB, int W, int CTAS>
__global__ void __launch_bounds__(W * 32, CTAS) decode_mma_kernel(const DecodeParams p, int per_warp) {
    using C = Cfg<D, G>;
    constexpr int kSub = C::SUB;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint4* qsm = reinterpret_cast<uint4*>(smem + kBarBytes);
    unsigned char* kparams = smem + kBarBytes + C::Q_BYTES;
    unsigned char* ring = kparams + W * C::KP_BUFS * C::KP_BYTES;

    const Geom& g = p.geom;
    pdl_trigger();   // a projection launched behind this kernel may start streaming its weights
    pdl_wait();      // queries, lengths and the cache may come from the kernel before this one
    KIVI_TRACE(0);
    // the warp index through a broadcast, so that everything derived from it is known to be warp-uniform
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int r = lane >> 2, t = lane & 3;
    constexpr int B = 1 << LOGB;                       // tokens per page
    constexpr int PB = B >= kSub ? 1 : kSub / B;       // pages a slot touches
    constexpr int WG = G / 16;                         // weight of a key group (a 16-row residual tile weighs kTileWeight)

    if (threadIdx.x == 0) {
        for (int s = 0; s < per_warp * W; ++s) mbar_init(&full[s], kBarArrivals);
        fence_barrier_init();
    }

    // ---- this CTA's job: a unit, or one of the k parts a unit is cut into ----------------------------
    // Units are (sequence, kv head) pairs in order. The first `units1` of them are cut into k1 parts each, the
    // rest into k2 parts (decode_merge.cuh: JobPlan); CTAs are dispatched in index order, so the large jobs start
    // first and the small ones fill the last, partial wave of the launch.
    const DecodeJob job = decode_job(p, blockIdx.x);
    const int i = job.unit / g.nkv, kv = job.unit - i * g.nkv;
    const UnitShape shape = unit_shape(p, i);
    const SegmentItems it = segment_items(shape, WG, (int)share_begin(shape.w, job.parts, job.part),
                                          (int)share_begin(shape.w, job.parts, job.part + 1));
    const bool whole_unit = job.parts == 1;   // then this CTA writes the output itself, else a partial for the merge
    if (!it.any && !whole_unit) {
        // a part of a unit too short to have an item for everyone: a neutral partial (weight 0 whatever the others hold), so that the merge need not know
        for (int idx = threadIdx.x; idx < g.qpk * D; idx += W * 32) p.ws_o[(size_t)job.slot * g.qpk * D + idx] = 0.0f;
        if (threadIdx.x < g.qpk) {
            p.ws_ml[((size_t)job.slot * g.qpk + threadIdx.x) * 2] = -1.0e30f;
            p.ws_ml[((size_t)job.slot * g.qpk + threadIdx.x) * 2 + 1] = 0.0f;
        }
        return;
    }

    // ---- staging -------------------------------------------------------------------------------
    // Every warp owns `per_warp` ring slots and the mbarriers that go with them, fills them itself
    // and is the only one to wait on them: its items are, in order, the slots of its key groups
    // (group warp, warp + W, ...) and then its residual tiles (key rows, then value rows). After
    // draining an item it issues the one `per_warp` items ahead into the slot it just freed.
    // All shared-memory traffic below goes through 32-bit shared-window addresses.
    const uint32_t ring32 = smem_u32(ring) + (uint32_t)(warp * per_warp) * C::SLOT;
    const uint32_t bars32 = smem_u32(full) + (uint32_t)(warp * per_warp) * 8u;
    const uint32_t q32 = smem_u32(qsm) + (uint32_t)lane * 16u;
    const uint32_t kp32 = smem_u32(kparams) + (uint32_t)warp * C::KP_BUFS * C::KP_BYTES;
    constexpr int logb = LOGB, bmask = B - 1;
    const size_t page_code_bytes = (size_t)B * (D / 2);
    const size_t page_stride = (size_t)g.nkv * page_code_bytes;

    // per-lane constants of the 16-byte copies. Page strides fit 32 bits, so page * stride + base
    // is one wide multiply-add.
    constexpr uint32_t SLOT_PAGE_BYTES = (B >= kSub ? kSub : B) * (D / 2);   // a page's share of a slot's codes
    static_assert(SLOT_PAGE_BYTES % 512 == 0, "cp.async staging moves 512 bytes per warp instruction");
    // Value codes land swizzled: the 16-byte chunk column c of token s sits at column c ^ ((s >> VSW_SHIFT) & (VCOLS - 1)),
    // so that the eight token rows of an ldmatrix block fall into eight different bank groups. A warp
    // instruction copies 512 contiguous bytes (8 or 16 token rows starting at a multiple of that), which makes
    // the swizzle a lane constant: lane = token * VCOLS + column and the token bits in question are lane bits 3+.
    const uint32_t v_stage_off = (uint32_t)((lane & ~(C::VCOLS - 1)) | ((lane & (C::VCOLS - 1)) ^ ((lane >> 3) & (C::VCOLS - 1)))) * 16u;
    const uint32_t page_stride32 = (uint32_t)page_stride;
    const int* bt = p.seq.block_tables + (size_t)i * p.seq.bt_stride;
    int slot = slot_of(p.seq, i);
    if (!index_in_pool(slot, p.cache.num_slots)) { slot = 0; if (threadIdx.x == 0) atomicAdd(&g_decode_rejected, 1u); }
    const uint8_t* kc_lane = p.cache.k_code + (size_t)kv * page_code_bytes + lane * 16;
    const uint8_t* vc_lane = p.cache.v_code + (size_t)kv * page_code_bytes + lane * 16;
    const __half* k_res = p.cache.k_scratch + ((size_t)slot * g.nkv + kv) * g.scratch_rows * D;
    const __half* v_res = p.cache.v_scratch + ((size_t)slot * g.nkv + kv) * g.scratch_rows * D;
    constexpr int CH = kSub * C::HG / 8;   // 16-byte chunks per value-parameter array per slot
    const bool vp_on = lane < 2 * CH;
    const int vp_c = lane < CH ? lane : lane - CH;
    const int vp_tok = (vp_c * 8) / C::HG;              // slot-relative token of this lane's chunk
    const int vp_page = vp_tok >> logb;                  // which of the slot's pages it lies in
    const __half* vp_lane = (lane < CH ? p.cache.v_scale : p.cache.v_zero) +
                            ((size_t)kv * B + (vp_tok & bmask)) * C::HG;
    const uint32_t vp_dst = (lane < CH ? C::VS : C::VZ) + vp_c * 16;
    const uint32_t vp_stride32 = (uint32_t)(g.nkv * B * C::HG);
    constexpr int CK = D / 8;              // chunks per key-parameter array
    const bool kp_on = lane < 2 * CK;
    const int kp_c = lane < CK ? lane : lane - CK;
    const __half* kp_lane = (lane < CK ? p.cache.k_scale : p.cache.k_zero) + (size_t)kv * D + kp_c * 8;
    const uint32_t kp_dst = (lane < CK ? C::KS : C::KZ) + kp_c * 16;
    const uint32_t kp_stride32 = (uint32_t)(g.nkv * D);
    static_assert(2 * CK <= 32 && 2 * CH <= 32, "parameter copies must fit one warp instruction");

    // this warp's items: the key groups it.g0 + warp, + W, ... and then every W-th residual tile
    const int ngroups = it.g1 - it.g0, ntiles = it.t1 - it.t0;
    const int my_groups = ngroups > warp ? (ngroups - warp + W - 1) / W : 0;
    const int my_quant = my_groups * C::SUBS;
    const int res_first = ((warp - ngroups) % W + W) % W;   // residual tiles go to the least loaded warps first
    const int my_res = ntiles > res_first ? (ntiles - res_first + W - 1) / W : 0;
    const int my_items = my_quant + 2 * my_res;
    const int res_valid = shape.res_valid;
    int i_item = 0, i_slot = 0, i_grp = it.g0 + warp, i_sub = 0, i_tile = it.t0 + res_first, i_isv = 0, i_kbuf = 0;
    auto issue_next = [&]() {
        if (i_item >= my_items) return;
        const uint32_t st = ring32 + (uint32_t)i_slot * C::SLOT;
        const uint32_t bar = bars32 + (uint32_t)i_slot * 8u;
        if (i_item < my_quant) {
            const int tokbase = i_grp * G + i_sub * kSub;
            const int lp = tokbase >> logb;
            // the slot's page ids: lanes 0..PB-1 fetch them, shuffles hand them round
            int my_page = lane < PB ? bt[lp + lane] : 0;
            if (!index_in_pool(my_page, p.cache.num_blocks)) { my_page = 0; atomicAdd(&g_decode_rejected, 1u); }
            uint32_t pg[PB];
#pragma unroll
            for (int j = 0; j < PB; ++j) pg[j] = (uint32_t)__shfl_sync(0xffffffffu, my_page, j);
            if (lane == 0) mbar_expect_tx32(bar, 0u);
            {
                // each page's share of the slot is contiguous in both memories: lane l moves the
                // 16-byte chunks l, l+32, ... of it, one cp.async warp instruction per 512 bytes
                const uint32_t dst = st + (uint32_t)lane * 16u;
                const uint32_t dstv = st + v_stage_off;
#pragma unroll
                for (int j = 0; j < PB; ++j) {
                    const uint8_t* ks = kc_lane + (size_t)pg[j] * page_stride32 + (B > kSub ? (size_t)(tokbase & bmask) * (D / 2) : 0);
                    const uint8_t* vs = vc_lane + (size_t)pg[j] * page_stride32 + (B > kSub ? (size_t)(tokbase & bmask) * (D / 2) : 0);
#pragma unroll
                    for (int h = 0; h < (int)SLOT_PAGE_BYTES / 512; ++h) {
                        cp_async16_32(dst + C::KC + j * SLOT_PAGE_BYTES + h * 512, ks + h * 512);
                        cp_async16_32(dstv + C::VC + j * SLOT_PAGE_BYTES + h * 512, vs + h * 512);
                    }
                }
            }
            if (vp_on) {   // value scale / zero of the slot's 32 tokens
                uint32_t pv = pg[0];
#pragma unroll
                for (int j = 1; j < PB; ++j) pv = vp_page == j ? pg[j] : pv;
                cp_async16_32(st + vp_dst, vp_lane + (size_t)pv * vp_stride32 +
                                               (B > kSub ? (size_t)(tokbase & bmask) * C::HG : 0));
            }
            if (i_sub == 0) {   // key scale / zero of the group, from its first page
                const uint32_t dst = C::KP_BUFS ? kp32 + (uint32_t)i_kbuf * C::KP_BYTES : st;
                if (kp_on) cp_async16_32(dst + kp_dst, kp_lane + (size_t)pg[0] * kp_stride32);
                if (C::KP_BUFS > 1) i_kbuf ^= 1;
            }
            if (++i_sub == C::SUBS) { i_sub = 0; i_grp += W; }
        } else {
            const int row0 = i_tile * kResTile;
            const int rows = min(kResTile, res_valid - row0);
            if (lane == 0) mbar_expect_tx32(bar, 0u);
            const __half* src = (i_isv ? v_res : k_res) + (size_t)row0 * D;
            constexpr int CPR = D / 8;
            for (int c = lane; c < rows * CPR; c += 32) {
                const int rr = c / CPR, cc = c - rr * CPR;
                cp_async16_32(st + rr * C::RES_STRIDE + cc * 16, src + (size_t)rr * D + cc * 8);
            }
            if (i_isv) { i_isv = 0; i_tile += W; } else i_isv = 1;
        }
        cp_async_arrive_noinc32(bar);
        ++i_item;
        if (++i_slot == per_warp) i_slot = 0;
    };
    int c_slot = 0;
    uint32_t c_phase = 0;
    auto advance_consumer = [&]() { if (++c_slot == per_warp) { c_slot = 0; c_phase ^= 1u; } };

    KIVI_TRACE(1);

    // ---- per-warp state --------------------------------------------------------------------------
    uint32_t qs[4 * C::KW];   // query fragment times the key scales of the current group (residual: natural pairs)
    constexpr bool kSplitQ = KIVI_QK_SPLIT == 1 || (KIVI_QK_SPLIT == 2 && D == 64);
    uint32_t ql[kSplitQ ? 4 * C::KW : 1];   // rounding residual of qs
    const float scale_log2 = rsqrtf((float)D) * kLog2e;
    const float sc_code = scale_log2 * 16777216.0f;   // undo the 2^-24 of the subnormal codes
    // Scores are s = raw * mult + add (log2 units); the state keeps m and b = add - m per head.
    float m0 = -1.0e30f, m1 = -1.0e30f, l0 = 0.0f, l1 = 0.0f;
    float add0 = 0.0f, add1 = 0.0f, b0 = 1.0e30f, b1 = 1.0e30f;
    float zacc[C::HG][2];
#pragma unroll
    for (int cg = 0; cg < C::HG; ++cg) zacc[cg][0] = zacc[cg][1] = 0.0f;
    float o[C::NMMA][4];
#pragma unroll
    for (int m = 0; m < C::NMMA; ++m) o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.0f;
    bool failed = false;

    // Online-softmax update shared by both phases: raw accumulators x[4] of tokens (rowA: x0,x1;
    // rowB: x2,x3) for heads (2t, 2t+1) -> probabilities in x[]; state rescaled when a score exceeds
    // the running maximum by more than the slack.
    auto softmax_step = [&](float (&x)[4], const float mult) {
        // exponents relative to the running maximum; the common case needs no reduction at all:
        // only when some score tops the maximum by more than the slack is the tile maximum formed
        // (three shuffle rounds) and the state rescaled.
        float e0 = fmaf(x[0], mult, b0), e1 = fmaf(x[1], mult, b1);
        float e2 = fmaf(x[2], mult, b0), e3 = fmaf(x[3], mult, b1);
        if (__any_sync(0xffffffffu, fmaxf(fmaxf(e0, e1), fmaxf(e2, e3)) > kRescaleSlack)) {
            float mx0 = fmaxf(x[0], x[2]), mx1 = fmaxf(x[1], x[3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            const float n0 = fmaxf(m0, fmaf(mx0, mult, add0)), n1 = fmaxf(m1, fmaf(mx1, mult, add1));
            const float c0 = fast_exp2(m0 - n0), c1 = fast_exp2(m1 - n1);
            l0 *= c0; l1 *= c1;
#pragma unroll
            for (int cg = 0; cg < C::HG; ++cg) { zacc[cg][0] *= c0; zacc[cg][1] *= c1; }
#pragma unroll
            for (int m = 0; m < C::NMMA; ++m) { o[m][0] *= c0; o[m][1] *= c1; o[m][2] *= c0; o[m][3] *= c1; }
            m0 = n0; m1 = n1;
            b0 = add0 - m0; b1 = add1 - m1;
            e0 = fmaf(x[0], mult, b0); e1 = fmaf(x[1], mult, b1);
            e2 = fmaf(x[2], mult, b0); e3 = fmaf(x[3], mult, b1);
        }
        x[0] = fast_exp2(e0); x[1] = fast_exp2(e1);
        x[2] = fast_exp2(e2); x[3] = fast_exp2(e3);
        l0 += x[0] + x[2];
        l1 += x[1] + x[3];
    };

    // lane-constant byte offsets inside a slot
    const uint32_t k_off = C::KC + row_token(r) * (D / 2) + (D / 8) * t;
    // ldmatrix.x4.trans over the swizzled value codes: lanes 0-7 / 8-15 / 16-23 / 24-31 address the token rows of
    // the blocks (chunk column c, tokens 0-7), (c, tokens 8-15), (c+1, tokens 0-7), (c+1, tokens 8-15); block row
    // rho is token row_token(rho), the order the probability tile comes out of the QK^T MMA in. Transposed, a
    // lane holds the 16-bit words (4 channels 4r..4r+3 of the column) of tokens (2t, 2t+1) of each block --
    // the A fragment of O^T += V^T P with no byte permute.
    uint32_t v_ldm[C::VCOLS / 2];
    {
        const int blk = lane >> 3;
        const int tok = row_token(lane & 7) + 8 * (blk & 1);
#pragma unroll
        for (int h2 = 0; h2 < C::VCOLS / 2; ++h2) {
            const int col = (blk >> 1) + 2 * h2;
            v_ldm[h2] = C::VC + tok * (D / 2) + ((col ^ ((tok >> C::VSW_SHIFT) & (C::VCOLS - 1))) * 16);
        }
    }
    const uint32_t vs_off = C::VS + row_token(r) * C::HG * 2;
    const uint32_t ks_off = C::KS + (D / 2) * t;
    constexpr uint32_t TILE_STEP = 16u * (D / 2);            // bytes between 16-token tiles of codes

    // ---- query fragments of the unit, shared by all warps ----
    // Lane (r, t): head r of the group (zero when r >= heads per group), channels [D/4*t, D/4*(t+1)),
    // as the pairs the nibble masks produce; odd channels carry a 2^-4 factor.
    const bool head_on = r < g.qpk;
    const __half* qrow = p.q + ((size_t)i * g.nh + (size_t)kv * g.qpk + (head_on ? r : 0)) * D;
    if (warp == 0) {
        const uint32_t sixteenth = 0x2C002C00u;  // half2(1/16, 1/16)
#pragma unroll
        for (int j = 0; j < C::KW; ++j) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (head_on) v = *reinterpret_cast<const uint4*>(qrow + (D / 4) * t + 8 * j);
            uint32_t o4[4];
            pair_by_four(v, o4);
            qsm[j * 32 + lane] = make_uint4(o4[0], hmul2_u32(o4[1], sixteenth), o4[2], hmul2_u32(o4[3], sixteenth));
        }
    }
    for (int s_ = 0; s_ < per_warp; ++s_) issue_next();
    __syncthreads();   // the query fragments are in place

    // ================= key groups of int4 pages =================
    for (int gi = 0; gi < my_groups && !failed; ++gi) {
#pragma unroll 1
        for (int sub = 0; sub < C::SUBS; ++sub) {
            const uint32_t st = ring32 + (uint32_t)c_slot * C::SLOT;
            if (!mbar_wait32(bars32 + (uint32_t)c_slot * 8u, c_phase)) { failed = true; break; }

            if (sub == 0) {
                float ca[4] = {0.0f, 0.0f, 0.0f, 0.0f}, cb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t sixteenth = 0x2C002C00u;
                const uint32_t kbase = C::KP_BUFS ? kp32 + (uint32_t)(C::KP_BUFS > 1 ? (gi & 1) : 0) * C::KP_BYTES : st;
#pragma unroll
                for (int j = 0; j < C::KW; ++j) {
                    const uint4 qv = lds128(q32 + j * 512u);
                    const uint4 sv = lds128(kbase + ks_off + 16u * j);
                    const uint4 zv = lds128(kbase + ks_off + (C::KZ - C::KS) + 16u * j);
                    uint32_t sp[4], zp[4];
                    pair_by_four(sv, sp);
                    pair_by_four(zv, zp);
                    qs[4 * j + 0] = hmul2_u32(qv.x, sp[0]);
                    qs[4 * j + 1] = hmul2_u32(qv.y, sp[1]);
                    qs[4 * j + 2] = hmul2_u32(qv.z, sp[2]);
                    qs[4 * j + 3] = hmul2_u32(qv.w, sp[3]);
                    if constexpr (kSplitQ) {
                        ql[4 * j + 0] = hfma2_residual_u32(qv.x, sp[0], qs[4 * j + 0]);
                        ql[4 * j + 1] = hfma2_residual_u32(qv.y, sp[1], qs[4 * j + 1]);
                        ql[4 * j + 2] = hfma2_residual_u32(qv.z, sp[2], qs[4 * j + 2]);
                        ql[4 * j + 3] = hfma2_residual_u32(qv.w, sp[3], qs[4 * j + 3]);
                    }
                    // zero-point term: all rows equal; even channels scaled 2^-4 to match the odd 2^-4 of q
                    const uint32_t z0 = hmul2_u32(zp[0], sixteenth), z2 = hmul2_u32(zp[2], sixteenth);
                    mma16816(ca, z0, z0, zp[1], zp[1], qv.x, qv.y);
                    mma16816(cb, z2, z2, zp[3], zp[3], qv.z, qv.w);
                }
                add0 = (ca[0] + cb[0]) * 16.0f * scale_log2;
                add1 = (ca[1] + cb[1]) * 16.0f * scale_log2;
                b0 = add0 - m0;
                b1 = add1 - m1;
            }

#pragma unroll
            for (int tile = 0; tile < kSub / 16; ++tile) {
                // ---- QK^T: S^T[token, head]; two accumulators halve the dependent MMA chain ----
                float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                {
                    uint32_t ka[C::KW], kb[C::KW];
                    const uint32_t kaddr = st + k_off + tile * TILE_STEP;
                    if constexpr (C::KW == 4) {
                        const uint4 a = lds128(kaddr), b = lds128(kaddr + 8 * (D / 2));
                        ka[0] = a.x; ka[1] = a.y; ka[2] = a.z; ka[3] = a.w;
                        kb[0] = b.x; kb[1] = b.y; kb[2] = b.z; kb[3] = b.w;
                    } else {
                        const uint2 a = lds64(kaddr), b = lds64(kaddr + 8 * (D / 2));
                        ka[0] = a.x; ka[1] = a.y;
                        kb[0] = b.x; kb[1] = b.y;
                    }
#pragma unroll
                    for (int j = 0; j < C::KW; ++j) {
                        const uint32_t wa = ka[j], wb = kb[j], wa8 = shr8(wa), wb8 = shr8(wb);
                        const uint32_t a0 = wa & 0x000f000fu, a1 = wb & 0x000f000fu, a2 = wa & 0x00f000f0u, a3 = wb & 0x00f000f0u;
                        const uint32_t c0 = wa8 & 0x000f000fu, c1 = wb8 & 0x000f000fu, c2 = wa8 & 0x00f000f0u, c3 = wb8 & 0x00f000f0u;
                        mma16816(sc, a0, a1, a2, a3, qs[4 * j + 0], qs[4 * j + 1]);
                        mma16816(sd, c0, c1, c2, c3, qs[4 * j + 2], qs[4 * j + 3]);
                        if constexpr (kSplitQ) {
                            mma16816(sd, a0, a1, a2, a3, ql[4 * j + 0], ql[4 * j + 1]);
                            mma16816(sc, c0, c1, c2, c3, ql[4 * j + 2], ql[4 * j + 3]);
                        }
                    }
                }
                sc[0] += sd[0]; sc[1] += sd[1]; sc[2] += sd[2]; sc[3] += sd[3];
                softmax_step(sc, sc_code);

                // ---- P' = p * value scale (per channel group), token-major -> head-major ----
                uint32_t pb01[C::HG], pb23[C::HG];
                {
                    const uint32_t pa = st + vs_off + tile * (16u * C::HG * 2u);
#pragma unroll
                    for (int cg = 0; cg < C::HG; ++cg) {
                        const float sa = lds_half(pa + 2u * cg), sb = lds_half(pa + 8u * C::HG * 2u + 2u * cg);
                        const float za = lds_half(pa + (C::VZ - C::VS) + 2u * cg);
                        const float zb = lds_half(pa + (C::VZ - C::VS) + 8u * C::HG * 2u + 2u * cg);
                        pb01[cg] = movmatrix_trans(pack_half2(sc[0] * sa, sc[1] * sa));
                        pb23[cg] = movmatrix_trans(pack_half2(sc[2] * sb, sc[3] * sb));
                        zacc[cg][0] = fmaf(sc[0], za, fmaf(sc[2], zb, zacc[cg][0]));
                        zacc[cg][1] = fmaf(sc[1], za, fmaf(sc[3], zb, zacc[cg][1]));
                    }
                }

                // ---- PV: O^T[channel, head] += V^T[channel, token] P'[token, head] ----
                // MMA 2c (2c+1) takes nibbles 0,1 (2,3) of chunk column c: row r is channel 32c + 4r (+2), row r+8 the next one
#pragma unroll
                for (int h2 = 0; h2 < C::VCOLS / 2; ++h2) {
                    uint32_t x[4];
                    ldmatrix_x4_trans_32(x, st + v_ldm[h2] + tile * TILE_STEP);
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int col = 2 * h2 + cc;
                        const int cg = (32 * col) / C::VG;
                        const uint32_t xl = x[2 * cc], xh = x[2 * cc + 1];
                        const uint32_t xl8 = shr8(xl), xh8 = shr8(xh);
                        mma16816(o[2 * col + 0], xl & 0x000f000fu, xl & 0x00f000f0u, xh & 0x000f000fu,
                                 xh & 0x00f000f0u, pb01[cg], pb23[cg]);
                        mma16816(o[2 * col + 1], xl8 & 0x000f000fu, xl8 & 0x00f000f0u, xh8 & 0x000f000fu,
                                 xh8 & 0x00f000f0u, pb01[cg], pb23[cg]);
                    }
                }
            }
            __syncwarp();
            advance_consumer();
            issue_next();
        }
    }

    KIVI_TRACE(2);
    // accumulators leave the code scale: channels masked at bits 0-3 carry 2^-24, at bits 4-7 2^-20
#pragma unroll
    for (int m = 0; m < C::NMMA; ++m) {
        o[m][0] *= 16777216.0f; o[m][1] *= 16777216.0f;
        o[m][2] *= 1048576.0f;  o[m][3] *= 1048576.0f;
    }

    // ================= 16-row tiles of the fp16 residual =================
    if (my_res > 0 && !failed) {
        // natural channel pairs of q: (16m+2t, +1) and (16m+2t+8, +9)
#pragma unroll
        for (int m = 0; m < C::NMMA; ++m) {
            qs[2 * m] = head_on ? *reinterpret_cast<const uint32_t*>(qrow + 16 * m + 2 * t) : 0u;
            qs[2 * m + 1] = head_on ? *reinterpret_cast<const uint32_t*>(qrow + 16 * m + 2 * t + 8) : 0u;
        }
        add0 = add1 = 0.0f;
        b0 = -m0; b1 = -m1;
        // ldmatrix: lanes 0-7 / 8-15 / 16-23 / 24-31 give the row addresses of the four
        // 8x8 blocks (rows 0-7 | 8-15) x (channels +0 | +8).
        const uint32_t ldm_off = (row_token(lane & 7) + 8 * ((lane >> 3) & 1)) * C::RES_STRIDE + 16 * (lane >> 4);
        const int rA = row_token(r);
        const int tA = 2 * t + (t & 1), tB = 2 * t + ((t & 1) ^ 1);
        for (int tile = it.t0 + res_first; tile < it.t1; tile += W) {
            const uint32_t stk = ring32 + (uint32_t)c_slot * C::SLOT;
            if (!mbar_wait32(bars32 + (uint32_t)c_slot * 8u, c_phase)) { failed = true; break; }
            advance_consumer();
            const uint32_t stv = ring32 + (uint32_t)c_slot * C::SLOT;
            if (!mbar_wait32(bars32 + (uint32_t)c_slot * 8u, c_phase)) { failed = true; break; }
            advance_consumer();
            const int rows = min(kResTile, res_valid - tile * kResTile);
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int m = 0; m < C::NMMA; m += 2) {
                uint32_t a[4], b[4];
                ldmatrix_x4_32(a, stk + ldm_off + 32 * m);
                ldmatrix_x4_32(b, stk + ldm_off + 32 * (m + 1));
                mma16816(sc, a[0], a[1], a[2], a[3], qs[2 * m], qs[2 * m + 1]);
                mma16816(sd, b[0], b[1], b[2], b[3], qs[2 * m + 2], qs[2 * m + 3]);
            }
            // rows past the end of the residual hold stale bytes: give them a score no maximum will see
            const bool onA = rA < rows, onB = rA + 8 < rows;
            sc[0] = onA ? sc[0] + sd[0] : -1.0e30f; sc[1] = onA ? sc[1] + sd[1] : -1.0e30f;
            sc[2] = onB ? sc[2] + sd[2] : -1.0e30f; sc[3] = onB ? sc[3] + sd[3] : -1.0e30f;
            softmax_step(sc, scale_log2);
            if (!onA) { sc[0] = 0.0f; sc[1] = 0.0f; }
            if (!onB) { sc[2] = 0.0f; sc[3] = 0.0f; }
            const uint32_t pb01 = movmatrix_trans(pack_half2(sc[0], sc[1]));
            const uint32_t pb23 = movmatrix_trans(pack_half2(sc[2], sc[3]));
            const bool vA = tA < rows, vB = tB < rows, vA8 = tA + 8 < rows, vB8 = tB + 8 < rows;
#pragma unroll
            for (int col = 0; col < C::VCOLS; ++col) {
                // same channel-to-row assignment as the int4 path: rows (r, r+8) of MMA 2col + q are
                // channels (c0 + 2q, c0 + 2q + 1)
                const int c0 = 32 * col + 4 * r;
                auto load = [&](int tok, bool on) {
                    const uint2 v = lds64(stv + tok * C::RES_STRIDE + c0 * 2);
                    return on ? v : make_uint2(0u, 0u);
                };
                const uint2 xa = load(tA, vA), xb = load(tB, vB), xa8 = load(tA + 8, vA8), xb8 = load(tB + 8, vB8);
                mma16816(o[2 * col + 0], __byte_perm(xa.x, xb.x, 0x5410), __byte_perm(xa.x, xb.x, 0x7632),
                         __byte_perm(xa8.x, xb8.x, 0x5410), __byte_perm(xa8.x, xb8.x, 0x7632), pb01, pb23);
                mma16816(o[2 * col + 1], __byte_perm(xa.y, xb.y, 0x5410), __byte_perm(xa.y, xb.y, 0x7632),
                         __byte_perm(xa8.y, xb8.y, 0x5410), __byte_perm(xa8.y, xb8.y, 0x7632), pb01, pb23);
            }
            __syncwarp();
            issue_next();
            issue_next();
        }
    }

    KIVI_TRACE(3);
    // ---- finish the lane-partial sums ----
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
#pragma unroll
        for (int cg = 0; cg < C::HG; ++cg) {
            zacc[cg][0] += __shfl_xor_sync(0xffffffffu, zacc[cg][0], off);
            zacc[cg][1] += __shfl_xor_sync(0xffffffffu, zacc[cg][1], off);
        }
    }

    // every slot has been consumed: the ring can hold the warp states. A warp whose bounded wait ran out has copies
    // in flight and a wrong state: the CTA drains them, reports and leaves (the launch's output is then undefined).
    if (__syncthreads_or(failed ? 1 : 0)) {
        cp_async_wait_all();
        if (threadIdx.x == 0) {
            atomicAdd(&g_decode_wait_failures, 1u);
            if (p.status) atomicExch(p.status, 1);
        }
        return;
    }
    float* state = reinterpret_cast<float*>(ring) + (size_t)warp * C::STATE_FLOATS;
#pragma unroll
    for (int col = 0; col < C::VCOLS; ++col) {
        const int cg = (32 * col) / C::VG;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int ch = 32 * col + 4 * r + 2 * q;
            const float* acc = o[2 * col + q];
            state[(2 * t) * D + ch] = acc[0] + zacc[cg][0];
            state[(2 * t + 1) * D + ch] = acc[1] + zacc[cg][1];
            state[(2 * t) * D + ch + 1] = acc[2] + zacc[cg][0];
            state[(2 * t + 1) * D + ch + 1] = acc[3] + zacc[cg][1];
        }
    }
    if (r == 0) {
        state[8 * D + 2 * t] = m0; state[8 * D + 2 * t + 1] = m1;
        state[8 * D + 8 + 2 * t] = l0; state[8 * D + 8 + 2 * t + 1] = l1;
    }
    __syncthreads();

    KIVI_TRACE(4);
    const float* all = reinterpret_cast<const float*>(ring);
    for (int idx = threadIdx.x; idx < g.qpk * D; idx += W * 32) {
        const int hq = idx / D, d = idx - hq * D;
        float mx = -1.0e30f;
#pragma unroll
        for (int w = 0; w < W; ++w) mx = fmaxf(mx, all[w * C::STATE_FLOATS + 8 * D + hq]);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const float* sw = all + w * C::STATE_FLOATS;
            const float wt = fast_exp2(sw[8 * D + hq] - mx);
            l += wt * sw[8 * D + 8 + hq];
            acc += wt * sw[hq * D + d];
        }
        if (whole_unit) {
            store_out(p, ((size_t)i * g.nh + (size_t)kv * g.qpk + hq) * D + d, acc / fmaxf(l, 1.0e-30f));
        } else {
            const size_t part = (size_t)job.slot * g.qpk + hq;
            p.ws_o[part * D + d] = acc;
            if (d == 0) { p.ws_ml[part * 2] = mx; p.ws_ml[part * 2 + 1] = l; }
        }
    }
    KIVI_TRACE(5);
    KIVI_TRACE(6);
}

template <int D, int G, int LOGB, int W, int CTAS>
cudaError_t launch(const DecodeParams& p, cudaStream_t stream) {
    using C = Cfg<D, G>;
    // 227 KB of shared memory per SM may be opted into; every resident CTA also costs 1 KB.
    constexpr int kBudget = 227 * 1024 / CTAS - 1024 - 256;
    constexpr int kFixed = kBarBytes + C::Q_BYTES + W * C::KP_BUFS * C::KP_BYTES;
    int per_warp = (kBudget - kFixed) / (C::SLOT * W);
    if (per_warp > kMaxSlotsPerWarp) per_warp = kMaxSlotsPerWarp;
    if (per_warp * W > 64) per_warp = 64 / W;
    const int state_bytes = W * C::STATE_FLOATS * (int)sizeof(float);
    while (per_warp * W * C::SLOT < state_bytes) ++per_warp;
    if (per_warp < 2) return cudaErrorInvalidConfiguration;
    const int smem = kFixed + per_warp * W * C::SLOT;
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<D, G, LOGB, W, CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    return launch_pdl(decode_mma_kernel<D, G, LOGB, W, CTAS>, dim3(p.plan.jobs()), dim3(W * 32), smem, stream, p, per_warp);
}

// Warps per CTA and CTAs per SM. Twelve warps per SM leave each thread about 170 registers, which
// the unrolled two-tile body needs (at 128 it spills and throttles); several small CTAs instead of
// one large one overlap a CTA's ramp-up and final merge with the steady state of the others and
// give every warp a long run of groups to amortise its fixed costs. Measured on the Mistral-7B
// shape with 32-token slots (GB/s): 4x3 5043, 6x2 5008, 5x3 4768, 3x4 4691, 8x2 4628, 12x1 4537, 16x1 4113;
// with 64-token slots (half the per-slot wait/refill work, two slots per warp): 4x3 5461, 6x2 5359.
#ifndef KIVI_DECODE_WARPS
#define KIVI_DECODE_WARPS 4
#endif
#ifndef KIVI_DECODE_CTAS
#define KIVI_DECODE_CTAS 3
#endif
constexpr int kWarps = KIVI_DECODE_WARPS;
constexpr int kCtas = KIVI_DECODE_CTAS;

}  // namespace

int decode_mma_ctas_per_sm() { return kCtas; }

bool decode_mma_supports(const Geom& g, int retained_pages) {
    if (g.d != 64 && g.d != 128) return false;
    if (g.g != 32 && g.g != 64 && g.g != 128) return false;
    if (g.qpk > 8) return false;
    if (g.log2b != 4 && g.log2b != 5) return false;                    // pages of 16 or 32 tokens
    if ((g.b * g.hg * 2) % 16 || (g.b * g.d / 2) % 16) return false;   // async copies move 16-byte multiples
    if (retained_pages >= 0 && g.g != g.b) return false;  // a compact table breaks groups that span pages
    return true;
}

template <int D, int G>
cudaError_t launch_for_block(const DecodeParams& p, cudaStream_t stream) {
    if (p.geom.log2b == 4) return launch<D, G, 4, kWarps, kCtas>(p, stream);
    if (p.geom.log2b == 5) return launch<D, G, 5, kWarps, kCtas>(p, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_decode_mma(const DecodeParams& p, cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    const int d = p.geom.d, g = p.geom.g;
    if (d == 128 && g == 128) return launch_for_block<128, 128>(p, stream);
    if (d == 128 && g == 64) return launch_for_block<128, 64>(p, stream);
    if (d == 128 && g == 32) return launch_for_block<128, 32>(p, stream);
    if (d == 64 && g == 128) return launch_for_block<64, 128>(p, stream);
    if (d == 64 && g == 64) return launch_for_block<64, 64>(p, stream);
    if (d == 64 && g == 32) return launch_for_block<64, 32>(p, stream);
    return cudaErrorInvalidValue;
}

}  // namespace kivi

extern "C" int kivi_b200_decode_wait_failures(uint32_t* count) {
    if (!count) return KIVI_ERR_NULL_POINTER;
    return cudaMemcpyFromSymbol(count, kivi::g_decode_wait_failures, sizeof(unsigned int)) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

extern "C" int kivi_b200_decode_rejected_indices(uint32_t* count) {
    if (!count) return KIVI_ERR_NULL_POINTER;
    unsigned int mine = 0, generic = 0;
    if (cudaMemcpyFromSymbol(&mine, kivi::g_decode_rejected, sizeof(unsigned int)) != cudaSuccess) return KIVI_ERR_CUDA;
    if (kivi::decode_generic_rejected(&generic) != cudaSuccess) return KIVI_ERR_CUDA;
    *count = mine + generic;
    return KIVI_OK;
}

#ifdef KIVI_DECODE_TRACE
extern "C" int kivi_debug_decode_trace(unsigned long long* host_out, int ctas) {
    return (int)cudaMemcpyFromSymbol(host_out, kivi::g_decode_trace, sizeof(unsigned long long) * 8 * ctas);
}
#endif
