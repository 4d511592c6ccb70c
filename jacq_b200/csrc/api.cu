// C launch contract of libjacq_kivi_b200.so: argument validation, launch planning and the
// reference-lane (ABI v1) symbols. Declarations and the reference lines each entry point
// replaces are in include/jacq_kivi_b200.h.
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "decode_merge.cuh"
#include "kivi_common.cuh"

namespace kivi {

// Multiprocessors of the current device (148 on a B200), asked once per device.
int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return cached[dev];
}

namespace {

constexpr int kLongChunkTokens = 6144;
constexpr int kMinChunkTokens = 256;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_geometry(const kivi_geometry* s) {
    if (!s) return KIVI_ERR_NULL_POINTER;
    if (s->num_q_heads <= 0 || s->num_kv_heads <= 0 || s->head_dim <= 0 || s->block_size <= 0 ||
        s->group_size <= 0 || s->residual < 0)
        return KIVI_ERR_GEOMETRY;
    if (s->num_q_heads % s->num_kv_heads) return KIVI_ERR_GEOMETRY;
    if (s->head_dim % 8 || s->head_dim > 256) return KIVI_ERR_GEOMETRY;  // 16-byte rows, <= 4 bytes per lane
    if (s->group_size % s->block_size) return KIVI_ERR_GEOMETRY;
    const int vg = s->group_size < s->head_dim ? s->group_size : s->head_dim;
    if (s->head_dim % vg || vg % 8) return KIVI_ERR_GEOMETRY;
    return KIVI_OK;
}

int check_cache(const kivi_cache* c) {
    if (!c) return KIVI_ERR_NULL_POINTER;
    const void* ptrs[] = {c->k_code_pages, c->k_scale_pages, c->k_zero_pages, c->v_code_pages,
                          c->v_scale_pages, c->v_zero_pages, c->k_residual_scratch, c->v_residual_scratch};
    for (const void* p : ptrs) {
        if (!p) return KIVI_ERR_NULL_POINTER;
        if (!aligned16(p)) return KIVI_ERR_ALIGNMENT;
    }
    if (c->num_blocks < 0 || c->num_slots <= 0) return KIVI_ERR_RANGE;
    return KIVI_OK;
}

CachePtrs cache_ptrs(const kivi_cache& c) {
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

// Split of the context over CTAs. Work units are (sequence, kv head); when there are fewer of
// them than about two per SM, each unit's quantised tokens are cut into equal chunks (a multiple
// of the key group, at least kMinChunkTokens) so that the grid still fills the machine.
struct SplitPlan { int chunk_tokens; int max_chunks; };

SplitPlan plan_split(const Geom& g, int n, int max_old_tokens) {
    SplitPlan sp;
    const long long units = (long long)n * g.nkv;
    // as many chunks as fill the resident CTA slots (three per SM) without exceeding them: a second, partial
    // wave costs more than the idle slots (the residual CTAs a split adds are tiny and do not count)
    const long long slots = 3LL * sm_count();
    long long want = slots / units;
    if (want < 1) want = 1;
    // Long contexts: finer chunks are worth their partial results when they round the number of waves better
    // (256 units x 5 chunks = 2.9 waves of 444 slots instead of 256 CTAs on 444 slots), as long as a chunk stays
    // long enough to amortise a CTA's start and end (kLongChunkTokens; below it splitting measured slower).
    {
        auto efficiency = [&](long long w) {
            const long long ctas = units * w, waves = (ctas + slots - 1) / slots;
            return (double)ctas / (double)(waves * slots);
        };
        double best = efficiency(want);
        for (long long w = want + 1; w <= 64 && max_old_tokens / w >= kLongChunkTokens; ++w)
            if (efficiency(w) > best + 0.02) { best = efficiency(w); want = w; }
    }
    long long chunk = (max_old_tokens + want - 1) / want;
    if (chunk < kMinChunkTokens) chunk = kMinChunkTokens;
    const int gran = g.g > 64 ? g.g : ((64 + g.g - 1) / g.g) * g.g;  // multiple of the group, >= 64
    chunk = ((chunk + gran - 1) / gran) * gran;
    sp.chunk_tokens = (int)chunk;
    sp.max_chunks = max_old_tokens > 0 ? (int)((max_old_tokens + chunk - 1) / chunk) : 1;
    if (sp.max_chunks > 1) sp.max_chunks += 1;   // a split context gives the fp16 residual a CTA of its own
    return sp;
}

constexpr size_t kWsAlign = 256;
size_t align_up(size_t x) { return (x + kWsAlign - 1) / kWsAlign * kWsAlign; }

// Tensor-core kernel: how the (sequence, kv head) units are cut into jobs. The model behind the choice, fitted
// to measurements: three CTAs are resident on a multiprocessor and share it, so three equal jobs take one
// "round" s together; CTAs are handed out in index order, so a multiprocessor's queue of j jobs runs as
// floor(j / 3) full rounds and a last round of one or two jobs, which finish sooner than a full round but not in
// proportion (a lone CTA reaches 0.6 of the multiprocessor's rate -- 0.5 with key groups shorter than 128 tokens --, two reach 0.87). A launch takes as long as the
// longest queue, ceil(jobs / multiprocessors); a job costs a start-up plus its share of the unit; a launch that
// cuts anything pays for the merge kernel. Candidates: every unit in k parts; or whole units for as many full
// rounds as there are and the units left over in k2 parts each (the small jobs start last and even out the end).
// Lengths live on the device, so the plan assumes every unit is as long as the longest the launch allows.
constexpr int kJobFixedCost = 40;      // start-up of a CTA, in weight units of a 128-channel head with 128-token groups (about 7 us)
constexpr int kMergeCost = 60;         // the merge kernel behind a launch that cuts units
constexpr double kCutMargin = 1.05;    // a cut has to promise this much before it is preferred to whole units
constexpr int kMaxParts = 64;

JobPlan plan_jobs(const Geom& g, int n, int max_old_tokens) {
    const long long wg = g.g / 16;
    const long long w = (long long)(max_old_tokens / g.g) * wg + (long long)((g.r + g.g + 15) / 16) * 4;
    const long long units = (long long)n * g.nkv;
    const long long sms = sm_count(), resident = decode_mma_ctas_per_sm();
    // The two costs are times, and the time of a weight unit depends on the geometry: a 64-channel head takes
    // about 0.6 of a 128-channel one, and short key groups cost more per token (per group the query is rescaled and the zero-point term formed: about 4.7 tiles' worth). Fitted on
    // head 128 / group 128 (0.17 us per unit) and head 64 / group 32 (0.22 us per unit).
    const double unit_us = (g.d >= 128 ? 0.107 : 0.064) * (1.0 + 4.74 / (double)wg);
    const double fixed = kJobFixedCost * 0.17 / unit_us, merge = kMergeCost * 0.17 / unit_us;
    // a CTA alone on a multiprocessor: short groups leave a lone warp per scheduler waiting on itself more often
    const double lone_rate = wg >= 8 ? 0.6 : 0.5;
    long long kcap = w / (2 * wg);           // a part keeps at least two key groups' worth
    if (kcap < 1) kcap = 1;
    if (kcap > kMaxParts) kcap = kMaxParts;
    JobPlan best = {0, 1, (int)units, 1};
    // KIVI_DECODE_PARTS=k in the environment cuts every unit into k parts instead (for measurements)
    static const int forced = [] { const char* e = getenv("KIVI_DECODE_PARTS"); return e ? atoi(e) : 0; }();
    if (forced > 0) { best.k2 = forced < kcap ? forced : (int)kcap; return best; }
    auto job = [&](long long k) { return fixed + (double)((w + k - 1) / k); };
    // time of a queue of `jobs` equal jobs on one multiprocessor, in rounds
    auto rounds_of = [&](long long jobs) {
        const long long rest = jobs % resident;
        const double last = rest == 0 ? 0.0 : (double)rest / resident / (rest == 1 ? lone_rate : (rest == 2 ? 0.87 : 1.0));
        return (double)(jobs / resident) + last;
    };
    double best_t = rounds_of((units + sms - 1) / sms) * job(1);   // whole units
    auto offer = [&](double t, long long u1, long long k1, long long u2, long long k2) {
        if (t * kCutMargin < best_t) {
            best_t = t * kCutMargin;
            best.units1 = (int)u1; best.k1 = (int)k1; best.units2 = (int)u2; best.k2 = (int)k2;
        }
    };
    for (long long k = 2; k <= kcap; ++k)                          // every unit in k parts
        offer(rounds_of((units * k + sms - 1) / sms) * job(k) + merge, 0, 1, units, k);
    const long long full = units / (sms * resident);                // whole units in full rounds, the rest cut finer
    if (full >= 1 && units % (sms * resident) != 0) {
        const long long whole = full * sms * resident, rest = units - whole;
        for (long long k2 = 2; k2 <= kcap; ++k2)
            offer((double)full * job(1) + rounds_of((rest * k2 + sms - 1) / sms) * job(k2) + merge, whole, 1, rest, k2);
    }
    return best;
}

// Workspace: the partials of whichever decode kernel the geometry runs on (both, sized for the larger, where a
// dense launch takes the tensor-core kernel and a sparse one the generic kernel).
struct WsLayout { size_t ml_off, o_off, total; };
WsLayout ws_layout(const Geom& g, int n, int max_old_tokens) {
    WsLayout w;
    size_t parts = 0;
    if (decode_mma_supports(g, -1)) parts = (size_t)plan_jobs(g, n, max_old_tokens).slots() * g.qpk;
    if (!decode_mma_supports(g, 0)) {
        const SplitPlan sp = plan_split(g, n, max_old_tokens);
        const size_t chunk_parts = sp.max_chunks > 1 ? (size_t)n * g.nkv * sp.max_chunks * g.qpk : 0;
        if (chunk_parts > parts) parts = chunk_parts;
    }
    w.ml_off = 0;
    w.o_off = w.ml_off + align_up(parts * 2 * sizeof(float));
    w.total = w.o_off + align_up(parts * g.d * sizeof(float));
    if (w.total < kWsAlign) w.total = kWsAlign;   // never 0, which the size query returns for invalid arguments
    return w;
}

}  // namespace

size_t decode_workspace_total(const Geom& g, int n, int max_old_tokens) {
    return ws_layout(g, n, max_old_tokens).total;
}

int run_decode(const Geom& g, const CachePtrs& cache, const SeqAddressing& seq, const __half* q, float* out,
               __half* out_h, int n, int max_seq_cap, int max_old_tokens, int retained_pages, void* ws,
               size_t ws_bytes, cudaStream_t stream, const int* retained_dev) {
    DecodeParams p;
    p.geom = g; p.cache = cache; p.seq = seq; p.q = q; p.out = out; p.out_h = out_h; p.n = n;
    p.max_seq = max_seq_cap; p.retained_pages = retained_pages; p.retained_dev = retained_dev; p.status = nullptr;
    const bool tensor_path = decode_mma_supports(g, retained_dev ? 0 : retained_pages);
    const WsLayout wl = ws_layout(g, n, max_old_tokens);
    bool need_ws;
    if (tensor_path) {
        p.plan = plan_jobs(g, n, max_old_tokens);
        p.chunk_tokens = 0; p.max_chunks = 1;
        need_ws = p.plan.slots() > 0;
    } else {
        const SplitPlan sp = plan_split(g, n, max_old_tokens);
        p.plan = JobPlan{0, 1, 0, 1};
        p.chunk_tokens = sp.chunk_tokens;
        p.max_chunks = sp.max_chunks;
        need_ws = sp.max_chunks > 1;
    }
    if (need_ws) {
        if (!ws || ws_bytes < wl.total) return KIVI_ERR_WORKSPACE;
        if (!aligned16(ws)) return KIVI_ERR_ALIGNMENT;
    }
    unsigned char* base = static_cast<unsigned char*>(ws);
    p.ws_ml = base ? reinterpret_cast<float*>(base + wl.ml_off) : nullptr;
    p.ws_o = base ? reinterpret_cast<float*>(base + wl.o_off) : nullptr;
    cudaError_t e;
    if (tensor_path) {
        e = launch_decode_mma(p, stream);
        if (e == cudaSuccess) e = launch_decode_part_merge(p, stream);   // nothing to do unless a unit was cut
    } else {
        e = launch_decode_generic(p, stream);
        if (e == cudaSuccess) e = launch_decode_merge(p, stream);        // nothing to do unless the plan splits the context
    }
    return e == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

namespace {

// ------------------------------------------------------------------ reference lane (ABI v1) --

// Constants of the reference artefacts (snapshot decode_attention_kivi_paged_library_flash.cu:14-25;
// integrations/vllm_kivi/source_patch.py:661-672).
constexpr int kRefD = 128, kRefB = 32, kRefG = 32, kRefR = 128;
constexpr int kRefOldBlocks = 124, kRefLQ = kRefOldBlocks * kRefB, kRefMaxQueries = 160;
constexpr int kRefMaxNew = kRefR + kRefB;

Geom ref_geom(int nh, int nkv) {
    kivi_geometry s = {nh, nkv, kRefD, kRefB, kRefG, kRefR};
    return make_geom(s);
}

[[noreturn]] void die(const char* what, cudaError_t e) {
    fprintf(stderr, "CUDA error %s in %s\n", cudaGetErrorString(e), what);
    exit(1);
}

// Workspace of the v1 decode symbols. Their signatures carry no workspace and the reference's entry points
// never allocate, so the partial results of a cut launch live in a fixed array of the library's device image
// (every GPU that loads the library carries it; all v1 calls on a device share it, like the reference's calls
// share nothing they would have to). Its size covers the largest v1 launch (160 queries, 4096 tokens) on a B200's
// 148 multiprocessors; on a device whose launch plan would need more, the first call falls back to cudaMalloc.
constexpr int kMaxDevices = 64;
constexpr size_t kRefWorkspaceBytes = 2560u << 10;
}  // namespace
}  // namespace kivi
static __device__ __align__(256) unsigned char g_ref_workspace[kivi::kRefWorkspaceBytes];
namespace kivi {
namespace {
void* g_ref_ws[kMaxDevices];
size_t g_ref_ws_bytes[kMaxDevices];
std::once_flag g_ref_ws_once[kMaxDevices];

void* ref_workspace(const Geom& g, int n, size_t* bytes, cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) die("cudaGetDevice", e);
    if (dev < 0 || dev >= kMaxDevices) { fprintf(stderr, "device index %d out of range\n", dev); exit(1); }
    (void)g; (void)n;
    std::call_once(g_ref_ws_once[dev], [dev, stream] {
        size_t need = 0;
        const Geom lanes[2] = {ref_geom(40, 8), ref_geom(20, 4)};
        for (const Geom& lane : lanes)
            for (int q = 1; q <= kRefMaxQueries; ++q) {
                size_t t = ws_layout(lane, q, kRefLQ).total;
                if (t > need) need = t;
            }
        void* ptr = nullptr;
        if (need <= kRefWorkspaceBytes && cudaGetSymbolAddress(&ptr, g_ref_workspace) == cudaSuccess && ptr) {
            g_ref_ws[dev] = ptr;
            g_ref_ws_bytes[dev] = kRefWorkspaceBytes;
            return;
        }
        cudaError_t err = cudaMalloc(&g_ref_ws[dev], need);
        if (err != cudaSuccess) die("cudaMalloc(v1 decode workspace)", err);
        err = cudaMemsetAsync(g_ref_ws[dev], 0, need, stream);
        if (err != cudaSuccess) die("cudaMemsetAsync(v1 decode workspace)", err);
        g_ref_ws_bytes[dev] = need;
    });
    *bytes = g_ref_ws_bytes[dev];
    return g_ref_ws[dev];
}

CachePtrs ref_cache(const unsigned char* kc, const kivi_f16* ks, const kivi_f16* kz, const unsigned char* vc,
                    const kivi_f16* vs, const kivi_f16* vz, const kivi_f16* kr, const kivi_f16* vr) {
    CachePtrs c;
    c.k_code = const_cast<unsigned char*>(kc);
    c.k_scale = reinterpret_cast<__half*>(const_cast<kivi_f16*>(ks));
    c.k_zero = reinterpret_cast<__half*>(const_cast<kivi_f16*>(kz));
    c.v_code = const_cast<unsigned char*>(vc);
    c.v_scale = reinterpret_cast<__half*>(const_cast<kivi_f16*>(vs));
    c.v_zero = reinterpret_cast<__half*>(const_cast<kivi_f16*>(vz));
    c.k_scratch = reinterpret_cast<__half*>(const_cast<kivi_f16*>(kr));
    c.v_scratch = reinterpret_cast<__half*>(const_cast<kivi_f16*>(vr));
    c.num_blocks = c.num_slots = 0x7fffffff;   // the reference's signatures state no pool sizes
    return c;
}

void ref_decode(int nh, int nkv, const kivi_f16* Q, const int* seq_lens, int seq_len, const int* bt,
                const CachePtrs& cache, int n, int retained, float* O, cudaStream_t stream) {
    if (n <= 0) return;
    const Geom g = ref_geom(nh, nkv);
    SeqAddressing a;
    a.seq_lens = seq_lens; a.seq_len_scalar = seq_len;
    a.block_tables = bt; a.bt_stride = 0; a.bt_width = kRefOldBlocks;
    a.slot_ids = nullptr; a.slot_shared = 1;
    size_t ws_bytes = 0;
    void* ws = ref_workspace(g, n, &ws_bytes, stream);
    int rc = run_decode(g, cache, a, reinterpret_cast<const __half*>(Q), O, nullptr, n, kRefLQ + kRefR, kRefLQ, retained, ws, ws_bytes,
                        stream);
    if (rc != KIVI_OK) { fprintf(stderr, "jac_launch: %s\n", kivi_b200_status_string(rc)); exit(1); }
}

void ref_write(int nkv, const CachePtrs& cache, const kivi_f16* new_k, const kivi_f16* new_v, const int* bt,
               int start_seq_len, int num_new, cudaStream_t stream) {
    WriteParams p;
    p.geom = ref_geom(nkv * 5, nkv);
    p.cache = cache;
    p.seq.seq_lens = nullptr; p.seq.seq_len_scalar = start_seq_len;
    p.seq.block_tables = bt; p.seq.bt_stride = 0; p.seq.bt_width = kRefOldBlocks;
    p.seq.slot_ids = nullptr; p.seq.slot_shared = 1;
    p.new_k = reinterpret_cast<const __half*>(new_k);
    p.new_v = reinterpret_cast<const __half*>(new_v);
    p.new_offsets = nullptr; p.num_new_scalar = num_new; p.n = 1;
    cudaError_t e = launch_cache_write(p, num_new, stream);
    if (e != cudaSuccess) die("KIVI cache write", e);
}

}  // namespace
}  // namespace kivi

using namespace kivi;

// ------------------------------------------------------------------ ABI v2 -------------------

extern "C" int kivi_b200_abi_version(void) { return JACQ_KIVI_B200_ABI_VERSION; }

extern "C" const char* kivi_b200_status_string(int status) {
    switch (status) {
        case KIVI_OK: return "ok";
        case KIVI_ERR_NULL_POINTER: return "a required pointer is NULL";
        case KIVI_ERR_GEOMETRY: return "unsupported or inconsistent KIVI geometry";
        case KIVI_ERR_RANGE: return "batch, length or count out of range";
        case KIVI_ERR_ALIGNMENT: return "a tensor base is not 16-byte aligned";
        case KIVI_ERR_WORKSPACE: return "decode workspace missing or too small";
        case KIVI_ERR_CUDA: return "the CUDA runtime reported an error on launch";
        case KIVI_ERR_BLOCK_TABLE: return "block table too narrow for the stated sequence lengths";
        default: return "unknown status";
    }
}

extern "C" int kivi_b200_validate_geometry(const kivi_geometry* geom, int* fast_path) {
    int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    if (fast_path) *fast_path = decode_mma_supports(make_geom(*geom), -1) ? 1 : 0;
    return KIVI_OK;
}

extern "C" int kivi_b200_cache_write(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* new_k,
                                     const kivi_f16* new_v, const int32_t* block_tables, int max_blocks_per_seq,
                                     const int32_t* start_seq_lens, const int32_t* new_offsets,
                                     const int32_t* slot_ids, int batch, int max_new_per_seq, int max_start_seq_len,
                                     cudaStream_t stream) {
    int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    rc = check_cache(cache);
    if (rc != KIVI_OK) return rc;
    if (!new_k || !new_v || !block_tables || !start_seq_lens || !new_offsets) return KIVI_ERR_NULL_POINTER;
    if (!aligned16(new_k) || !aligned16(new_v)) return KIVI_ERR_ALIGNMENT;
    if (batch < 0 || max_new_per_seq < 0 || max_start_seq_len < 0 || max_blocks_per_seq < 0) return KIVI_ERR_RANGE;
    if (batch == 0 || max_new_per_seq == 0) return KIVI_OK;
    if (!slot_ids && batch > cache->num_slots) return KIVI_ERR_RANGE;
    const Geom g = make_geom(*geom);
    const long long max_end = (long long)max_start_seq_len + max_new_per_seq;
    if (max_end > 0x3fffffff) return KIVI_ERR_RANGE;
    if ((long long)split_old((int)max_end, g.r, g.g) > (long long)max_blocks_per_seq * g.b) return KIVI_ERR_BLOCK_TABLE;
    WriteParams p;
    p.geom = g;
    p.cache = cache_ptrs(*cache);
    p.seq.seq_lens = start_seq_lens; p.seq.seq_len_scalar = 0;
    p.seq.block_tables = block_tables; p.seq.bt_stride = max_blocks_per_seq; p.seq.bt_width = max_blocks_per_seq;
    p.seq.slot_ids = slot_ids; p.seq.slot_shared = 0;
    p.new_k = reinterpret_cast<const __half*>(new_k);
    p.new_v = reinterpret_cast<const __half*>(new_v);
    p.new_offsets = new_offsets; p.num_new_scalar = 0; p.n = batch;
    return launch_cache_write(p, max_new_per_seq, stream) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

extern "C" size_t kivi_b200_decode_workspace_bytes(const kivi_geometry* geom, int batch, int max_seq_len) {
    if (check_geometry(geom) != KIVI_OK || batch <= 0 || max_seq_len < 0) return 0;
    const Geom g = make_geom(*geom);
    return ws_layout(g, batch, split_old(max_seq_len, g.r, g.g)).total;
}

extern "C" int kivi_b200_decode_plan(const kivi_geometry* geom, int batch, int max_seq_len, int32_t plan_out[4]) {
    const int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    if (!plan_out) return KIVI_ERR_NULL_POINTER;
    if (batch <= 0 || max_seq_len < 0) return KIVI_ERR_RANGE;
    const Geom g = make_geom(*geom);
    if (!decode_mma_supports(g, -1)) { plan_out[0] = 0; plan_out[1] = 1; plan_out[2] = batch * g.nkv; plan_out[3] = 1; return KIVI_OK; }
    const JobPlan pl = plan_jobs(g, batch, split_old(max_seq_len, g.r, g.g));
    plan_out[0] = pl.units1; plan_out[1] = pl.k1; plan_out[2] = pl.units2; plan_out[3] = pl.k2;
    return KIVI_OK;
}

extern "C" int kivi_b200_decode_part_items(const kivi_geometry* geom, int seq_len, int part, int parts, int32_t items_out[4]) {
    const int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    if (!items_out) return KIVI_ERR_NULL_POINTER;
    if (seq_len < 0 || parts < 1 || part < 0 || part >= parts) return KIVI_ERR_RANGE;
    const Geom g = make_geom(*geom);
    if (g.g % 16) return KIVI_ERR_GEOMETRY;
    const DecodeBounds b = decode_bounds(seq_len, g.r, g.g, -1, 0x3fffffff / g.b, g.b);
    const UnitShape u = unit_shape_of(b.old_valid, b.res_valid, g.g);
    const SegmentItems it = segment_items(u, g.g / 16, (int)share_begin(u.w, parts, part), (int)share_begin(u.w, parts, part + 1));
    items_out[0] = it.g0; items_out[1] = it.g1; items_out[2] = it.t0; items_out[3] = it.t1;
    return KIVI_OK;
}

extern "C" int kivi_b200_decode_workspace_init(void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!workspace) return workspace_bytes ? KIVI_ERR_NULL_POINTER : KIVI_OK;
    return cudaMemsetAsync(workspace, 0, workspace_bytes, stream) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

extern "C" int kivi_b200_decode_sparse(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                                       const int32_t* retained_block_tables, int max_blocks_per_seq,
                                       const int32_t* seq_lens, const int32_t* retained_pages, const int32_t* slot_ids,
                                       int batch, int max_seq_len, float* out, void* workspace, size_t workspace_bytes,
                                       cudaStream_t stream) {
    int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    rc = check_cache(cache);
    if (rc != KIVI_OK) return rc;
    if (!q || !retained_block_tables || !seq_lens || !retained_pages || !out) return KIVI_ERR_NULL_POINTER;
    if (!aligned16(q) || !aligned16(out)) return KIVI_ERR_ALIGNMENT;
    if (batch < 0 || max_seq_len < 0 || max_seq_len > 0x3fffffff || max_blocks_per_seq < 0) return KIVI_ERR_RANGE;
    if (batch == 0) return KIVI_OK;
    if (!slot_ids && batch > cache->num_slots) return KIVI_ERR_RANGE;
    const Geom g = make_geom(*geom);
    SeqAddressing a;
    a.seq_lens = seq_lens; a.seq_len_scalar = 0;
    a.block_tables = retained_block_tables; a.bt_stride = max_blocks_per_seq; a.bt_width = max_blocks_per_seq;
    a.slot_ids = slot_ids; a.slot_shared = 0;
    // the launch is planned for the longest dense context; a sequence scans min(its count, its dense pages,
    // the table width) pages of its compact table
    long long max_old = split_old(max_seq_len, g.r, g.g);
    if (max_old > (long long)max_blocks_per_seq * g.b) max_old = (long long)max_blocks_per_seq * g.b;
    return run_decode(g, cache_ptrs(*cache), a, reinterpret_cast<const __half*>(q), out, nullptr, batch, max_seq_len,
                      (int)max_old, -1, workspace, workspace_bytes, stream, retained_pages);
}

namespace {
int decode_v2(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q, const int32_t* block_tables,
              int max_blocks_per_seq, const int32_t* seq_lens, const int32_t* slot_ids, int batch, int max_seq_len,
              float* out, kivi_f16* out_h, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    rc = check_cache(cache);
    if (rc != KIVI_OK) return rc;
    if (!q || !block_tables || !seq_lens || (!out && !out_h)) return KIVI_ERR_NULL_POINTER;
    if (!aligned16(q) || !aligned16(out) || !aligned16(out_h)) return KIVI_ERR_ALIGNMENT;
    if (batch < 0 || max_seq_len < 0 || max_seq_len > 0x3fffffff || max_blocks_per_seq < 0) return KIVI_ERR_RANGE;
    if (batch == 0) return KIVI_OK;
    if (!slot_ids && batch > cache->num_slots) return KIVI_ERR_RANGE;
    const Geom g = make_geom(*geom);
    const int max_old = split_old(max_seq_len, g.r, g.g);
    if ((long long)max_old > (long long)max_blocks_per_seq * g.b) return KIVI_ERR_BLOCK_TABLE;
    SeqAddressing a;
    a.seq_lens = seq_lens; a.seq_len_scalar = 0;
    a.block_tables = block_tables; a.bt_stride = max_blocks_per_seq; a.bt_width = max_blocks_per_seq;
    a.slot_ids = slot_ids; a.slot_shared = 0;
    // max_seq_len also clamps a device-side length beyond the stated bound, so the launch plan and
    // the workspace stay valid whatever seq_lens holds.
    return run_decode(g, cache_ptrs(*cache), a, reinterpret_cast<const __half*>(q), out, reinterpret_cast<__half*>(out_h), batch,
                      max_seq_len, max_old, -1, workspace, workspace_bytes, stream);
}
}  // namespace

extern "C" int kivi_b200_decode(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                                const int32_t* block_tables, int max_blocks_per_seq, const int32_t* seq_lens,
                                const int32_t* slot_ids, int batch, int max_seq_len, float* out, void* workspace,
                                size_t workspace_bytes, cudaStream_t stream) {
    if (!out) return KIVI_ERR_NULL_POINTER;
    return decode_v2(geom, cache, q, block_tables, max_blocks_per_seq, seq_lens, slot_ids, batch, max_seq_len, out, nullptr,
                     workspace, workspace_bytes, stream);
}

extern "C" int kivi_b200_decode_f16(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                                    const int32_t* block_tables, int max_blocks_per_seq, const int32_t* seq_lens,
                                    const int32_t* slot_ids, int batch, int max_seq_len, kivi_f16* out, void* workspace,
                                    size_t workspace_bytes, cudaStream_t stream) {
    if (!out) return KIVI_ERR_NULL_POINTER;
    return decode_v2(geom, cache, q, block_tables, max_blocks_per_seq, seq_lens, slot_ids, batch, max_seq_len, nullptr, out,
                     workspace, workspace_bytes, stream);
}

// ------------------------------------------------------------------ decode without a workspace --
//
// Scratch of kivi_b200_decode_noalloc: a fixed array in the library's device image, so the entry
// point never allocates. Every GPU that loads the library carries these bytes until the process
// exits. All calls share it.
static __device__ __align__(256) unsigned char g_noalloc_scratch[KIVI_B200_NOALLOC_SCRATCH_BYTES];

namespace {
// Device address of g_noalloc_scratch, looked up once per device (std::call_once: two host threads may make
// their first call at the same time). In host code the array's name is only a handle for the runtime, not
// an address a kernel could use.
void* g_noalloc_ptr[kivi::kMaxDevices];
std::once_flag g_noalloc_once[kivi::kMaxDevices];
}  // namespace

extern "C" int kivi_b200_decode_noalloc(const kivi_geometry* geom, const kivi_cache* cache, const kivi_f16* q,
                                        const int32_t* block_tables, int max_blocks_per_seq,
                                        const int32_t* seq_lens, const int32_t* slot_ids, int batch,
                                        int max_seq_len, float* out, cudaStream_t stream) {
    int rc = check_geometry(geom);
    if (rc != KIVI_OK) return rc;
    rc = check_cache(cache);
    if (rc != KIVI_OK) return rc;
    if (!q || !block_tables || !seq_lens || !out) return KIVI_ERR_NULL_POINTER;
    if (!aligned16(q) || !aligned16(out)) return KIVI_ERR_ALIGNMENT;
    if (batch < 0 || max_seq_len < 0 || max_seq_len > 0x3fffffff || max_blocks_per_seq < 0) return KIVI_ERR_RANGE;
    if (batch == 0) return KIVI_OK;
    if (!slot_ids && batch > cache->num_slots) return KIVI_ERR_RANGE;
    const Geom g = make_geom(*geom);
    const int max_old = split_old(max_seq_len, g.r, g.g);
    if ((long long)max_old > (long long)max_blocks_per_seq * g.b) return KIVI_ERR_BLOCK_TABLE;
    // the launch plan decides how much scratch this call needs; refuse what the fixed array cannot hold
    const WsLayout wl = ws_layout(g, batch, max_old);
    if (wl.total > (size_t)KIVI_B200_NOALLOC_SCRATCH_BYTES) return KIVI_ERR_WORKSPACE;

    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return KIVI_ERR_CUDA;
    // first call on this device (with it current): resolve the array's device address
    std::call_once(g_noalloc_once[dev], [dev] {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) == cudaSuccess) g_noalloc_ptr[dev] = ptr;
    });
    void* scratch = g_noalloc_ptr[dev];
    if (!scratch) return KIVI_ERR_CUDA;
    // nothing in the array has to start from a known value: a launch reads only the partials it wrote itself
    SeqAddressing a;
    a.seq_lens = seq_lens; a.seq_len_scalar = 0;
    a.block_tables = block_tables; a.bt_stride = max_blocks_per_seq; a.bt_width = max_blocks_per_seq;
    a.slot_ids = slot_ids; a.slot_shared = 0;
    return run_decode(g, cache_ptrs(*cache), a, reinterpret_cast<const __half*>(q), out, nullptr, batch, max_seq_len, max_old,
                      -1, scratch, (size_t)KIVI_B200_NOALLOC_SCRATCH_BYTES, stream);
}

extern "C" int kivi_b200_gemv_f16(const kivi_f16* w, const kivi_f16* x, kivi_f16* y_f16, float* y_f32, int out_dim,
                                  int in_dim, int batch, cudaStream_t stream) {
    if (!w || !x || (!y_f16 && !y_f32)) return KIVI_ERR_NULL_POINTER;
    if (out_dim <= 0 || in_dim <= 0 || batch < 1 || batch > 64 || in_dim % 8) return KIVI_ERR_RANGE;
    if (!aligned16(w) || !aligned16(x)) return KIVI_ERR_ALIGNMENT;
    const __half* wh = reinterpret_cast<const __half*>(w);
    const __half* xh = reinterpret_cast<const __half*>(x);
    __half* yh = reinterpret_cast<__half*>(y_f16);
    if (skinny_gemm_supports(in_dim, batch))
        return launch_skinny_gemm(wh, xh, yh, y_f32, out_dim, in_dim, batch, stream) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
    return launch_gemv(wh, xh, yh, y_f32, out_dim, in_dim, batch, stream) == cudaSuccess ? KIVI_OK : KIVI_ERR_CUDA;
}

// ------------------------------------------------------------------ ABI v1 symbols -----------

#define KIVI_V1_CACHE_ARGS                                                                              \
    const unsigned char* K_CODE_PAGES, const kivi_f16* K_SCALE_PAGES, const kivi_f16* K_ZERO_PAGES,      \
    const unsigned char* V_CODE_PAGES, const kivi_f16* V_SCALE_PAGES, const kivi_f16* V_ZERO_PAGES,      \
    const kivi_f16* K_RESIDUAL_SCRATCH, const kivi_f16* V_RESIDUAL_SCRATCH
#define KIVI_V1_CACHE                                                                                    \
    ref_cache(K_CODE_PAGES, K_SCALE_PAGES, K_ZERO_PAGES, V_CODE_PAGES, V_SCALE_PAGES, V_ZERO_PAGES,      \
              K_RESIDUAL_SCRATCH, V_RESIDUAL_SCRATCH)

extern "C" void jac_launch(const kivi_f16* Q, const int* BLOCK_TABLE, KIVI_V1_CACHE_ARGS, int SEQ_LEN, float* O,
                           cudaStream_t stream) {
    ref_decode(40, 8, Q, nullptr, SEQ_LEN, BLOCK_TABLE, KIVI_V1_CACHE, 1, -1, O, stream);
}
extern "C" void jac_launch_tp2_local(const kivi_f16* Q, const int* BLOCK_TABLE, KIVI_V1_CACHE_ARGS, int SEQ_LEN,
                                     float* O, cudaStream_t stream) {
    ref_decode(20, 4, Q, nullptr, SEQ_LEN, BLOCK_TABLE, KIVI_V1_CACHE, 1, -1, O, stream);
}
extern "C" void jac_launch_batched(const kivi_f16* Q, const int* SEQ_LENS, const int* BLOCK_TABLE, KIVI_V1_CACHE_ARGS,
                                   int NUM_QUERIES, float* O, cudaStream_t stream) {
    if (NUM_QUERIES > kRefMaxQueries) { fprintf(stderr, "NUM_QUERIES out of range for jac_launch_batched: %d\n", NUM_QUERIES); exit(1); }
    ref_decode(40, 8, Q, SEQ_LENS, 0, BLOCK_TABLE, KIVI_V1_CACHE, NUM_QUERIES, -1, O, stream);
}
extern "C" void jac_launch_batched_tp2_local(const kivi_f16* Q, const int* SEQ_LENS, const int* BLOCK_TABLE,
                                             KIVI_V1_CACHE_ARGS, int NUM_QUERIES, float* O, cudaStream_t stream) {
    if (NUM_QUERIES > kRefMaxQueries) { fprintf(stderr, "NUM_QUERIES out of range for jac_launch_batched_tp2_local: %d\n", NUM_QUERIES); exit(1); }
    ref_decode(20, 4, Q, SEQ_LENS, 0, BLOCK_TABLE, KIVI_V1_CACHE, NUM_QUERIES, -1, O, stream);
}
extern "C" void jac_launch_sparse_retained(const kivi_f16* Q, const int* RETAINED_BLOCK_TABLE, KIVI_V1_CACHE_ARGS,
                                           int SEQ_LEN, int NUM_RETAINED_PAGES, float* O, cudaStream_t stream) {
    ref_decode(40, 8, Q, nullptr, SEQ_LEN, RETAINED_BLOCK_TABLE, KIVI_V1_CACHE, 1,
               NUM_RETAINED_PAGES < 0 ? 0 : NUM_RETAINED_PAGES, O, stream);
}
extern "C" void jac_launch_sparse_retained_tp2_local(const kivi_f16* Q, const int* RETAINED_BLOCK_TABLE,
                                                     KIVI_V1_CACHE_ARGS, int SEQ_LEN, int NUM_RETAINED_PAGES, float* O,
                                                     cudaStream_t stream) {
    ref_decode(20, 4, Q, nullptr, SEQ_LEN, RETAINED_BLOCK_TABLE, KIVI_V1_CACHE, 1,
               NUM_RETAINED_PAGES < 0 ? 0 : NUM_RETAINED_PAGES, O, stream);
}

extern "C" void jac_launch_cache_write(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES, kivi_f16* K_ZERO_PAGES,
                                       unsigned char* V_CODE_PAGES, kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                       kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                       const kivi_f16* NEW_K, const kivi_f16* NEW_V, const int* BLOCK_TABLE,
                                       int SEQ_LEN, cudaStream_t stream) {
    ref_write(8, KIVI_V1_CACHE, NEW_K, NEW_V, BLOCK_TABLE, SEQ_LEN - 1, 1, stream);
}
extern "C" void jac_launch_cache_write_batched(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES,
                                               kivi_f16* K_ZERO_PAGES, unsigned char* V_CODE_PAGES,
                                               kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                               kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                               const kivi_f16* NEW_K, const kivi_f16* NEW_V, const int* BLOCK_TABLE,
                                               int START_SEQ_LEN, int NUM_NEW, cudaStream_t stream) {
    if (NUM_NEW < 1 || NUM_NEW > kRefMaxNew) {
        fprintf(stderr, "NUM_NEW out of range for jac_launch_cache_write_batched: %d\n", NUM_NEW);
        exit(1);
    }
    ref_write(8, KIVI_V1_CACHE, NEW_K, NEW_V, BLOCK_TABLE, START_SEQ_LEN, NUM_NEW, stream);
}

extern "C" void kivi_b200_cache_write_launch(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES,
                                             kivi_f16* K_ZERO_PAGES, unsigned char* V_CODE_PAGES,
                                             kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                             kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                             const kivi_f16* NEW_K, const kivi_f16* NEW_V, const int64_t* SLOT_MAPPING,
                                             const int* BLOCK_TABLE, int seq_len, int NKV_RUNTIME, cudaStream_t stream) {
    (void)SLOT_MAPPING;  // validated by the caller, never used for addressing (source_patch.py:1675)
    if (NKV_RUNTIME < 1) { fprintf(stderr, "NKV_RUNTIME out of range for kivi_cache_write_launch: %d\n", NKV_RUNTIME); exit(1); }
    ref_write(NKV_RUNTIME, KIVI_V1_CACHE, NEW_K, NEW_V, BLOCK_TABLE, seq_len - 1, 1, stream);
}
extern "C" void kivi_b200_cache_write_batched_launch(unsigned char* K_CODE_PAGES, kivi_f16* K_SCALE_PAGES,
                                                     kivi_f16* K_ZERO_PAGES, unsigned char* V_CODE_PAGES,
                                                     kivi_f16* V_SCALE_PAGES, kivi_f16* V_ZERO_PAGES,
                                                     kivi_f16* K_RESIDUAL_SCRATCH, kivi_f16* V_RESIDUAL_SCRATCH,
                                                     const kivi_f16* NEW_K, const kivi_f16* NEW_V,
                                                     const int64_t* SLOT_MAPPING, const int* BLOCK_TABLE,
                                                     int START_SEQ_LEN, int NUM_NEW, int NKV_RUNTIME,
                                                     cudaStream_t stream) {
    (void)SLOT_MAPPING;
    if (NUM_NEW < 1) return;
    if (NKV_RUNTIME < 1) { fprintf(stderr, "NKV_RUNTIME out of range for kivi_cache_write_batched_launch: %d\n", NKV_RUNTIME); exit(1); }
    ref_write(NKV_RUNTIME, KIVI_V1_CACHE, NEW_K, NEW_V, BLOCK_TABLE, START_SEQ_LEN, NUM_NEW, stream);
}

// The reference's binding declares the hand-CUDA writer with C++ linkage and __half pointers
// (integrations/vllm_kivi/source_patch.py:624-637); export those exact names too.
void kivi_cache_write_launch(unsigned char* K_CODE_PAGES, __half* K_SCALE_PAGES, __half* K_ZERO_PAGES,
                             unsigned char* V_CODE_PAGES, __half* V_SCALE_PAGES, __half* V_ZERO_PAGES,
                             __half* K_RESIDUAL_SCRATCH, __half* V_RESIDUAL_SCRATCH, const __half* NEW_K,
                             const __half* NEW_V, const int64_t* SLOT_MAPPING, const int* BLOCK_TABLE, int seq_len,
                             int NKV_RUNTIME, cudaStream_t stream) {
    kivi_b200_cache_write_launch(K_CODE_PAGES, (kivi_f16*)K_SCALE_PAGES, (kivi_f16*)K_ZERO_PAGES, V_CODE_PAGES,
                                 (kivi_f16*)V_SCALE_PAGES, (kivi_f16*)V_ZERO_PAGES, (kivi_f16*)K_RESIDUAL_SCRATCH,
                                 (kivi_f16*)V_RESIDUAL_SCRATCH, (const kivi_f16*)NEW_K, (const kivi_f16*)NEW_V,
                                 SLOT_MAPPING, BLOCK_TABLE, seq_len, NKV_RUNTIME, stream);
}
void kivi_cache_write_batched_launch(unsigned char* K_CODE_PAGES, __half* K_SCALE_PAGES, __half* K_ZERO_PAGES,
                                     unsigned char* V_CODE_PAGES, __half* V_SCALE_PAGES, __half* V_ZERO_PAGES,
                                     __half* K_RESIDUAL_SCRATCH, __half* V_RESIDUAL_SCRATCH, const __half* NEW_K,
                                     const __half* NEW_V, const int64_t* SLOT_MAPPING, const int* BLOCK_TABLE,
                                     int START_SEQ_LEN, int NUM_NEW, int NKV_RUNTIME, cudaStream_t stream) {
    kivi_b200_cache_write_batched_launch(K_CODE_PAGES, (kivi_f16*)K_SCALE_PAGES, (kivi_f16*)K_ZERO_PAGES, V_CODE_PAGES,
                                         (kivi_f16*)V_SCALE_PAGES, (kivi_f16*)V_ZERO_PAGES,
                                         (kivi_f16*)K_RESIDUAL_SCRATCH, (kivi_f16*)V_RESIDUAL_SCRATCH,
                                         (const kivi_f16*)NEW_K, (const kivi_f16*)NEW_V, SLOT_MAPPING, BLOCK_TABLE,
                                         START_SEQ_LEN, NUM_NEW, NKV_RUNTIME, stream);
}
