// C ABI of the B200 expert-FFN path (declared in include/moexb.h): argument checks, launches, resident layers.
#include "moexb.h"
#include "common.cuh"
#include "router.cuh"
#include "experts_simt.cuh"
#include "formats.cuh"
#include "stream.cuh"
#include "tiled.cuh"
#include "prefill.cuh"
#include "decode_stack.cuh"
#include "ep.cuh"
#include "gguf_ingest.h"
#include "st_ingest.h"
#include "gguf_quant.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

using namespace moexb;

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

#define REQUIRE(cond, ...) do { if (!(cond)) return fail(MOEXB_ERR_ARG, __VA_ARGS__); } while (0)
#define CUDA_TRY(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) return fail(MOEXB_ERR_CUDA, "%s: %s", #x, cudaGetErrorString(e_)); } while (0)
#define LAUNCHED(name) do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return fail(MOEXB_ERR_CUDA, "launch of %s: %s", name, cudaGetErrorString(e_)); \
    g_launches.fetch_add(1, std::memory_order_relaxed); } while (0)
std::atomic<long long> g_launches{0};

inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Launch with programmatic stream serialization: the kernel's blocks may be scheduled before the kernel ahead of it in
// the stream has finished, and wait for it inside (pdl_wait in common.cuh). Only kernels that call pdl_wait before they
// touch their inputs are launched this way. MOEXB_PDL=0 in the environment turns it off (plain launches).
static bool pdl_enabled() {
    static const bool on = [] { const char* e = getenv("MOEXB_PDL"); return !(e && e[0] == '0'); }();
    return on;
}
template <typename... P, typename... A>
static cudaError_t launch_dep(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}
// Function attributes (the opt-in to more than 48 KB of dynamic shared memory, occupancy figures) belong to one device, so
// "once" means once per device: keyed by the device that is current in the calling thread, which is the one the launch
// that follows goes to.
constexpr int MAX_DEVICES = 64;
struct PerDeviceOnce {
    std::mutex mu;
    bool done[MAX_DEVICES] = {};
    cudaError_t err[MAX_DEVICES] = {};
    template <class F>
    cudaError_t run(F&& f) {
        int dev = -1;
        const cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) { err[dev] = f(); done[dev] = true; }
        return err[dev];
    }
};
inline bool fmt_ok(int fmt) { return fmt == FMT_SYM_F32 || fmt == FMT_SYM_F16 || fmt == FMT_ZP; }

// Calls f.template operator()<FMT>() for the run-time format.
template <class F>
int by_fmt(int fmt, F&& f) {
    switch (fmt) {
        case FMT_SYM_F32: return f.template operator()<FMT_SYM_F32>();
        case FMT_SYM_F16: return f.template operator()<FMT_SYM_F16>();
        case FMT_ZP: return f.template operator()<FMT_ZP>();
    }
    return fail(MOEXB_ERR_ARG, "unknown expert format %d", fmt);
}

// ---- half-normal quantile tables of the synthetic generator ---------------------------------------------------------

float half_to_float_host(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// table[i] = fp16 bits of sigma * q, q = the (i + 0.5) / N quantile of |N(0, 1)|, found by bisection on erf.
void build_table(double sigma, uint16_t* table) {
    for (int i = 0; i < SYNTH_TABLE_N; i++) {
        const double p = (i + 0.5) / SYNTH_TABLE_N;
        double lo = 0, hi = 10;
        for (int it = 0; it < 80; it++) {
            const double mid = 0.5 * (lo + hi);
            if (std::erf(mid / std::sqrt(2.0)) < p) lo = mid; else hi = mid;
        }
        table[i] = __half_as_ushort(__float2half_rn((float)(sigma * 0.5 * (lo + hi))));
    }
}
struct Tables { uint16_t s[SYNTH_TABLE_N], d[SYNTH_TABLE_N]; };
const Tables& host_tables() {
    static Tables t;
    static std::once_flag once;
    std::call_once(once, [] { build_table(0.02, t.s); build_table(0.01, t.d); });
    return t;
}

}  // namespace

constexpr int STAGING_BLOBS = 32;

struct moexb_ctx {
    int device = 0, max_tokens = 0, max_experts = 0, top_k = 0;
    uint16_t *table_s = nullptr, *table_d = nullptr;  // device copies of the synthetic tables
    // workspace of the layer-level calls
    float *xf = nullptr, *xn = nullptr, *logits = nullptr, *w = nullptr, *act = nullptr, *ypair = nullptr, *moe = nullptr;
    int *idx = nullptr, *counts = nullptr, *nitems = nullptr;
    moexb_pair_item* items = nullptr;
    moexb_pair* pairs = nullptr;
    const uint8_t** slots = nullptr;  // decode: K+1 blob pointers
    float* wts = nullptr;             // decode: K+1 weights
    // streaming (tensor-core) path
    uint16_t *xs = nullptr, *act_split = nullptr;       // activations / act as 16-bit hi + lo halves, permuted
    moexb_pair_item* subs = nullptr;                    // sub-items of at most 8 pairs
    int *nsub = nullptr, *err = nullptr;
    moexb_pair_item* subs2 = nullptr; int* nsub2 = nullptr;   // second sub-item list (the down tiles of the tensor-core path)
    int* route_done = nullptr;                          // per token tile: blocks of the routing kernel that have finished (returns to zero)
    int sms = 0, path = 0;                              // path: 0 = streaming kernels, 1 = fp32 SIMT kernels
    int fused_decode = 1;                               // one-token residual stacks run as one cooperative launch
    int pairs_per_pass = 8;                             // sub-item width of the tiled streaming kernels from 8 tokens on
    int prefill_min_tokens = 256;                       // batches from this size on use the tcgen05 grouped GEMM
    uint8_t* staging = nullptr;                         // reference-layout blobs on their way into a tiled image
    std::vector<void*> owned;
    // optional per-kernel timing of the layer-level calls
    bool profiling = false;
    struct Rec { int tag; cudaEvent_t a, b; };
    std::vector<Rec> recs;
    std::vector<cudaEvent_t> spare;
};

namespace {
// Brackets the launches made inside its scope with two events on the stream when the context is profiling.
struct ProfScope {
    moexb_ctx* c; cudaStream_t st; cudaEvent_t a = nullptr, b = nullptr; int tag;
    ProfScope(moexb_ctx* c_, int tag_, cudaStream_t st_) : c(c_), st(st_), tag(tag_) {
        if (!c || !c->profiling) return;
        auto get = [&] { cudaEvent_t e; if (c->spare.empty()) cudaEventCreate(&e); else { e = c->spare.back(); c->spare.pop_back(); } return e; };
        a = get(); b = get();
        cudaEventRecord(a, st);
    }
    ~ProfScope() { if (a) { cudaEventRecord(b, st); c->recs.push_back({tag, a, b}); } }
};
}  // namespace

#define PROF_CAT2(a, b) a##b
#define PROF_CAT(a, b) PROF_CAT2(a, b)
#define PROF(ctx, tag, stream) ProfScope PROF_CAT(prof_scope_, __LINE__)(ctx, tag, S(stream))

struct moexb_layer {
    moexb_ctx* ctx = nullptr;
    int fmt = 0, n_routed = 0, first_local = 0, n_local = 0, router_dtype = 0, layout = 0;
    uint8_t* image = nullptr;               // n_local + 1 blobs: the held routed experts, then the shared expert
    void* router = nullptr;                 // [n_routed + 1][H]
    const uint8_t** slot_table = nullptr;   // device, n_routed + 1 pointers
    std::vector<const uint8_t*> slot_host;
    // per expert id (index n_routed = the shared expert): weights were put there by an upload, a synthetic fill or a file load.
    // The image starts zeroed, so an expert that was never loaded contributes zeros; the shared expert runs for every token,
    // so the layer-level calls refuse to run it unloaded instead of silently adding nothing.
    std::vector<uint8_t> loaded;
};

extern "C" {

const char* moexb_last_error(void) { return g_err; }
int moexb_version(void) { return 1; }
size_t moexb_expert_bytes(int fmt) { return fmt_ok(fmt) ? expert_bytes(fmt) : 0; }

// ---- router ------------------------------------------------------------------------------------------------------

}  // extern "C"
template <typename WT>
static int gemv_any(const WT* W, const float* x, float* y, int I, int O, void* stream, int rows) {
    REQUIRE(W && x && y, "gemv: null pointer");
    REQUIRE(I > 0 && I % 128 == 0 && O > 0 && rows > 0, "gemv: I=%d must be a positive multiple of 128, O=%d, rows=%d", I, O, rows);
    if (rows >= 8) {
        constexpr int WARPS = 4, TO = 4, TR = 8;  // 16 outputs x 8 rows per block: 17 x 8 blocks for the 64-token router
        const int smem = TR * I * (int)sizeof(float);
        REQUIRE(smem <= 200 * 1024, "gemv: I=%d is too large for the batched kernel", I);
        static PerDeviceOnce once;
        const cudaError_t attr_err = once.run([] { return cudaFuncSetAttribute(gemm_rows_k<WT, WARPS, TO, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); });
        if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "gemv: shared memory attribute: %s", cudaGetErrorString(attr_err));
        CUDA_TRY(launch_dep(gemm_rows_k<WT, WARPS, TO, TR>, dim3((O + WARPS * TO - 1) / (WARPS * TO), (rows + TR - 1) / TR), WARPS * 32, smem, S(stream), W, x, y, I, O, rows));
    } else {
        constexpr int WARPS = 8;
        CUDA_TRY(launch_dep(gemv_rows_k<WT, WARPS>, dim3((O + WARPS - 1) / WARPS, rows), WARPS * 32, 0, S(stream), W, x, y, I, O));
    }
    LAUNCHED("gemv");
    return MOEXB_OK;
}
extern "C" {
int moexb_gemv_f16(const void* W, const float* x, float* y, int I, int O, void* stream, int rows) {
    return gemv_any(static_cast<const __half*>(W), x, y, I, O, stream, rows);
}
int moexb_gemv_f32(const float* W, const float* x, float* y, int I, int O, void* stream, int rows) {
    return gemv_any(W, x, y, I, O, stream, rows);
}

static int topk_launch(const float* logits, int E, int K, int norm, int* idx, float* w, void* stream, int T, int ld,
                       const uint8_t* const* slot_table, const uint8_t** slots_out, float* wts_out,
                       moexb_pair_item* dsubs = nullptr, moexb_pair* dpairs = nullptr, int* dnsub = nullptr) {
    REQUIRE(logits && idx && w, "router_topk: null pointer");
    REQUIRE(E > 0 && E % 32 == 0 && E <= 1024, "router_topk: E=%d must be a multiple of 32 up to 1024", E);
    REQUIRE(K > 0 && K < 32 && K <= E, "router_topk: K=%d out of range", K);
    REQUIRE(T > 0 && ld >= E, "router_topk: T=%d, ld=%d", T, ld);
    constexpr int WARPS = 2;
    const TopkOut o{idx, w, slot_table, slots_out, wts_out, dsubs, dpairs, dnsub};
    if (E <= 256) CUDA_TRY(launch_dep(router_topk_k<WARPS, 8>, (T + WARPS - 1) / WARPS, WARPS * 32, 0, S(stream), logits, E, K, norm, ld, T, o));
    else CUDA_TRY(launch_dep(router_topk_k<WARPS, 32>, (T + WARPS - 1) / WARPS, WARPS * 32, 0, S(stream), logits, E, K, norm, ld, T, o));
    LAUNCHED("router_topk");
    return MOEXB_OK;
}
int moexb_router_topk(const float* logits, int E, int K, int norm, int* idx, float* w, void* stream, int T, int ld) {
    return topk_launch(logits, E, K, norm, idx, w, stream, T, ld, nullptr, nullptr, nullptr);
}

// ---- routed experts ------------------------------------------------------------------------------------------------

static int decode_launch(moexb_ctx* prof, int fmt, const uint8_t* const* slots, const float* w, int K, const float* x, float* act,
                         float* out, void* stream, const int* nh) {
    REQUIRE(slots && w && x && act && out, "experts_forward: null pointer");
    REQUIRE(K > 0 && K <= 16, "experts_forward: K=%d out of range 1..16", K);
    return by_fmt(fmt, [&]<int FMT>() {
        constexpr int WARPS = 8;
        {
            PROF(prof, MOEXB_PROF_GATE_UP, stream);
            decode_gate_up_k<FMT, WARPS><<<dim3(EI / WARPS, K), WARPS * 32, 0, S(stream)>>>(slots, K, nh, x, act);
            LAUNCHED("decode_gate_up");
        }
        PROF(prof, MOEXB_PROF_DOWN, stream);
        decode_down_k<FMT, WARPS, 16><<<EH / WARPS, WARPS * 32, K * pad32_size(EI) * sizeof(float), S(stream)>>>(slots, w, K, nh, act, out);
        LAUNCHED("decode_down");
        return (int)MOEXB_OK;
    });
}
}  // extern "C"

// The context whose workspace the pointer-level one-token entry point may use on each device (moexb_set_default_ctx).
static std::mutex g_default_lock;
static moexb_ctx* g_default_ctx[MAX_DEVICES] = {};
static int stream_experts(moexb_ctx* c, int fmt, const moexb_pair* pairs, float* act32, float* ypair, void* stream);
static int split_launch(moexb_ctx* c, const float* x, int rows, bool f16, void* stream);

extern "C" {

int moexb_set_default_ctx(moexb_ctx* ctx, int device) {
    REQUIRE(device >= 0 && device < MAX_DEVICES, "set_default_ctx: device %d", device);
    REQUIRE(!ctx || ctx->device == device, "set_default_ctx: the context belongs to device %d", ctx ? ctx->device : -1);
    std::lock_guard<std::mutex> lock(g_default_lock);
    g_default_ctx[device] = ctx;
    return MOEXB_OK;
}

int moexb_experts_forward(int fmt, const uint8_t* const* slots, const float* w, int K, const float* x, float* act,
                          float* out, void* stream, const int* nh) {
    moexb_ctx* c = nullptr;
    {
        int dev = -1;
        if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < MAX_DEVICES) { std::lock_guard<std::mutex> lock(g_default_lock); c = g_default_ctx[dev]; }
    }
    if (!c || c->path == 1 || K > c->max_tokens * (c->top_k + 1)) return decode_launch(nullptr, fmt, slots, w, K, x, act, out, stream, nh);
    // With a default context: the streaming tensor-core kernels on the caller's reference-layout blobs. The K experts are K
    // one-pair sub-items of the one token; act receives the fp32 activations as the reference's scratch does.
    REQUIRE(slots && w && x && act && out, "experts_forward: null pointer");
    REQUIRE(K > 0 && K <= 16, "experts_forward: K=%d out of range 1..16", K);
    REQUIRE(fmt_ok(fmt), "experts_forward: unknown expert format %d", fmt);
    cudaStream_t st = S(stream);
    plan_decode_k<<<1, 32, 0, st>>>(slots, w, K, nh, c->subs, c->pairs, c->nsub);
    LAUNCHED("plan_decode");
    int rc = split_launch(c, x, 1, false, stream);
    if (rc != MOEXB_OK) return rc;
    if (nh) CUDA_TRY(cudaMemsetAsync(c->ypair, 0, (size_t)K * EH * sizeof(float), st));   // rows of the experts beyond *nh stay zero
    rc = stream_experts(c, fmt, c->pairs, act, c->ypair, stream);
    if (rc != MOEXB_OK) return rc;
    pairs_reduce_k<<<dim3((EH / 4 + 255) / 256, 1), 256, 0, st>>>(c->ypair, nullptr, out, K, EH, nullptr);
    LAUNCHED("pairs_reduce");
    return MOEXB_OK;
}

static int pairs_launch(moexb_ctx* prof, int fmt, const moexb_pair_item* items, const int* nitems, int grid_items, const moexb_pair* pairs,
                        const float* X, float* act, float* ypair, void* stream) {
    REQUIRE(items && pairs && X && act && ypair, "pairs_forward: null pointer");
    REQUIRE(grid_items > 0 && grid_items <= 65535, "pairs_forward: %d items", grid_items);
    return by_fmt(fmt, [&]<int FMT>() {
        constexpr int WARPS = 8;
        {
            PROF(prof, MOEXB_PROF_GATE_UP, stream);
            pairs_gate_up_k<FMT, WARPS><<<dim3(EI / WARPS, grid_items), WARPS * 32, 0, S(stream)>>>(items, pairs, X, act, nitems);
            LAUNCHED("pairs_gate_up");
        }
        PROF(prof, MOEXB_PROF_DOWN, stream);
        pairs_down_k<FMT, WARPS><<<dim3(EH / WARPS, grid_items), WARPS * 32, 0, S(stream)>>>(items, pairs, act, ypair, nitems);
        LAUNCHED("pairs_down");
        return (int)MOEXB_OK;
    });
}
int moexb_pairs_forward(int fmt, const moexb_pair_item* items, int n_items, const moexb_pair* pairs, const float* X,
                        float* act, float* ypair, void* stream) {
    if (n_items == 0) return fmt_ok(fmt) ? MOEXB_OK : fail(MOEXB_ERR_ARG, "unknown expert format %d", fmt);
    return pairs_launch(nullptr, fmt, items, nullptr, n_items, pairs, X, act, ypair, stream);
}
int moexb_pairs_forward_dev(int fmt, const moexb_pair_item* items, const int* nitems, int max_items,
                            const moexb_pair* pairs, const float* X, float* act, float* ypair, void* stream) {
    REQUIRE(nitems, "pairs_forward_dev: null item count");
    return pairs_launch(nullptr, fmt, items, nitems, max_items, pairs, X, act, ypair, stream);
}

int moexb_pairs_reduce(const float* ypair, const float* ycpu, float* moe, int K, int D, int T, const int* use_cpu, void* stream) {
    REQUIRE(ypair && moe, "pairs_reduce: null pointer");
    REQUIRE(K > 0 && D > 0 && D % 4 == 0 && T > 0 && T <= 65535, "pairs_reduce: K=%d D=%d T=%d", K, D, T);
    pairs_reduce_k<<<dim3((D / 4 + 255) / 256, T), 256, 0, S(stream)>>>(ypair, ycpu, moe, K, D, use_cpu);
    LAUNCHED("pairs_reduce");
    return MOEXB_OK;
}

int moexb_gated_add_rows(float* out, const float* sh, const float* gl, int gl_stride, int D, int T, void* stream) {
    REQUIRE(out && sh && gl, "gated_add_rows: null pointer");
    REQUIRE(D > 0 && T > 0 && T <= 65535 && gl_stride >= 0, "gated_add_rows: D=%d T=%d", D, T);
    gated_add_rows_k<<<dim3((D + 255) / 256, T), 256, 0, S(stream)>>>(out, sh, gl, gl_stride, D);
    LAUNCHED("gated_add_rows");
    return MOEXB_OK;
}

int moexb_group_pairs(const int* idx, const float* w, int T, int K, int E, const uint8_t* const* slot_table,
                      moexb_pair_item* items, moexb_pair* pairs, int* nitems, int* counts, void* stream) {
    REQUIRE(idx && w && slot_table && items && pairs && nitems && counts, "group_pairs: null pointer");
    REQUIRE(T > 0 && K > 0 && E > 0 && E <= 1024, "group_pairs: T=%d K=%d E=%d", T, K, E);
    constexpr int WARPS = 8;
    group_count_k<WARPS><<<(E + WARPS - 1) / WARPS, WARPS * 32, 0, S(stream)>>>(idx, T * K, E, counts);
    LAUNCHED("group_count");
    group_scatter_k<WARPS><<<(E + WARPS - 1) / WARPS, WARPS * 32, 0, S(stream)>>>(idx, w, T, K, E, slot_table, counts, items, pairs, nitems, nullptr, 0);
    LAUNCHED("group_scatter");
    return MOEXB_OK;
}

int moexb_shared_expert_add(int fmt, const uint8_t* blob, const float* gl, int gl_stride, const float* X, int T,
                            float* out, float* scratch, void* stream) {
    REQUIRE(blob && gl && X && out && scratch, "shared_expert_add: null pointer");
    REQUIRE(T > 0 && T <= 65535, "shared_expert_add: T=%d", T);
    // The shared expert is one item holding every token with weight 1; the gate enters in gated_add_rows.
    // scratch: act [T][I], sh [T][H], then the item and its T pairs.
    float *act = scratch, *sh = scratch + (size_t)T * EI;
    moexb_pair_item* item = reinterpret_cast<moexb_pair_item*>(sh + (size_t)T * EH);
    moexb_pair* pairs = reinterpret_cast<moexb_pair*>(item + 1);
    identity_pairs_k<<<(T + 255) / 256, 256, 0, S(stream)>>>(blob, T, item, pairs);
    LAUNCHED("identity_pairs");
    int rc = pairs_launch(nullptr, fmt, item, nullptr, 1, pairs, X, act, sh, stream);
    if (rc != MOEXB_OK) return rc;
    gated_add_rows_k<<<dim3((EH + 255) / 256, T), 256, 0, S(stream)>>>(out, sh, gl, gl_stride, EH);
    LAUNCHED("gated_add_rows");
    return MOEXB_OK;
}

// ---- formats ---------------------------------------------------------------------------------------------------------

int moexb_dequant(int fmt, const uint8_t* blob, float* out, void* stream) {
    REQUIRE(blob && out, "dequant: null pointer");
    return by_fmt(fmt, [&]<int FMT>() {
        dequant_k<FMT><<<(unsigned)((CHUNKS + 255) / 256), 256, 0, S(stream)>>>(blob, out);
        LAUNCHED("dequant");
        return (int)MOEXB_OK;
    });
}

int moexb_q4k_dequant(const uint8_t* blocks, long long n, float* y, void* stream) {
    REQUIRE(blocks && y, "q4k_dequant: null pointer");
    REQUIRE(n > 0 && n % 256 == 0, "q4k_dequant: n=%lld must be a positive multiple of 256", n);
    const long long threads = n / 256 * 4;
    q4k_dequant_k<<<(unsigned)((threads + 255) / 256), 256, 0, S(stream)>>>(blocks, n / 256, y);
    LAUNCHED("q4k_dequant");
    return MOEXB_OK;
}

int moexb_q4k_to_zp(const uint8_t* gate, const uint8_t* up, const uint8_t* down, uint8_t* blob, void* stream) {
    REQUIRE(gate && up && down && blob, "q4k_to_zp: null pointer");
    q4k_to_zp_k<<<(unsigned)((CHUNKS / 8 + 127) / 128), 128, 0, S(stream)>>>(gate, up, down, blob);
    LAUNCHED("q4k_to_zp");
    return MOEXB_OK;
}

// ---- synthetic experts --------------------------------------------------------------------------------------------------

static int synth_launch(int fmt, unsigned seed, int layer, int e0, int n, uint8_t* dst, const uint16_t* ts, const uint16_t* td, void* stream) {
    REQUIRE(dst && ts && td, "synth_experts: null pointer");
    REQUIRE(n > 0 && n <= 65535 && e0 >= 0 && layer >= 0, "synth_experts: layer=%d e0=%d n=%d", layer, e0, n);
    return by_fmt(fmt, [&]<int FMT>() {
        const size_t work = FMT == FMT_ZP ? CHUNKS / 8 : Q_BYTES / 4;
        synth_experts_k<FMT><<<dim3((unsigned)((work + 255) / 256), n), 256, 0, S(stream)>>>(seed, layer, e0, dst, ts, td);
        LAUNCHED("synth_experts");
        return (int)MOEXB_OK;
    });
}

int moexb_synth_expert_host(int fmt, unsigned seed, int layer, int expert, uint8_t* dst) {
    REQUIRE(dst && fmt_ok(fmt), "synth_expert_host: bad argument");
    const Tables& t = host_tables();
    if (fmt == FMT_ZP) {
        for (size_t sb = 0; sb < CHUNKS / 8; sb++) {
            uint8_t blk[144], *qb, *cs, *sup;
            synth_q4k_block(seed, layer, expert, sb, t.d, blk);
            zp_block_dst(dst, sb, qb, cs, sup);
            q4k_block_to_zp(blk, qb, cs, sup);
        }
        return MOEXB_OK;
    }
    for (size_t i = 0; i < Q_BYTES / 4; i++) {
        const uint32_t w = synth_nibble_word(seed, layer, expert, i);
        memcpy(dst + 4 * i, &w, 4);
    }
    for (size_t g = 0; g < CHUNKS / 2; g++) {
        const uint16_t h = synth_scale_h(seed, layer, expert, g, t.s);
        if (fmt == FMT_SYM_F16) memcpy(dst + Q_BYTES + 2 * g, &h, 2);
        else { const float f = half_to_float_host(h); memcpy(dst + Q_BYTES + 4 * g, &f, 4); }
    }
    return MOEXB_OK;
}

int moexb_synth_q4k_host(unsigned seed, int layer, int expert, uint8_t* gate, uint8_t* up, uint8_t* down) {
    REQUIRE(gate && up && down, "synth_q4k_host: null pointer");
    const Tables& t = host_tables();
    constexpr size_t NB = (size_t)EH * EI / 256;
    for (size_t sb = 0; sb < 3 * NB; sb++) {
        uint8_t* d = sb < NB ? gate + sb * 144 : sb < 2 * NB ? up + (sb - NB) * 144 : down + (sb - 2 * NB) * 144;
        synth_q4k_block(seed, layer, expert, sb, t.d, d);
    }
    return MOEXB_OK;
}

// ---- context and resident layers -----------------------------------------------------------------------------------------

}  // extern "C"
template <class T>
static int dev_alloc(moexb_ctx* ctx, T** p, size_t n) {
    void* v = nullptr;
    cudaError_t e = cudaMalloc(&v, n * sizeof(T));
    if (e != cudaSuccess) return fail(MOEXB_ERR_NOMEM, "cudaMalloc of %zu bytes: %s", n * sizeof(T), cudaGetErrorString(e));
    ctx->owned.push_back(v);
    *p = static_cast<T*>(v);
    return MOEXB_OK;
}

extern "C" {
int moexb_ctx_create(int device, int max_tokens, int max_experts, int top_k, moexb_ctx** out) {
    REQUIRE(out, "ctx_create: null output");
    REQUIRE(max_tokens > 0 && max_tokens <= 65535 && max_experts > 0 && max_experts % 32 == 0 && max_experts <= 1024 && top_k > 0 && top_k <= 15,
            "ctx_create: max_tokens=%d max_experts=%d top_k=%d", max_tokens, max_experts, top_k);
    CUDA_TRY(cudaSetDevice(device));
    moexb_ctx* c = new (std::nothrow) moexb_ctx;
    if (!c) return fail(MOEXB_ERR_NOMEM, "out of host memory");
    c->device = device; c->max_tokens = max_tokens; c->max_experts = max_experts; c->top_k = top_k;
    const size_t T = max_tokens, P = T * (top_k + 1);
    int rc = MOEXB_OK;
    auto A = [&](auto** p, size_t n) { if (rc == MOEXB_OK) rc = dev_alloc(c, p, n); };
    A(&c->table_s, SYNTH_TABLE_N); A(&c->table_d, SYNTH_TABLE_N);
    A(&c->xf, T * EH); A(&c->xn, T * EH); A(&c->logits, T * (max_experts + 1)); A(&c->w, T * top_k); A(&c->idx, T * top_k);
    A(&c->act, P * EI); A(&c->ypair, P * EH); A(&c->moe, T * EH);
    A(&c->counts, (size_t)max_experts); A(&c->nitems, 1); A(&c->items, (size_t)max_experts + 1); A(&c->pairs, P);
    A(&c->slots, (size_t)top_k + 1); A(&c->wts, (size_t)top_k + 1);
    A(&c->xs, T * 2 * EH); A(&c->act_split, P * 2 * EI); A(&c->subs, (size_t)max_experts + 1 + P / ST_MAXP + 1);
    A(&c->nsub, 2); A(&c->err, 1); A(&c->subs2, (size_t)max_experts + 1 + P / (PF_NMAX / 2) + 1); A(&c->nsub2, 1); A(&c->route_done, (size_t)max_tokens); A(&c->staging, (size_t)STAGING_BLOBS * expert_bytes(FMT_ZP));
    if (rc == MOEXB_OK && cudaMemset(c->err, 0, sizeof(int)) != cudaSuccess) rc = fail(MOEXB_ERR_CUDA, "ctx_create: memset");
    if (rc == MOEXB_OK && cudaMemset(c->route_done, 0, (size_t)max_tokens * sizeof(int)) != cudaSuccess) rc = fail(MOEXB_ERR_CUDA, "ctx_create: memset");
    if (rc == MOEXB_OK && cudaDeviceGetAttribute(&c->sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) rc = fail(MOEXB_ERR_CUDA, "ctx_create: device attribute");
    if (rc != MOEXB_OK) { moexb_ctx_destroy(c); return rc; }
    const Tables& t = host_tables();
    cudaError_t e = cudaMemcpy(c->table_s, t.s, sizeof t.s, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(c->table_d, t.d, sizeof t.d, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { moexb_ctx_destroy(c); return fail(MOEXB_ERR_CUDA, "table upload: %s", cudaGetErrorString(e)); }
    *out = c;
    return MOEXB_OK;
}

int moexb_ctx_destroy(moexb_ctx* ctx) {
    if (!ctx) return MOEXB_OK;
    {
        std::lock_guard<std::mutex> lock(g_default_lock);
        for (moexb_ctx*& d : g_default_ctx) if (d == ctx) d = nullptr;
    }
    for (void* p : ctx->owned) cudaFree(p);
    for (auto& r : ctx->recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (auto e : ctx->spare) cudaEventDestroy(e);
    delete ctx;
    return MOEXB_OK;
}

int moexb_synth_experts(moexb_ctx* ctx, int fmt, unsigned seed, int layer, int e0, int n, uint8_t* dst, void* stream) {
    REQUIRE(ctx, "synth_experts: null context");
    return synth_launch(fmt, seed, layer, e0, n, dst, ctx->table_s, ctx->table_d, stream);
}

int moexb_layer_create(moexb_ctx* ctx, int fmt, int n_routed, int first_local, int n_local, int router_dtype, int layout, moexb_layer** out) {
    REQUIRE(ctx && out, "layer_create: null pointer");
    REQUIRE(fmt_ok(fmt), "layer_create: unknown expert format %d", fmt);
    REQUIRE(n_routed > 0 && n_routed % 32 == 0 && n_routed <= ctx->max_experts, "layer_create: n_routed=%d (context allows %d)", n_routed, ctx->max_experts);
    REQUIRE(first_local >= 0 && n_local >= 0 && first_local + n_local <= n_routed, "layer_create: local experts [%d, %d) outside 0..%d", first_local, first_local + n_local, n_routed);
    REQUIRE(router_dtype == MOEXB_F32 || router_dtype == 2, "layer_create: router dtype %d", router_dtype);
    REQUIRE(layout == MOEXB_LAYOUT_TILED || layout == MOEXB_LAYOUT_REFERENCE, "layer_create: layout %d", layout);
    CUDA_TRY(cudaSetDevice(ctx->device));
    moexb_layer* L = new (std::nothrow) moexb_layer;
    if (!L) return fail(MOEXB_ERR_NOMEM, "out of host memory");
    L->ctx = ctx; L->fmt = fmt; L->n_routed = n_routed; L->first_local = first_local; L->n_local = n_local; L->router_dtype = router_dtype; L->layout = layout;
    const size_t eb = expert_bytes(fmt);
    cudaError_t e = cudaMalloc((void**)&L->image, (size_t)(n_local + 1) * eb);
    if (e == cudaSuccess) e = cudaMemset(L->image, 0, (size_t)(n_local + 1) * eb);
    L->loaded.assign(n_routed + 1, 0);
    if (e == cudaSuccess) e = cudaMalloc(&L->router, (size_t)(n_routed + 1) * EH * (router_dtype == MOEXB_F32 ? 4 : 2));
    if (e == cudaSuccess) e = cudaMalloc((void**)&L->slot_table, (size_t)(n_routed + 1) * sizeof(void*));
    if (e == cudaSuccess) {
        L->slot_host.assign(n_routed + 1, nullptr);
        for (int i = 0; i < n_local; i++) L->slot_host[first_local + i] = L->image + (size_t)i * eb;
        L->slot_host[n_routed] = L->image + (size_t)n_local * eb;
        e = cudaMemcpy(L->slot_table, L->slot_host.data(), L->slot_host.size() * sizeof(void*), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) { moexb_layer_destroy(L); return fail(MOEXB_ERR_NOMEM, "layer_create: %s", cudaGetErrorString(e)); }
    *out = L;
    return MOEXB_OK;
}

int moexb_layer_destroy(moexb_layer* L) {
    if (!L) return MOEXB_OK;
    cudaFree(L->image); cudaFree(L->router); cudaFree((void*)L->slot_table);
    delete L;
    return MOEXB_OK;
}

uint8_t* moexb_layer_blob(moexb_layer* L, int e) {
    if (!L || e < 0 || e > L->n_routed) return nullptr;
    return const_cast<uint8_t*>(L->slot_host[e]);
}
const uint8_t* const* moexb_layer_slot_table(moexb_layer* L) { return L ? L->slot_table : nullptr; }
void* moexb_layer_router(moexb_layer* L) { return L ? L->router : nullptr; }

}  // extern "C"

// Reference-layout blobs at src (device) -> the layer's layout at dst, n experts.
static int to_layer_layout(moexb_layer* L, const uint8_t* src, uint8_t* dst, int n, cudaStream_t st) {
    const size_t eb = expert_bytes(L->fmt);
    if (L->layout == MOEXB_LAYOUT_REFERENCE) {
        CUDA_TRY(cudaMemcpyAsync(dst, src, n * eb, cudaMemcpyDeviceToDevice, st));
        return MOEXB_OK;
    }
    return by_fmt(L->fmt, [&]<int FMT>() {
        tile_expert_k<FMT, true><<<dim3(TL_SLICES, n), 256, 0, st>>>(src, dst);
        LAUNCHED("tile_expert");
        return (int)MOEXB_OK;
    });
}

extern "C" {

int moexb_layer_upload_expert(moexb_layer* L, int e, const uint8_t* blob_host) {
    REQUIRE(L && blob_host, "layer_upload_expert: null pointer");
    REQUIRE(e >= 0 && e <= L->n_routed && L->slot_host[e], "layer_upload_expert: expert %d is not held by this layer", e);
    CUDA_TRY(cudaMemcpy(L->ctx->staging, blob_host, expert_bytes(L->fmt), cudaMemcpyHostToDevice));
    const int rc = to_layer_layout(L, L->ctx->staging, const_cast<uint8_t*>(L->slot_host[e]), 1, nullptr);
    if (rc != MOEXB_OK) return rc;
    CUDA_TRY(cudaStreamSynchronize(nullptr));
    L->loaded[e] = 1;
    return MOEXB_OK;
}

int moexb_layer_export_expert(moexb_layer* L, int e, uint8_t* blob_host) {
    REQUIRE(L && blob_host, "layer_export_expert: null pointer");
    REQUIRE(e >= 0 && e <= L->n_routed && L->slot_host[e], "layer_export_expert: expert %d is not held by this layer", e);
    const uint8_t* src = L->slot_host[e];
    if (L->layout == MOEXB_LAYOUT_TILED) {
        const int rc = by_fmt(L->fmt, [&]<int FMT>() {
            tile_expert_k<FMT, false><<<TL_SLICES, 256>>>(src, L->ctx->staging);
            LAUNCHED("untile_expert");
            return (int)MOEXB_OK;
        });
        if (rc != MOEXB_OK) return rc;
        src = L->ctx->staging;
    }
    CUDA_TRY(cudaMemcpy(blob_host, src, expert_bytes(L->fmt), cudaMemcpyDeviceToHost));
    return MOEXB_OK;
}

int moexb_layer_set_router(moexb_layer* L, const void* W_host) {
    REQUIRE(L && W_host, "layer_set_router: null pointer");
    CUDA_TRY(cudaMemcpy(L->router, W_host, (size_t)(L->n_routed + 1) * EH * (L->router_dtype == MOEXB_F32 ? 4 : 2), cudaMemcpyHostToDevice));
    return MOEXB_OK;
}

int moexb_layer_fill_synth(moexb_layer* L, unsigned seed, int layer_index, void* stream) {
    REQUIRE(L, "layer_fill_synth: null layer");
    const size_t eb = expert_bytes(L->fmt);
    moexb_ctx* c = L->ctx;
    // held routed experts, then the shared expert (id n_routed), through the staging buffer in batches
    for (int i = 0; i < L->n_local + 1; i += STAGING_BLOBS) {
        const int n = min(STAGING_BLOBS, L->n_local + 1 - i);
        const int routed = min(n, max(0, L->n_local - i));
        int rc = MOEXB_OK;
        if (routed) rc = synth_launch(L->fmt, seed, layer_index, L->first_local + i, routed, c->staging, c->table_s, c->table_d, stream);
        if (rc == MOEXB_OK && routed < n) rc = synth_launch(L->fmt, seed, layer_index, L->n_routed, 1, c->staging + routed * eb, c->table_s, c->table_d, stream);
        if (rc == MOEXB_OK) rc = to_layer_layout(L, c->staging, L->image + (size_t)i * eb, n, S(stream));
        if (rc != MOEXB_OK) return rc;
    }
    for (int i = 0; i < L->n_local; i++) L->loaded[L->first_local + i] = 1;
    L->loaded[L->n_routed] = 1;
    return MOEXB_OK;
}

// ---- GGUF ingest ----------------------------------------------------------------------------------------------------------

int moexb_gguf_open(const char* path, moexb_gguf** out) {
    REQUIRE(path && out, "gguf_open: null pointer");
    std::string err;
    moexb_gguf* g = gguf_open(path, err);
    if (!g) return fail(MOEXB_ERR_ARG, "gguf_open: %s", err.c_str());
    *out = g;
    return MOEXB_OK;
}

int moexb_gguf_close(moexb_gguf* g) {
    delete g;
    return MOEXB_OK;
}

int moexb_gguf_tensor_count(const moexb_gguf* g) { return g ? (int)g->tensors.size() : 0; }

const char* moexb_gguf_tensor_name(const moexb_gguf* g, int i) {
    return g && i >= 0 && i < (int)g->tensors.size() ? g->tensors[i].name.c_str() : nullptr;
}

int moexb_gguf_tensor(const moexb_gguf* g, const char* name, int* type, int* n_dims, long long* ne, const void** data, long long* nbytes) {
    REQUIRE(g && name, "gguf_tensor: null pointer");
    const GgufTensor* t = g->find(name);
    if (!t) return fail(MOEXB_ERR_ARG, "tensor %s is missing from the GGUF", name);
    if (type) *type = (int)t->type;
    if (n_dims) *n_dims = t->n_dims;
    if (ne) for (int d = 0; d < 4; d++) ne[d] = t->ne[d];
    if (data) *data = t->data;
    if (nbytes) *nbytes = t->nbytes;
    return MOEXB_OK;
}

}  // extern "C"

// A Q4_K tensor of the block with the shape the path needs, or an error naming what differs.
static int gguf_expect(const moexb_gguf* g, const std::string& name, std::initializer_list<long long> ne, const GgufTensor** out) {
    const GgufTensor* t = g->find(name);
    if (!t) return fail(MOEXB_ERR_ARG, "tensor %s is missing from the GGUF", name.c_str());
    int bn, bb;
    if (!gq_block(t->type, bn, bb) || !t->data)
        return fail(MOEXB_ERR_UNSUPPORTED, "layer_load_gguf: %s has ggml type %u, which this loader cannot re-quantise (Q4_K is carried over bit for bit; "
                    "Q5_K, Q6_K, Q8_0, IQ4_NL, IQ4_XS, Q4_0/1, Q5_0/1, F16, BF16 and F32 are refitted to 4 bits)", name.c_str(), t->type);
    bool same = t->n_dims == (int)ne.size();
    int d = 0;
    for (long long v : ne) same = same && t->ne[d++] == v;
    if (!same) return fail(MOEXB_ERR_ARG, "tensor %s has shape [%lld, %lld, %lld, %lld] (%d dimensions), not the one this layer needs",
                           name.c_str(), t->ne[0], t->ne[1], t->ne[2], t->ne[3], t->n_dims);
    *out = t;
    return MOEXB_OK;
}

// One expert from three GGUF tensors of any readable type (gate, up [I][H]; down [H][I]; row-major, `type[k]` blocks) into a
// zero-point blob in the reference layout, on the host: Q4_K rows are carried over bit for bit, the others refitted
// (gguf_quant.h). What gg_experts does per expert (gguf.h:666-694).
static bool expert_to_zp_host(const uint32_t type[3], const uint8_t* const src[3], uint8_t* blob) {
    std::vector<float> w(EH);
    for (int k = 0; k < 3; k++) {
        const int rows = k < 2 ? EI : EH, cols = k < 2 ? EH : EI;
        int bn, bb;
        if (!gq_block(type[k], bn, bb)) return false;
        const size_t row_bytes = (size_t)cols / bn * bb;
        for (int r = 0; r < rows; r++) {
            const size_t row = (size_t)(k == 0 ? 0 : k == 1 ? EI : 0) + r;   // row inside [gate | up] or inside down
            const size_t qoff = k < 2 ? row * (EH / 2) : DOWN_Q_OFF + row * (EI / 2);
            const size_t c0 = k < 2 ? row * (EH / 32) : DOWN_C_OFF + row * (EI / 32);
            uint8_t* qb = blob + qoff;
            uint8_t* cs = blob + Q_BYTES + c0 * 2;
            uint16_t* sup = reinterpret_cast<uint16_t*>(blob + Q_BYTES + CHUNKS * 2 + (c0 / 8) * 4);
            const uint8_t* p = src[k] + (size_t)r * row_bytes;
            if (type[k] == GQ_Q4_K) {
                for (int b = 0; b < cols / 256; b++) q4k_block_to_zp(p + (size_t)b * 144, qb + b * 128, cs + b * 16, reinterpret_cast<uint8_t*>(sup + 2 * b));
            } else {
                if (!gq_dequant(type[k], p, cols, w.data())) return false;
                zp_row_from_values(w.data(), cols, qb, cs, sup);
            }
        }
    }
    return true;
}

// `n` router values at src (F32, F16 or BF16, by ggml type id) into the layer's router dtype at dst (host).
static bool router_rows_to(uint32_t type, const uint8_t* src, long long n, int router_dtype, void* dst) {
    if (type != GGML_F32 && type != GGML_F16 && type != GGML_BF16) return false;
    for (long long i = 0; i < n; i++) {
        float v;
        if (type == GGML_F32) memcpy(&v, src + 4 * i, 4);
        else {
            uint16_t h; memcpy(&h, src + 2 * i, 2);
            if (type == GGML_F16) { __half hh; memcpy(&hh, &h, 2); v = __half2float(hh); }
            else { const uint32_t u = (uint32_t)h << 16; memcpy(&v, &u, 4); }
        }
        if (router_dtype == MOEXB_F32) static_cast<float*>(dst)[i] = v;
        else static_cast<__half*>(dst)[i] = __float2half_rn(v);
    }
    return true;
}

extern "C" {

int moexb_layer_load_gguf(moexb_layer* L, const moexb_gguf* g, int block, int* loaded) {
    REQUIRE(L && g, "layer_load_gguf: null pointer");
    REQUIRE(block >= 0, "layer_load_gguf: block %d", block);
    if (loaded) *loaded = 0;
    if (L->fmt != FMT_ZP) return fail(MOEXB_ERR_UNSUPPORTED, "layer_load_gguf: GGUF expert tensors load into a MOEXB_FMT_ZP layer (this one has format %d)", L->fmt);
    const std::string p = "blk." + std::to_string(block) + ".";
    const long long E = L->n_routed;
    const GgufTensor* t[3];
    int rc = gguf_expect(g, p + "ffn_gate_exps.weight", {EH, EI, E}, &t[0]);
    if (rc == MOEXB_OK) rc = gguf_expect(g, p + "ffn_up_exps.weight", {EH, EI, E}, &t[1]);
    if (rc == MOEXB_OK) rc = gguf_expect(g, p + "ffn_down_exps.weight", {EI, EH, E}, &t[2]);
    if (rc != MOEXB_OK) return rc;
    moexb_ctx* c = L->ctx;
    CUDA_TRY(cudaSetDevice(c->device));
    constexpr size_t PART = (size_t)EH * EI / 256 * 144;  // raw bytes of one expert's gate, up or down
    const size_t eb = expert_bytes(FMT_ZP);
    static_assert(3 * PART <= (size_t)Q_BYTES + 2 * CHUNKS + CHUNKS / 8 * 4, "raw Q4_K of one expert fits a staging blob");
    constexpr int HALF = STAGING_BLOBS / 2;  // raw tensors in the first half of the staging buffer, blobs in the second
    // src[k] = the three raw tensors of the experts to convert, `n` of them, into the layer from slot `dst0` on
    auto convert = [&](const uint8_t* const* src, int n, uint8_t* dst) -> int {
        for (int i = 0; i < n; i++)
            for (int k = 0; k < 3; k++)
                CUDA_TRY(cudaMemcpyAsync(c->staging + i * eb + k * PART, src[3 * i + k], PART, cudaMemcpyHostToDevice, nullptr));
        for (int i = 0; i < n; i++) {
            const uint8_t* raw = c->staging + i * eb;
            q4k_to_zp_k<<<(unsigned)((CHUNKS / 8 + 127) / 128), 128>>>(raw, raw + PART, raw + 2 * PART, c->staging + (HALF + i) * eb);
            LAUNCHED("q4k_to_zp");
        }
        return to_layer_layout(L, c->staging + HALF * eb, dst, n, nullptr);
    };
    // Any tensor in another type than Q4_K: the experts are re-quantised on the host (gguf_quant.h), a batch of them spread
    // over the host threads, and uploaded as finished blobs. per[k]: bytes of one expert inside tensor k.
    auto convert_host = [&](const GgufTensor* const tt[3], int first, int n, uint8_t* dst) -> int {
        size_t per[3]; uint32_t ty[3];
        for (int k = 0; k < 3; k++) { int bn, bb; gq_block(tt[k]->type, bn, bb); per[k] = (size_t)EH * EI / bn * bb; ty[k] = tt[k]->type; }
        std::vector<uint8_t> blobs((size_t)STAGING_BLOBS * eb);
        for (int i = 0; i < n; i += STAGING_BLOBS) {
            const int m = min(STAGING_BLOBS, n - i);
            std::atomic<int> next{0}, bad{0};
            auto work = [&] {
                for (int j; (j = next.fetch_add(1)) < m;) {
                    const uint8_t* src3[3];
                    for (int k = 0; k < 3; k++) src3[k] = tt[k]->data + (size_t)(first + i + j) * per[k];
                    if (!expert_to_zp_host(ty, src3, blobs.data() + (size_t)j * eb)) bad = 1;
                }
            };
            std::vector<std::thread> th;
            const int nt = (int)std::min<unsigned>(std::max(1u, std::thread::hardware_concurrency()), (unsigned)m);
            for (int q = 1; q < nt; q++) th.emplace_back(work);
            work();
            for (auto& x : th) x.join();
            if (bad) return fail(MOEXB_ERR_UNSUPPORTED, "layer_load_gguf: a block of block %d could not be re-quantised", block);
            CUDA_TRY(cudaMemcpy(c->staging, blobs.data(), (size_t)m * eb, cudaMemcpyHostToDevice));
            const int rc2 = to_layer_layout(L, c->staging, dst + (size_t)i * eb, m, nullptr);
            if (rc2 != MOEXB_OK) return rc2;
            CUDA_TRY(cudaStreamSynchronize(nullptr));
        }
        return MOEXB_OK;
    };
    const uint8_t* src[3 * HALF];
    const bool all_q4k = t[0]->type == GGML_Q4_K && t[1]->type == GGML_Q4_K && t[2]->type == GGML_Q4_K;
    if (!all_q4k) {
        rc = convert_host(t, L->first_local, L->n_local, L->image);
        if (rc != MOEXB_OK) return rc;
    } else
    for (int i = 0; i < L->n_local; i += HALF) {
        const int n = min(HALF, L->n_local - i);
        for (int j = 0; j < n; j++)
            for (int k = 0; k < 3; k++) src[3 * j + k] = t[k]->data + (size_t)(L->first_local + i + j) * PART;
        rc = convert(src, n, L->image + (size_t)i * eb);
        if (rc != MOEXB_OK) return rc;
        CUDA_TRY(cudaStreamSynchronize(nullptr));
    }
    int got = L->n_local ? 1 : 0;
    for (int i = 0; i < L->n_local; i++) L->loaded[L->first_local + i] = 1;
    // the shared expert, when the file holds it as Q4_K too
    const GgufTensor *sg = g->find(p + "ffn_gate_shexp.weight"), *su = g->find(p + "ffn_up_shexp.weight"), *sd = g->find(p + "ffn_down_shexp.weight");
    int sbn, sbb;
    if (sg && su && sd && sg->data && su->data && sd->data && gq_block(sg->type, sbn, sbb) && gq_block(su->type, sbn, sbb) && gq_block(sd->type, sbn, sbb) &&
        sg->n_dims == 2 && su->n_dims == 2 &&
        sd->n_dims == 2 && sg->ne[0] == EH && sg->ne[1] == EI && su->ne[0] == EH && su->ne[1] == EI && sd->ne[0] == EI && sd->ne[1] == EH) {
        if (sg->type == GGML_Q4_K && su->type == GGML_Q4_K && sd->type == GGML_Q4_K) {
            src[0] = sg->data; src[1] = su->data; src[2] = sd->data;
            rc = convert(src, 1, L->image + (size_t)L->n_local * eb);
        } else {
            const GgufTensor* st3[3] = {sg, su, sd};
            rc = convert_host(st3, 0, 1, L->image + (size_t)L->n_local * eb);
        }
        if (rc != MOEXB_OK) return rc;
        CUDA_TRY(cudaStreamSynchronize(nullptr));
        got |= 2;
        L->loaded[L->n_routed] = 1;
    }
    // router rows and the shared expert's gate vector
    const GgufTensor *rt = g->find(p + "ffn_gate_inp.weight"), *rs = g->find(p + "ffn_gate_inp_shexp.weight");
    const size_t esz = L->router_dtype == MOEXB_F32 ? 4 : 2;
    std::vector<uint8_t> rows((size_t)E * EH * esz);
    if (rt && rt->n_dims == 2 && rt->ne[0] == EH && rt->ne[1] == E && rt->data && router_rows_to(rt->type, rt->data, E * EH, L->router_dtype, rows.data())) {
        CUDA_TRY(cudaMemcpy(L->router, rows.data(), rows.size(), cudaMemcpyHostToDevice));
        got |= 4;
    }
    if (rs && rs->ne[0] == EH && rs->nbytes == rs->row_bytes && rs->data && router_rows_to(rs->type, rs->data, EH, L->router_dtype, rows.data())) {
        CUDA_TRY(cudaMemcpy(static_cast<uint8_t*>(L->router) + (size_t)E * EH * esz, rows.data(), EH * esz, cudaMemcpyHostToDevice));
        got |= 8;
    }
    if (loaded) *loaded = got;
    return MOEXB_OK;
}

// gg_dequant (gguf.h:85-255) for the block types this library reads, on the host: n values (a multiple of the block size).
int moexb_gguf_dequant_host(int ggml_type, const uint8_t* src_host, long long n, float* y_host) {
    REQUIRE(src_host && y_host && n > 0, "gguf_dequant_host: bad argument");
    if (!gq_dequant((uint32_t)ggml_type, src_host, n, y_host))
        return fail(MOEXB_ERR_UNSUPPORTED, "gguf_dequant_host: ggml type %d is not readable here, or n=%lld is not a multiple of its block size", ggml_type, n);
    return MOEXB_OK;
}

// gg_zp_row (gguf.h:302-330) on the host: one row of `cols` weights (a multiple of 256) of a GGUF tensor into the zero-point
// form - nibble bytes qb[cols / 2], [sc, mn] cs[cols / 32 * 2], (d, dm) fp16 bits sup[cols / 256 * 2].
int moexb_gguf_row_to_zp(int ggml_type, const uint8_t* src_host, int cols, uint8_t* qb, uint8_t* cs, uint16_t* sup) {
    REQUIRE(src_host && qb && cs && sup, "gguf_row_to_zp: null pointer");
    REQUIRE(cols > 0 && cols % 256 == 0, "gguf_row_to_zp: cols=%d must be a positive multiple of 256", cols);
    if (ggml_type == (int)GQ_Q4_K) {
        for (int b = 0; b < cols / 256; b++) q4k_block_to_zp(src_host + (size_t)b * 144, qb + b * 128, cs + b * 16, reinterpret_cast<uint8_t*>(sup + 2 * b));
        return MOEXB_OK;
    }
    std::vector<float> w(cols);
    if (!gq_dequant((uint32_t)ggml_type, src_host, cols, w.data())) return fail(MOEXB_ERR_UNSUPPORTED, "gguf_row_to_zp: ggml type %d is not readable here", ggml_type);
    zp_row_from_values(w.data(), cols, qb, cs, sup);
    return MOEXB_OK;
}

// ---- safetensors container ingest ----------------------------------------------------------------------------------------

int moexb_st_open(const char* path, moexb_st** out) {
    REQUIRE(path && out, "st_open: null pointer");
    std::string err;
    moexb_st* s = st_open(path, err);
    if (!s) return fail(MOEXB_ERR_ARG, "st_open: %s", err.c_str());
    *out = s;
    return MOEXB_OK;
}

int moexb_st_close(moexb_st* s) {
    delete s;
    return MOEXB_OK;
}

int moexb_st_tensor_count(const moexb_st* s) { return s ? (int)s->tensors.size() : 0; }

const char* moexb_st_tensor_name(const moexb_st* s, int i) {
    return s && i >= 0 && i < (int)s->tensors.size() ? s->tensors[i].name.c_str() : nullptr;
}

int moexb_st_tensor(const moexb_st* s, const char* name, char* dtype, int* n_dims, long long* shape, const void** data, long long* nbytes) {
    REQUIRE(s && name, "st_tensor: null pointer");
    const StTensorInfo* t = s->find(name);
    if (!t) return fail(MOEXB_ERR_ARG, "missing tensor %s", name);
    if (dtype) { strncpy(dtype, t->dtype.c_str(), 7); dtype[7] = 0; }
    if (n_dims) *n_dims = (int)std::min<size_t>(t->shape.size(), 8);
    if (shape) for (size_t d = 0; d < t->shape.size() && d < 8; d++) shape[d] = t->shape[d];
    if (data) *data = t->data;
    if (nbytes) *nbytes = t->nbytes;
    return MOEXB_OK;
}

int moexb_layer_load_st(moexb_layer* L, const moexb_st* s, const char* prefix, int* loaded) {
    REQUIRE(L && s && prefix, "layer_load_st: null pointer");
    if (loaded) *loaded = 0;
    moexb_ctx* c = L->ctx;
    CUDA_TRY(cudaSetDevice(c->device));
    const std::string p(prefix);
    const size_t eb = expert_bytes(L->fmt), sp = eb - Q_BYTES;  // scale part of the layer's format
    // the container's scale part: F32 group scales (symmetric) or the zero-point bytes; an fp16-scale layer takes F32
    // scales only when every one of them is an fp16 value, so that nothing is rounded on the way in
    const size_t sp_file = L->fmt == FMT_ZP ? expert_bytes(FMT_ZP) - Q_BYTES : expert_bytes(FMT_SYM_F32) - Q_BYTES;
    const char* want_dtype = L->fmt == FMT_ZP ? "U8" : "F32";
    std::vector<__half> narrow(L->fmt == FMT_SYM_F16 ? CHUNKS / 2 : 0);
    for (int i = 0; i < L->n_local; i += STAGING_BLOBS) {
        const int n = min(STAGING_BLOBS, L->n_local - i);
        for (int j = 0; j < n; j++) {
            const std::string ep = p + "mlp.experts." + std::to_string(L->first_local + i + j) + ".";
            const StTensorInfo *q = s->find(ep + "merged_weight"), *qs = s->find(ep + "qs");
            if (!q || !qs) return fail(MOEXB_ERR_ARG, "missing tensor %s%s", ep.c_str(), q ? "qs" : "merged_weight");
            if ((size_t)q->nbytes != Q_BYTES) return fail(MOEXB_ERR_ARG, "%smerged_weight has %lld bytes, not the %zu of this expert shape", ep.c_str(), q->nbytes, (size_t)Q_BYTES);
            if ((size_t)qs->nbytes != sp_file || qs->dtype != want_dtype)
                return fail(MOEXB_ERR_UNSUPPORTED, "%sqs (%s, %lld bytes) is not the scale part of this layer's expert format (%s, %zu bytes)",
                            ep.c_str(), qs->dtype.c_str(), qs->nbytes, want_dtype, sp_file);
            uint8_t* dst = c->staging + (size_t)j * eb;
            CUDA_TRY(cudaMemcpyAsync(dst, q->data, Q_BYTES, cudaMemcpyHostToDevice, nullptr));
            if (L->fmt == FMT_SYM_F16) {
                for (size_t k = 0; k < CHUNKS / 2; k++) {
                    float f;
                    memcpy(&f, qs->data + 4 * k, 4);
                    narrow[k] = __float2half_rn(f);
                    if (!(__half2float(narrow[k]) == f))
                        return fail(MOEXB_ERR_UNSUPPORTED, "%sqs: scale %zu (%.9g) is not an fp16 value; load this container into a MOEXB_FMT_SYM_F32 layer", ep.c_str(), k, f);
                }
                CUDA_TRY(cudaMemcpy(dst + Q_BYTES, narrow.data(), sp, cudaMemcpyHostToDevice));  // synchronous: narrow is reused
            } else {
                CUDA_TRY(cudaMemcpyAsync(dst + Q_BYTES, qs->data, sp, cudaMemcpyHostToDevice, nullptr));
            }
        }
        const int rc = to_layer_layout(L, c->staging, L->image + (size_t)i * eb, n, nullptr);
        if (rc != MOEXB_OK) return rc;
        CUDA_TRY(cudaStreamSynchronize(nullptr));
    }
    int got = L->n_local ? 1 : 0;
    for (int i = 0; i < L->n_local; i++) L->loaded[L->first_local + i] = 1;
    // router rows (mlp.gate.weight [E][H]) and the shared expert's gate vector (mlp.shared_expert_gate.weight [1][H])
    const size_t esz = L->router_dtype == MOEXB_F32 ? 4 : 2;
    const long long E = L->n_routed;
    std::vector<uint8_t> rows((size_t)E * EH * esz);
    auto ggml_of = [](const std::string& d) { return d == "F32" ? (int)GGML_F32 : d == "F16" ? (int)GGML_F16 : d == "BF16" ? (int)GGML_BF16 : -1; };
    auto convert = [&](const StTensorInfo* t, long long n) {
        const int ty = t ? ggml_of(t->dtype) : -1;
        if (ty < 0 || t->nbytes != n * (ty == (int)GGML_F32 ? 4 : 2)) return false;
        return router_rows_to((uint32_t)ty, t->data, n, L->router_dtype, rows.data());
    };
    if (convert(s->find(p + "mlp.gate.weight"), E * EH)) {
        CUDA_TRY(cudaMemcpy(L->router, rows.data(), rows.size(), cudaMemcpyHostToDevice));
        got |= 4;
    }
    if (convert(s->find(p + "mlp.shared_expert_gate.weight"), EH)) {
        CUDA_TRY(cudaMemcpy(static_cast<uint8_t*>(L->router) + (size_t)E * EH * esz, rows.data(), EH * esz, cudaMemcpyHostToDevice));
        got |= 8;
    }
    if (loaded) *loaded = got;
    return MOEXB_OK;
}

}  // extern "C"

// ---- streaming (tensor-core) expert path ------------------------------------------------------------------------------------

template <int FMT, bool DOWN>
static int stream_launch_one(moexb_ctx* c, const StreamArgs& a, void* stream) {
    constexpr int NW = 4, STAGES = FMT == FMT_SYM_F16 ? 4 : 3;
    constexpr int SMEM = st_smem_bytes<FMT, DOWN, NW, STAGES>();
    static PerDeviceOnce once;
    const cudaError_t attr_err = once.run([] { return cudaFuncSetAttribute(stream_k<FMT, DOWN, NW, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); });
    if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "stream kernel shared memory: %s", cudaGetErrorString(attr_err));
    PROF(c, DOWN ? MOEXB_PROF_DOWN : MOEXB_PROF_GATE_UP, stream);
    stream_k<FMT, DOWN, NW, STAGES><<<2 * c->sms, (NW + 1) * 32, SMEM, S(stream)>>>(a);
    LAUNCHED(DOWN ? "stream_down" : "stream_gate_up");
    return MOEXB_OK;
}

// gate/up then down over the sub-items already planned in the context (subs, nsub);
// xs = the split activations [token][2][H]; act32 optional.
static int stream_experts(moexb_ctx* c, int fmt, const moexb_pair* pairs, float* act32, float* ypair, void* stream) {
    StreamArgs a{c->subs, c->nsub, pairs, reinterpret_cast<const __nv_bfloat16*>(c->xs), act32, reinterpret_cast<__nv_bfloat16*>(c->act_split), ypair, c->err};
    return by_fmt(fmt, [&]<int FMT>() {
        int rc = stream_launch_one<FMT, false>(c, a, stream);
        if (rc != MOEXB_OK) return rc;
        StreamArgs d = a;
        d.xs = reinterpret_cast<const __nv_bfloat16*>(c->act_split);
        return stream_launch_one<FMT, true>(c, d, stream);
    });
}

template <int FMT, bool DOWN, int NW, int D, int NB = 1, int CPS = 2, bool PLAN = false>
static int tiled_launch_cfg(moexb_ctx* c, const TiledArgs& a, const PlanArgs& pa, void* stream) {
    constexpr int SMEM = tl_smem_bytes<FMT, DOWN, NW, D, NB, PLAN>();
    static_assert(SMEM * CPS <= 227 * 1024, "shared memory of the resident CTAs");
    static PerDeviceOnce once;
    const cudaError_t attr_err = once.run([] { return cudaFuncSetAttribute(stream_tiled_k<FMT, DOWN, NW, D, NB, CPS, PLAN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); });
    if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "tiled stream kernel shared memory: %s", cudaGetErrorString(attr_err));
    PROF(c, DOWN ? MOEXB_PROF_DOWN : MOEXB_PROF_GATE_UP, stream);
    CUDA_TRY(launch_dep(stream_tiled_k<FMT, DOWN, NW, D, NB, CPS, PLAN>, CPS * c->sms, NW * 32, SMEM, S(stream), a, pa));
    LAUNCHED(DOWN ? "stream_tiled_down" : "stream_tiled_gate_up");
    return MOEXB_OK;
}

// Two shapes of the same kernel, both two CTAs per SM: a few tokens leave only a handful of row tiles per SM, so CTAs of
// 4 warps with 4 slices in flight each spread them over every SM; from 8 tokens on there is work for 16 warps per SM
// (CTAs of 8 warps, 2 slices in flight each - the same bytes in flight, twice the issue slots in use).
// From 8 tokens on the symmetric formats also take sub-items of up to 8 pairs (two column blocks; tiled_maxp below): the
// gate/up columns of 8 pairs are 66 KB, so that kernel runs as one CTA of 16 warps per SM.
// plan: the gate/up kernel makes the work list itself (no planning launch before it).
template <int FMT, bool DOWN, bool PLAN = false>
static int tiled_launch_one(moexb_ctx* c, const TiledArgs& a, int T, void* stream, const PlanArgs& pa = PlanArgs{}) {
    static_assert(!PLAN || FMT == FMT_SYM_F16, "the in-kernel work list fits beside the ring of the fp16-scale format only");
    if (T < 8) return tiled_launch_cfg<FMT, DOWN, 4, 4, 1, 2, PLAN>(c, a, pa, stream);
    if (FMT == FMT_ZP || c->pairs_per_pass == 4) return tiled_launch_cfg<FMT, DOWN, 8, 2, 1, 2, PLAN>(c, a, pa, stream);
    if constexpr (FMT == FMT_ZP) return MOEXB_OK;
    else if constexpr (DOWN) return tiled_launch_cfg<FMT, DOWN, 8, 2, 2, 2, PLAN>(c, a, pa, stream);
    else return tiled_launch_cfg<FMT, DOWN, 16, 2, 2, 1, PLAN>(c, a, pa, stream);
}
// Pairs per sub-item that tiled_launch_one's kernels take.
static int tiled_maxp(const moexb_ctx* c, int fmt, int T) { return (T >= 8 && fmt != FMT_ZP) ? c->pairs_per_pass : 4; }
// Whether the gate/up kernel can make the work list of this batch itself (tiled.cuh: plan_in_cta).
// (fp16-scale format: with the wider slices of the other formats the list does not fit beside two CTAs' rings.)
// One token on one GPU needs no list (the routing kernel writes the nine one-pair sub-items itself); across GPUs the list is
// made in the kernel for any batch, because a planning launch would sit behind the wait for the peers.
static bool plan_in_kernel(const moexb_ctx* c, int fmt, int T, int K, int E, bool ep = false) {
    static const bool on = [] { const char* e = getenv("MOEXB_PLAN_IN_KERNEL"); return !(e && e[0] == '0'); }();
    return on && fmt == FMT_SYM_F16 && (T >= 2 || ep) && T <= PL_MAX_TOKENS && K <= PL_MAX_K && E <= PL_MAX_E;
}

// The same on blobs in the tiled layout (sub-item slots point into a tiled layer image). plan: null = the list is already
// in the context (subs, nsub, pairs); else the gate/up kernel makes it and leaves it there for the down kernel.
static int tiled_experts(moexb_ctx* c, int fmt, const moexb_pair* pairs, float* act32, float* ypair, int T, void* stream, const PlanArgs* plan = nullptr) {
    TiledArgs a{c->subs, c->nsub, pairs, c->xs, act32, c->act_split, ypair, c->err};
    return by_fmt(fmt, [&]<int FMT>() {
        int rc;
        if constexpr (FMT == FMT_SYM_F16) rc = plan ? tiled_launch_one<FMT, false, true>(c, a, T, stream, *plan) : tiled_launch_one<FMT, false>(c, a, T, stream);
        else rc = tiled_launch_one<FMT, false>(c, a, T, stream);
        if (rc != MOEXB_OK) return rc;
        TiledArgs d = a;
        d.xs = c->act_split;
        return tiled_launch_one<FMT, true>(c, d, T, stream);
    });
}

// ---- prefill: grouped GEMM on tcgen05 ----------------------------------------------------------------------------------------

template <int FMT, bool DOWN>
static int prefill_launch_one(moexb_ctx* c, const PrefillArgs& a, void* stream) {
    constexpr int SMEM = pf_smem_bytes<FMT, DOWN>();
    static PerDeviceOnce once;
    const cudaError_t attr_err = once.run([] { return cudaFuncSetAttribute(prefill_k<FMT, DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); });
    if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "prefill kernel shared memory: %s", cudaGetErrorString(attr_err));
    PROF(c, DOWN ? MOEXB_PROF_DOWN : MOEXB_PROF_GATE_UP, stream);
    prefill_k<FMT, DOWN><<<c->sms, PF_THREADS, SMEM, S(stream)>>>(a);
    LAUNCHED(DOWN ? "prefill_down" : "prefill_gate_up");
    return MOEXB_OK;
}

// Experts of a large batch on the tensor-core grouped GEMM: items/nitems = the grouped work list (tiled blobs), xf = the
// activations as fp32 [T][H]; parts = 1 when xf holds exact bf16 values, else 2.
static int prefill_experts(moexb_ctx* c, int fmt, const moexb_pair* pairs, const float* xf, int T, int parts, float* ypair, void* stream,
                           bool pre_split = false) {
    if (!pre_split) {   // pre_split: the context already holds the fp16 columns (expert parallelism: the token owners made them)
        PROF(c, MOEXB_PROF_OTHER, stream);
        const size_t n = (size_t)T * EH;
        split8_rows_k<<<(unsigned)((n + 255) / 256), 256, 0, S(stream)>>>(xf, c->xs, EH, parts, n);
        LAUNCHED("split8_rows");
    }
    // the planner left two tile lists in the context: subs (up to 128 / parts pairs: gate/up) and subs2 (up to 64 pairs: down,
    // whose act columns are always hi + lo)
    auto run = [&]<int FMT>() {
        PrefillArgs a{c->subs, c->nsub, pairs, c->xs, c->act_split, nullptr, ypair, c->err, parts};
        int rc = prefill_launch_one<FMT, false>(c, a, stream);
        if (rc != MOEXB_OK) return rc;
        PrefillArgs d = a;
        d.tiles = c->subs2; d.ntiles = c->nsub2; d.xs = c->act_split; d.parts = 2;
        return prefill_launch_one<FMT, true>(c, d, stream);
    };
    if (fmt == FMT_SYM_F16) return run.template operator()<FMT_SYM_F16>();
    return fail(MOEXB_ERR_UNSUPPORTED, "prefill kernels: format %d", fmt);
}

// f16: the consumer is the tiled kernel of a symmetric format (fp16 operands); otherwise bf16
static int split_launch(moexb_ctx* c, const float* x, int rows, bool f16, void* stream) {
    PROF(c, MOEXB_PROF_OTHER, stream);
    const size_t n = (size_t)rows * EH;
    if (f16) split_rows_k<true><<<(unsigned)((n + 255) / 256), 256, 0, S(stream)>>>(x, c->xs, EH, n);
    else split_rows_k<false><<<(unsigned)((n + 255) / 256), 256, 0, S(stream)>>>(x, c->xs, EH, n);
    LAUNCHED("split_rows");
    return MOEXB_OK;
}

extern "C" int moexb_pairs_forward_tc(moexb_ctx* c, int fmt, const moexb_pair_item* items, int n_items, const moexb_pair* pairs,
                                      const float* X, int T, int npairs, float* act, float* ypair, void* stream) {
    REQUIRE(c && items && pairs && X && ypair, "pairs_forward_tc: null pointer");
    REQUIRE(fmt_ok(fmt), "pairs_forward_tc: unknown expert format %d", fmt);
    REQUIRE(T > 0 && T <= c->max_tokens, "pairs_forward_tc: T=%d exceeds the context's max_tokens=%d", T, c->max_tokens);
    REQUIRE(npairs > 0 && npairs <= c->max_tokens * (c->top_k + 1), "pairs_forward_tc: npairs=%d exceeds the context's capacity %d", npairs, c->max_tokens * (c->top_k + 1));
    REQUIRE(n_items >= 0 && n_items <= c->max_experts + 1, "pairs_forward_tc: n_items=%d exceeds the context's capacity %d", n_items, c->max_experts + 1);
    if (n_items == 0) return MOEXB_OK;
    int rc = split_launch(c, X, T, false, stream);
    if (rc != MOEXB_OK) return rc;
    plan_subitems_k<<<1, 1024, 0, S(stream)>>>(items, nullptr, n_items, c->subs, c->nsub, ST_MAXP);
    LAUNCHED("plan_subitems");
    return stream_experts(c, fmt, pairs, act, ypair, stream);
}

extern "C" int moexb_ctx_set_fused_decode(moexb_ctx* c, int on) {
    REQUIRE(c, "ctx_set_fused_decode: null context");
    c->fused_decode = on != 0;
    return MOEXB_OK;
}

extern "C" int moexb_ctx_set_pairs_per_pass(moexb_ctx* c, int pairs) {
    REQUIRE(c && (pairs == 4 || pairs == 8), "ctx_set_pairs_per_pass: 4 or 8");
    c->pairs_per_pass = pairs;
    return MOEXB_OK;
}

extern "C" int moexb_ctx_set_prefill_min_tokens(moexb_ctx* c, int tokens) {
    REQUIRE(c && tokens >= 1, "ctx_set_prefill_min_tokens: bad argument");
    c->prefill_min_tokens = tokens;
    return MOEXB_OK;
}

extern "C" int moexb_ctx_set_path(moexb_ctx* c, int path) {
    REQUIRE(c && (path == 0 || path == 1), "ctx_set_path: path must be 0 (streaming) or 1 (fp32 SIMT)");
    c->path = path;
    return MOEXB_OK;
}

// Waits for the device and returns the error word of the streaming kernels (0 = none; 1 / 2 = a consumer / the producer
// gave up waiting on a pipeline barrier), clearing it.
extern "C" int moexb_ctx_status(moexb_ctx* c, int* status) {
    REQUIRE(c && status, "ctx_status: null pointer");
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemcpy(status, c->err, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status) CUDA_TRY(cudaMemset(c->err, 0, sizeof(int)));
    return MOEXB_OK;
}

// Makes one bounded device-side wait run out on purpose and reports what the kernels' error word then holds.
// which = 0: the mbarrier wait of the streaming / grouped-GEMM pipelines (a barrier that expects bytes nobody sends);
// which = 1: the grid barrier of the one-token stack kernel (one CTA, two arrivals expected); which = 2: the wait of the
// expert-parallel kernels for a flag that another GPU raises (nobody raises it). All with `polls` polls instead of the
// production limits. Nothing faults or hangs: the kernel returns, the context stays usable.
extern "C" int moexb_ctx_selftest_timeout(moexb_ctx* c, int which, int polls, int* status) {
    REQUIRE(c && status, "ctx_selftest_timeout: null pointer");
    REQUIRE(which >= 0 && which <= 2 && polls > 0 && polls <= (1 << 20), "ctx_selftest_timeout: which=%d polls=%d", which, polls);
    CUDA_TRY(cudaSetDevice(c->device));
    CUDA_TRY(cudaMemset(c->nsub, 0, 2 * sizeof(int)));   // scratch of the self-test: [0] result of the wait
    unsigned* sync = reinterpret_cast<unsigned*>(c->counts);       // scratch: barrier counter and abort flag
    CUDA_TRY(cudaMemset(sync, 0, 2 * sizeof(unsigned)));
    if (which == 0) selftest_mbar_timeout_k<<<1, 32>>>(c->err, ST_ERR_FULL_WAIT, polls, c->nsub);
    else if (which == 1) selftest_grid_barrier_timeout_k<<<1, 32>>>(sync, c->err, polls, c->nsub);
    else selftest_ep_wait_timeout_k<<<1, 32>>>(sync, c->err, polls, c->nsub);
    LAUNCHED("selftest_timeout");
    return moexb_ctx_status(c, status);
}

extern "C" {

// Router logits (column n_routed = the shared expert's gate logit) and top-K for T tokens, into the context workspace.
// decode: also emit the K+1 one-pair sub-items of a single token (slots, weights, sub-items, pairs).
}  // extern "C"
// Router logits (into the context, [T][E + 1]) and the top-K selection in one launch; decode: also the K + 1 one-pair
// sub-items of a single token.
struct RouteEp { const EpDevice* dev; int row_bytes; unsigned phase; const unsigned* step; };
template <typename WT>
static int route_launch(moexb_ctx* c, moexb_layer* L, const float* xf, int T, int K, void* stream, bool decode, int tok0 = 0, const RouteEp* rep = nullptr) {
    // tok0: the T rows at xf are tokens tok0.. of the batch - their logits, ids and weights go to those rows of the workspace
    const int E = L->n_routed;
    const WT* W = static_cast<const WT*>(L->router);
    float* logits = c->logits + (size_t)tok0 * (E + 1);
    TopkOut o{c->idx + (size_t)tok0 * K, c->w + (size_t)tok0 * K, L->slot_table, decode ? c->slots : nullptr, decode ? c->wts : nullptr,
              decode ? c->subs : nullptr, decode ? c->pairs : nullptr, decode ? c->nsub : nullptr};
    if (rep) { o.ep = rep->dev; o.ep_row_bytes = rep->row_bytes; o.ep_phase = rep->phase; o.ep_step = rep->step; }
    auto run = [&]<int NJ>() -> int {
        // expert parallelism with few own tokens: one token per block row, so that each token's selection and dispatch stores are
        // done by a block of their own instead of one block sending a whole tile of 8
        if (T < 8 || (rep && T <= 16)) {
            constexpr int WARPS = 8;
            CUDA_TRY(launch_dep(route_gemv_k<WT, WARPS, NJ>, dim3((E + 1 + WARPS - 1) / WARPS, T), WARPS * 32, 0, S(stream), W, xf, logits, EH, E, K, 1, c->route_done, o));
        } else {
            // 16 outputs per block spread a small batch over more SMs; a prefill chunk has blocks to spare and re-reads
            // the router weights less with 32 outputs per block
            auto gemm = [&]<int TO, int TR>() -> int {
                constexpr int WARPS = 8, SMEM = TR * EH * (int)sizeof(float);
                static PerDeviceOnce once;
                const cudaError_t attr_err = once.run([] { return cudaFuncSetAttribute(route_gemm_k<WT, WARPS, TO, TR, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); });
                if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "router kernel shared memory: %s", cudaGetErrorString(attr_err));
                CUDA_TRY(launch_dep(route_gemm_k<WT, WARPS, TO, TR, NJ>, dim3((E + 1 + WARPS * TO - 1) / (WARPS * TO), (T + TR - 1) / TR), WARPS * 32, SMEM, S(stream),
                                    W, xf, logits, EH, E, K, 1, T, c->route_done, o));
                return MOEXB_OK;
            };
            // a small batch: 16 outputs x 8 tokens per block, to reach every SM; a prefill chunk goes to the register-tiled
            // kernel (32 tokens x 16 outputs per block, FMA-bound)
            auto gemm2 = [&]() -> int {
                constexpr int SMEM = 2 * rg2_stage_bytes<WT>();
                static PerDeviceOnce once;
                const cudaError_t attr_err = once.run([] { return cudaFuncSetAttribute(route_gemm2_k<WT, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); });
                if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "router kernel shared memory: %s", cudaGetErrorString(attr_err));
                CUDA_TRY(launch_dep(route_gemm2_k<WT, NJ>, dim3((E + 1 + RG2_TN - 1) / RG2_TN, (T + RG2_TM - 1) / RG2_TM), 256, SMEM, S(stream),
                                    W, xf, logits, E, K, 1, T, c->route_done, o));
                return MOEXB_OK;
            };
            const int rc = T >= 256 ? gemm2() : gemm.template operator()<2, 8>();
            if (rc != MOEXB_OK) return rc;
        }
        LAUNCHED("route");
        return MOEXB_OK;
    };
    return E <= 256 ? run.template operator()<8>() : run.template operator()<32>();
}

extern "C" {
static int layer_route(moexb_ctx* c, moexb_layer* L, const float* xf, int T, int K, void* stream, bool decode, int tok0 = 0, const RouteEp* rep = nullptr) {
    PROF(c, MOEXB_PROF_ROUTER, stream);
    return L->router_dtype == MOEXB_F32 ? route_launch<float>(c, L, xf, T, K, stream, decode, tok0, rep) : route_launch<__half>(c, L, xf, T, K, stream, decode, tok0, rep);
}

// One layer. xin: the layer input as f32 [T][H]. flags as moexb_layer_forward. pre_normed: the context already holds
// rmsnorm(xin) and its bf16 split (left there by the previous layer of a stack); next_norm: leave rmsnorm(out) and its
// split in the context for the next layer.
static int layer_impl(moexb_ctx* c, moexb_layer* L, const float* xin, int T, int K, float* out, int* idx_out, float* w_out, int flags,
                      void* stream, bool pre_normed, bool next_norm, int sh0 = 0, int sh1 = -1, bool x_bf16 = false) {
    if (sh1 < 0) sh1 = T;
    const bool shared = !(flags & 1) && sh1 > sh0, block = flags & 2, partial = flags & 4;
    const bool all_local = L->n_local == L->n_routed;
    const int E = L->n_routed, ld = E + 1;
    cudaStream_t st = S(stream);
    const bool tiled = L->layout == MOEXB_LAYOUT_TILED;
    const bool streaming = tiled || c->path == 0;
    // large batches of symmetric-format experts go to the tcgen05 grouped GEMM (bf16 operands); the rest to the streaming kernels
    const bool prefill = tiled && L->fmt == FMT_SYM_F16 && T >= c->prefill_min_tokens;
    const bool f16 = tiled && L->fmt != FMT_ZP && !prefill;  // element type of the split activations the streaming kernels read
    const float* xf = xin;  // what the router and the experts see
    if (block) {
        xf = c->xn;
        if (!pre_normed) {
            PROF(c, MOEXB_PROF_OTHER, stream);
            if (f16) rmsnorm_split_k<true><<<T, 256, 0, st>>>(xin, c->xn, c->xs, 1e-6f);
            else rmsnorm_split_k<false><<<T, 256, 0, st>>>(xin, c->xn, c->xs, 1e-6f);
            LAUNCHED("rmsnorm_split");
        }
    } else if (streaming && !prefill) {
        const int rc = split_launch(c, xf, T, f16, stream);
        if (rc != MOEXB_OK) return rc;
    }
    const bool decode = T == 1 && all_local && shared && !partial;
    int rc = layer_route(c, L, xf, T, K, stream, decode);
    if (rc != MOEXB_OK) return rc;
    int ranks = K;                  // rows of ypair per token that the final reduction adds
    const float* extra = nullptr;   // + the shared expert's rows
    if (partial && !streaming) return fail(MOEXB_ERR_UNSUPPORTED, "layer_forward: partial outputs need the streaming kernels");
    if (decode && !streaming) {
        // one token on the fp32 SIMT kernels: the K routed experts and the shared expert as K+1 decode experts
        rc = decode_launch(c, L->fmt, c->slots, c->wts, K + 1, xf, c->act, block ? c->moe : out, stream, nullptr);
        if (rc != MOEXB_OK) return rc;
        if (block) {
            PROF(c, MOEXB_PROF_COMBINE, stream);
            residual_add_k<<<(unsigned)((EH / 4 + 255) / 256), 256, 0, st>>>(xin, c->moe, out, EH);
            LAUNCHED("residual_add");
            if (next_norm) { rmsnorm_split_k<false><<<1, 256, 0, st>>>(out, c->xn, c->xs, 1e-6f); LAUNCHED("rmsnorm_split"); }
        }
        ranks = 0;
    } else if (decode) {
        rc = tiled ? tiled_experts(c, L->fmt, c->pairs, nullptr, c->ypair, T, stream) : stream_experts(c, L->fmt, c->pairs, nullptr, c->ypair, stream);
        if (rc != MOEXB_OK) return rc;
        ranks = K + 1;
    } else {
        const int parts = (x_bf16 && !block) ? 1 : 2;
        const int maxp = prefill ? PF_NMAX / parts : (tiled ? tiled_maxp(c, L->fmt, T) : ST_MAXP);
        const bool in_kernel = tiled && !prefill && plan_in_kernel(c, L->fmt, T, K, E);
        const PlanArgs plan{c->idx, c->w, T, K, E, L->slot_table, L->first_local, L->first_local + L->n_local, shared ? c->logits + E : nullptr, ld, sh0, sh1, maxp, c->subs, c->pairs, c->nsub, nullptr, nullptr, 0u};
        if (!in_kernel) {
            PROF(c, MOEXB_PROF_GROUP, stream);
            // room in shared memory for the routed pairs (12 bytes each), so that the list is written out in full lines
            constexpr int PLAN_STAGE_MAX = 196608;
            static PerDeviceOnce plan_once;
            const cudaError_t plan_attr = plan_once.run([] { return cudaFuncSetAttribute(group_plan1_k<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PLAN_STAGE_MAX); });
            const int stage_pairs = plan_attr == cudaSuccess && (size_t)T * K * 12 <= PLAN_STAGE_MAX ? T * K : 0;
            CUDA_TRY(launch_dep(group_plan1_k<false>, 1, 1024, (size_t)stage_pairs * 12, st, c->idx, c->w, T, K, E, L->slot_table, c->items, c->pairs, c->nitems, c->subs, c->nsub, maxp,
                                prefill ? c->subs2 : nullptr, c->nsub2, PF_NMAX / 2, shared ? c->logits + E : nullptr, ld, sh0, sh1, stage_pairs,
                                (const unsigned*)nullptr, (const unsigned*)nullptr, 0u, 0, 0, (int*)nullptr));
            LAUNCHED("group_plan");
            // pairs of experts that are not held here are never written: the SIMT reduction path needs zeros there, the fused
            // reduction skips them by expert id
            if (!all_local && !streaming) CUDA_TRY(cudaMemsetAsync(c->ypair, 0, (size_t)T * K * EH * sizeof(float), st));
        }
        rc = prefill ? prefill_experts(c, L->fmt, c->pairs, xf, T, parts, c->ypair, stream)
           : tiled ? tiled_experts(c, L->fmt, c->pairs, nullptr, c->ypair, T, stream, in_kernel ? &plan : nullptr)
           : streaming ? stream_experts(c, L->fmt, c->pairs, nullptr, c->ypair, stream)
                       : pairs_launch(c, L->fmt, c->items, c->nitems, min(E, T * K) + 1, c->pairs, xf, c->act, c->ypair, stream);
        if (rc != MOEXB_OK) return rc;
        if (shared) extra = c->ypair + (size_t)T * K * EH;
    }
    if (ranks) {
        PROF(c, MOEXB_PROF_COMBINE, stream);
        const float* xres = (block && !partial) ? xin : nullptr;
        float* xn_next = next_norm ? c->xn : nullptr;
        const int* held = (!all_local && ranks == K) ? c->idx : nullptr;
        if (f16) CUDA_TRY(launch_dep(reduce_residual_norm_k<true>, T, 256, 0, st, c->ypair, extra, xres, out, ranks, xn_next, c->xs, 1e-6f, sh0, sh1, held, L->first_local, L->first_local + L->n_local));
        else CUDA_TRY(launch_dep(reduce_residual_norm_k<false>, T, 256, 0, st, c->ypair, extra, xres, out, ranks, xn_next, c->xs, 1e-6f, sh0, sh1, held, L->first_local, L->first_local + L->n_local));
        LAUNCHED("reduce_residual_norm");
    }
    if (idx_out) CUDA_TRY(cudaMemcpyAsync(idx_out, c->idx, (size_t)T * K * sizeof(int), cudaMemcpyDeviceToDevice, st));
    if (w_out) CUDA_TRY(cudaMemcpyAsync(w_out, c->w, (size_t)T * K * sizeof(float), cudaMemcpyDeviceToDevice, st));
    return MOEXB_OK;
}

// The layer input as f32: bf16 inputs are widened (exactly) into the context.
static int layer_input(moexb_ctx* c, const void* X, int x_dtype, int T, void* stream, const float** xin) {
    if (x_dtype == MOEXB_BF16) {
        PROF(c, MOEXB_PROF_OTHER, stream);
        const size_t n = (size_t)T * EH;
        bf16_to_f32_k<<<(unsigned)((n / 2 + 255) / 256), 256, 0, S(stream)>>>(static_cast<const __nv_bfloat16*>(X), c->xf, n);
        LAUNCHED("bf16_to_f32");
        *xin = c->xf;
    } else *xin = static_cast<const float*>(X);
    return MOEXB_OK;
}

int moexb_layer_forward(moexb_ctx* c, moexb_layer* L, const void* X, int x_dtype, int T, int K, float* out, int* idx_out,
                        float* w_out, int flags, void* stream) {
    REQUIRE(c && L && X && out, "layer_forward: null pointer");
    REQUIRE(L->ctx == c, "layer_forward: layer belongs to another context");
    REQUIRE(T > 0 && T <= c->max_tokens, "layer_forward: T=%d exceeds the context's max_tokens=%d", T, c->max_tokens);
    REQUIRE(K > 0 && K <= c->top_k, "layer_forward: K=%d exceeds the context's top_k=%d", K, c->top_k);
    REQUIRE(x_dtype == MOEXB_F32 || x_dtype == MOEXB_BF16, "layer_forward: x_dtype=%d", x_dtype);
    REQUIRE((flags & 1) || L->loaded[L->n_routed], "layer_forward: the shared expert of this layer was never loaded (upload it, or pass flags bit 0 to leave it out)");
    const float* xin;
    int rc = layer_input(c, X, x_dtype, T, stream, &xin);
    if (rc != MOEXB_OK) return rc;
    return layer_impl(c, L, xin, T, K, out, idx_out, w_out, flags, stream, false, false, 0, -1, x_dtype == MOEXB_BF16);
}

int moexb_layer_forward_ep(moexb_ctx* c, moexb_layer* L, const void* X, int x_dtype, int T, int K, float* out, int* idx_out,
                           float* w_out, int shared_t0, int shared_t1, int pre_normed, void* stream) {
    REQUIRE(c && L && X && out, "layer_forward_ep: null pointer");
    REQUIRE(L->ctx == c, "layer_forward_ep: layer belongs to another context");
    REQUIRE(T > 0 && T <= c->max_tokens, "layer_forward_ep: T=%d exceeds the context's max_tokens=%d", T, c->max_tokens);
    REQUIRE(K > 0 && K <= c->top_k, "layer_forward_ep: K=%d exceeds the context's top_k=%d", K, c->top_k);
    REQUIRE(x_dtype == MOEXB_F32 || x_dtype == MOEXB_BF16, "layer_forward_ep: x_dtype=%d", x_dtype);
    REQUIRE(shared_t0 >= 0 && shared_t0 <= shared_t1 && shared_t1 <= T, "layer_forward_ep: shared token range [%d, %d) outside 0..%d", shared_t0, shared_t1, T);
    REQUIRE(shared_t0 == shared_t1 || L->loaded[L->n_routed], "layer_forward_ep: the shared expert of this layer was never loaded");
    const float* xin;
    int rc = layer_input(c, X, x_dtype, T, stream, &xin);
    if (rc != MOEXB_OK) return rc;
    return layer_impl(c, L, xin, T, K, out, idx_out, w_out, 2 | 4, stream, pre_normed != 0, false, shared_t0, shared_t1);
}

int moexb_ep_residual_norm(moexb_ctx* c, moexb_layer* next, const float* x, const float* total, float* out, int T, void* stream) {
    REQUIRE(c && x && total && out, "ep_residual_norm: null pointer");
    REQUIRE(T > 0 && T <= c->max_tokens, "ep_residual_norm: T=%d exceeds the context's max_tokens=%d", T, c->max_tokens);
    const bool f16 = next && next->layout == MOEXB_LAYOUT_TILED && next->fmt != FMT_ZP;
    float* xn = next ? c->xn : nullptr;
    PROF(c, MOEXB_PROF_COMBINE, stream);
    const float* no_extra = nullptr; const int* no_idx = nullptr;
    if (f16) CUDA_TRY(launch_dep(reduce_residual_norm_k<true>, T, 256, 0, S(stream), total, no_extra, x, out, 1, xn, c->xs, 1e-6f, 0, 0, no_idx, 0, 0));
    else CUDA_TRY(launch_dep(reduce_residual_norm_k<false>, T, 256, 0, S(stream), total, no_extra, x, out, 1, xn, c->xs, 1e-6f, 0, 0, no_idx, 0, 0));
    LAUNCHED("ep_residual_norm");
    return MOEXB_OK;
}

// ---- stack of layers as one CUDA graph ----------------------------------------------------------------------------------

struct moexb_stack {
    moexb_ctx* ctx = nullptr;
    int T = 0, K = 0, x_dtype = 0, n_layers = 0, kernels = 0;
    int out_rows = 0;            // rows of the result: T, or the own tokens of an expert-parallel rank
    void* x_in = nullptr;        // [T][H] of x_dtype
    float* buf[2] = {nullptr, nullptr};
    float* result = nullptr;     // = buf[(n_layers - 1) & 1]
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaStream_t cap = nullptr;
    // one-token residual stacks: a single cooperative launch instead of a graph
    bool fused = false;
    DecodeLayer* dlayers = nullptr;   // device
    unsigned* dsync = nullptr;        // device: barrier counter, abort flag
    int fmt = 0, router_dtype = 0, n_routed = 0;
};

int moexb_stack_destroy(moexb_stack* s) {
    if (!s) return MOEXB_OK;
    if (s->exec) cudaGraphExecDestroy(s->exec);
    if (s->graph) cudaGraphDestroy(s->graph);
    if (s->cap) cudaStreamDestroy(s->cap);
    cudaFree(s->x_in); cudaFree(s->buf[0]); cudaFree(s->buf[1]); cudaFree(s->dlayers); cudaFree(s->dsync);
    delete s;
    return MOEXB_OK;
}

}  // extern "C"
template <int FMT, typename WT, bool XBF>
static int decode_stack_launch(moexb_stack* s, void* stream) {
    moexb_ctx* c = s->ctx;
    constexpr int SMEM = ds_smem_bytes<FMT>();
    static PerDeviceOnce once;
    const cudaError_t attr_err = once.run([] {
        cudaError_t e = cudaFuncSetAttribute(decode_stack_k<FMT, WT, XBF>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        int per_sm = 0;
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_k<FMT, WT, XBF>, DS_THREADS, SMEM);
        if (e == cudaSuccess && per_sm < 1) e = cudaErrorLaunchOutOfResources;   // the persistent CTA does not fit an SM of this device
        return e;
    });
    if (attr_err != cudaSuccess) return fail(MOEXB_ERR_CUDA, "decode stack kernel: %s", cudaGetErrorString(attr_err));
    CUDA_TRY(cudaMemsetAsync(s->dsync, 0, 2 * sizeof(unsigned), S(stream)));
    DecodeStackArgs a{s->dlayers, s->n_layers, s->n_routed, s->K, s->x_in, s->buf[0], c->logits, c->act_split, c->ypair, c->wts, nullptr, nullptr, s->dsync, c->err};
    void* args[] = {&a};
    // cooperative: every CTA is resident, which the grid barrier inside relies on
    CUDA_TRY(cudaLaunchCooperativeKernel((void*)decode_stack_k<FMT, WT, XBF>, dim3(c->sms), dim3(DS_THREADS), args, SMEM, S(stream)));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return MOEXB_OK;
}
static int decode_stack_run(moexb_stack* s, void* stream) {
    auto by_x = [&]<int FMT, typename WT>() {
        return s->x_dtype == MOEXB_BF16 ? decode_stack_launch<FMT, WT, true>(s, stream) : decode_stack_launch<FMT, WT, false>(s, stream);
    };
    auto by_w = [&]<int FMT>() {
        return s->router_dtype == MOEXB_F32 ? by_x.template operator()<FMT, float>() : by_x.template operator()<FMT, __half>();
    };
    return s->fmt == FMT_SYM_F16 ? by_w.template operator()<FMT_SYM_F16>() : s->fmt == FMT_ZP ? by_w.template operator()<FMT_ZP>() : by_w.template operator()<FMT_SYM_F32>();
}
extern "C" {

int moexb_stack_create(moexb_ctx* c, moexb_layer* const* layers, int n_layers, int T, int K, int x_dtype, int residual, moexb_stack** out) {
    REQUIRE(c && layers && out, "stack_create: null pointer");
    REQUIRE(n_layers > 0 && T > 0 && T <= c->max_tokens && K > 0 && K <= c->top_k, "stack_create: n_layers=%d T=%d K=%d", n_layers, T, K);
    REQUIRE(x_dtype == MOEXB_F32 || x_dtype == MOEXB_BF16, "stack_create: x_dtype=%d", x_dtype);
    REQUIRE(!c->profiling, "stack_create: switch profiling off before capturing a graph");
    for (int l = 0; l < n_layers; l++) {
        REQUIRE(layers[l] && layers[l]->ctx == c, "stack_create: layer %d is null or belongs to another context", l);
        REQUIRE(layers[l]->fmt == layers[0]->fmt && layers[l]->layout == layers[0]->layout, "stack_create: layer %d differs from layer 0 in format or layout", l);
        REQUIRE(layers[l]->loaded[layers[l]->n_routed], "stack_create: the shared expert of layer %d was never loaded", l);
    }
    CUDA_TRY(cudaSetDevice(c->device));
    moexb_stack* s = new (std::nothrow) moexb_stack;
    if (!s) return fail(MOEXB_ERR_NOMEM, "out of host memory");
    s->ctx = c; s->T = T; s->K = K; s->x_dtype = x_dtype; s->n_layers = n_layers; s->out_rows = T;
    const size_t n = (size_t)T * EH;
    cudaError_t e = cudaMalloc(&s->x_in, n * (x_dtype == MOEXB_BF16 ? 2 : 4));
    if (e == cudaSuccess) e = cudaMalloc((void**)&s->buf[0], n * 4);
    if (e == cudaSuccess) e = cudaMalloc((void**)&s->buf[1], n * 4);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->cap, cudaStreamNonBlocking);
    if (e != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_NOMEM, "stack_create: %s", cudaGetErrorString(e)); }
    // one token through residual blocks of resident symmetric-format experts: one cooperative launch for the whole stack
    // (a CTA of the cooperative kernel owns at most two router rows, so E + 1 <= 2 x SMs)
    bool fused = c->fused_decode && T == 1 && residual && K <= DS_MAXK && n_layers <= DS_MAXLAYERS && layers[0]->n_routed + 1 <= 2 * c->sms && layers[0]->layout == MOEXB_LAYOUT_TILED;
    for (int l = 0; l < n_layers && fused; l++)
        fused = layers[l]->n_local == layers[l]->n_routed && layers[l]->n_routed == layers[0]->n_routed && layers[l]->n_routed <= 256 &&
                layers[l]->n_routed % 32 == 0 && layers[l]->router_dtype == layers[0]->router_dtype;
    if (fused) {
        std::vector<DecodeLayer> h(n_layers);
        for (int l = 0; l < n_layers; l++) h[l] = {layers[l]->router, layers[l]->slot_table};
        e = cudaMalloc((void**)&s->dlayers, n_layers * sizeof(DecodeLayer));
        if (e == cudaSuccess) e = cudaMalloc((void**)&s->dsync, 2 * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemcpy(s->dlayers, h.data(), n_layers * sizeof(DecodeLayer), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_NOMEM, "stack_create: %s", cudaGetErrorString(e)); }
        s->fused = true; s->fmt = layers[0]->fmt; s->router_dtype = layers[0]->router_dtype; s->n_routed = layers[0]->n_routed;
        s->kernels = 1; s->result = s->buf[0];
        *out = s;
        return MOEXB_OK;
    }
    const long long before = g_launches.load();
    e = cudaStreamBeginCapture(s->cap, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_CUDA, "stack_create: begin capture: %s", cudaGetErrorString(e)); }
    const float* xin = nullptr;
    int rc = layer_input(c, s->x_in, x_dtype, T, s->cap, &xin);
    for (int l = 0; l < n_layers && rc == MOEXB_OK; l++) {
        // layer l leaves rmsnorm(x_{l+1}) and its split in the context, so layer l+1 starts at its router
        if (residual) rc = layer_impl(c, layers[l], xin, T, K, s->buf[l & 1], nullptr, nullptr, 2, s->cap, l > 0, l + 1 < n_layers);
        else rc = layer_impl(c, layers[l], xin, T, K, s->buf[l & 1], nullptr, nullptr, 0, s->cap, false, false, 0, -1, l == 0 && x_dtype == MOEXB_BF16);
        xin = s->buf[l & 1];
    }
    e = cudaStreamEndCapture(s->cap, &s->graph);
    s->kernels = (int)(g_launches.load() - before);
    g_launches.store(before);  // captured, not yet run
    if (rc != MOEXB_OK) { moexb_stack_destroy(s); return rc; }
    if (e == cudaSuccess) e = cudaGraphInstantiate(&s->exec, s->graph, 0);
    if (e != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_CUDA, "stack_create: graph: %s", cudaGetErrorString(e)); }
    s->result = s->buf[(n_layers - 1) & 1];
    *out = s;
    return MOEXB_OK;
}

int moexb_stack_kernel_count(moexb_stack* s) { return s ? s->kernels : 0; }

int moexb_stack_run(moexb_stack* s, const void* X, float* out, void* stream) {
    REQUIRE(s && X && out, "stack_run: null pointer");
    const size_t n = (size_t)s->T * EH;
    CUDA_TRY(cudaMemcpyAsync(s->x_in, X, n * (s->x_dtype == MOEXB_BF16 ? 2 : 4), cudaMemcpyDeviceToDevice, S(stream)));
    if (s->fused) { const int rc = decode_stack_run(s, stream); if (rc != MOEXB_OK) return rc; }
    else {
        CUDA_TRY(cudaGraphLaunch(s->exec, S(stream)));
        g_launches.fetch_add(s->kernels, std::memory_order_relaxed);
    }
    CUDA_TRY(cudaMemcpyAsync(out, s->result, (size_t)s->out_rows * EH * 4, cudaMemcpyDeviceToDevice, S(stream)));
    return MOEXB_OK;
}

int moexb_stack_run_host(moexb_stack* s, const void* X_host, float* out_host, void* stream) {
    REQUIRE(s && X_host && out_host, "stack_run_host: null pointer");
    const size_t n = (size_t)s->T * EH;
    CUDA_TRY(cudaMemcpyAsync(s->x_in, X_host, n * (s->x_dtype == MOEXB_BF16 ? 2 : 4), cudaMemcpyHostToDevice, S(stream)));
    if (s->fused) { const int rc = decode_stack_run(s, stream); if (rc != MOEXB_OK) return rc; }
    else {
        CUDA_TRY(cudaGraphLaunch(s->exec, S(stream)));
        g_launches.fetch_add(s->kernels, std::memory_order_relaxed);
    }
    CUDA_TRY(cudaMemcpyAsync(out_host, s->result, (size_t)s->out_rows * EH * 4, cudaMemcpyDeviceToHost, S(stream)));
    CUDA_TRY(cudaStreamSynchronize(S(stream)));
    return MOEXB_OK;
}

// ---- expert parallelism: token all-to-all over peer memory (ep.cuh) -----------------------------------------------------------

struct moexb_ep {
    moexb_ctx* ctx = nullptr;
    EpGeom g{};
    EpPeers peers{};
    EpLayout lay{};
    int n_routed = 0;
    float* x = nullptr;         // [n_own_max][H] residual rows of the own tokens
    unsigned* step = nullptr;   // device: steps begun so far
    EpDevice* dev = nullptr;    // device copy of geometry, peer pointers and layout (what the routing kernel's push reads)
    // what the context pointed at before its activations, ids and weights moved into the exchange buffer
    uint16_t* saved_xs = nullptr; int* saved_idx = nullptr; float* saved_w = nullptr;
    // host-side state of the layer in progress (set by dispatch, used by experts)
    bool prefill = false; int parts = 2;
};

size_t moexb_ep_buffer_bytes(int max_tokens, int top_k, int world) {
    if (max_tokens <= 0 || top_k <= 0 || world <= 0 || world > EP_MAX_RANKS) return 0;
    return ep_layout(max_tokens, top_k, world).bytes;
}

int moexb_ep_buffer_alloc(size_t bytes, void** ptr, unsigned char* handle) {
    REQUIRE(ptr && bytes > 0, "ep_buffer_alloc: bad argument");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(MOEXB_ERR_NOMEM, "ep_buffer_alloc: cudaMalloc of %zu bytes: %s", bytes, cudaGetErrorString(e));
    e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess && handle) {
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "an IPC handle is 64 bytes");
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, p);
        if (e == cudaSuccess) memcpy(handle, &h, 64);
    }
    if (e != cudaSuccess) { cudaFree(p); return fail(MOEXB_ERR_CUDA, "ep_buffer_alloc: %s", cudaGetErrorString(e)); }
    *ptr = p;
    return MOEXB_OK;
}

int moexb_ep_buffer_open(const unsigned char* handle, void** ptr) {
    REQUIRE(handle && ptr, "ep_buffer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return MOEXB_OK;
}

int moexb_ep_buffer_close(void* ptr) {
    if (ptr) CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return MOEXB_OK;
}

int moexb_ep_buffer_free(void* ptr) {
    if (ptr) CUDA_TRY(cudaFree(ptr));
    return MOEXB_OK;
}

int moexb_ep_create(moexb_ctx* c, int rank, int world, int T, int K, int n_routed, void* const* bufs, moexb_ep** out) {
    REQUIRE(c && bufs && out, "ep_create: null pointer");
    REQUIRE(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world, "ep_create: rank %d of %d (at most %d ranks)", rank, world, EP_MAX_RANKS);
    REQUIRE(T >= world && T <= c->max_tokens, "ep_create: T=%d must be at least the number of ranks (%d) and at most the context's max_tokens=%d", T, world, c->max_tokens);
    REQUIRE(K > 0 && K <= c->top_k, "ep_create: K=%d exceeds the context's top_k=%d", K, c->top_k);
    REQUIRE(n_routed >= world && n_routed <= c->max_experts, "ep_create: n_routed=%d", n_routed);
    for (int r = 0; r < world; r++) REQUIRE(bufs[r], "ep_create: the exchange buffer of rank %d is null", r);
    CUDA_TRY(cudaSetDevice(c->device));
    moexb_ep* e = new (std::nothrow) moexb_ep;
    if (!e) return fail(MOEXB_ERR_NOMEM, "out of host memory");
    e->ctx = c; e->n_routed = n_routed;
    e->g.rank = rank; e->g.world = world; e->g.T = T; e->g.K = K; e->g.n_own_max = (T + world - 1) / world;
    for (int r = 0; r <= EP_MAX_RANKS; r++) {
        const int rr = min(r, world);
        e->g.tok0[r] = rr * (T / world) + min(rr, T % world);
        e->g.exp0[r] = rr * (n_routed / world) + min(rr, n_routed % world);
    }
    for (int r = 0; r < EP_MAX_RANKS; r++) e->peers.base[r] = r < world ? static_cast<uint8_t*>(bufs[r]) : nullptr;
    e->lay = ep_layout(T, K, world);
    cudaError_t err = cudaMalloc((void**)&e->x, (size_t)e->g.n_own_max * EH * sizeof(float));
    if (err == cudaSuccess) err = cudaMalloc((void**)&e->step, sizeof(unsigned));
    if (err == cudaSuccess) err = cudaMalloc((void**)&e->dev, sizeof(EpDevice));
    if (err == cudaSuccess) err = cudaMemset(e->step, 0, sizeof(unsigned));
    if (err == cudaSuccess) { const EpDevice h{e->g, e->peers, e->lay}; err = cudaMemcpy(e->dev, &h, sizeof h, cudaMemcpyHostToDevice); }
    if (err != cudaSuccess) { cudaFree(e->x); cudaFree(e->step); cudaFree(e->dev); delete e; return fail(MOEXB_ERR_NOMEM, "ep_create: %s", cudaGetErrorString(err)); }
    // the context's activation columns, ids and weights now live in this rank's exchange buffer, where the peers write them
    uint8_t* local = e->peers.base[rank];
    e->saved_xs = c->xs; e->saved_idx = c->idx; e->saved_w = c->w;
    c->xs = reinterpret_cast<uint16_t*>(local + e->lay.xs);
    c->idx = reinterpret_cast<int*>(local + e->lay.idx);
    c->w = reinterpret_cast<float*>(local + e->lay.w);
    *out = e;
    return MOEXB_OK;
}

int moexb_ep_destroy(moexb_ep* e) {
    if (!e) return MOEXB_OK;
    e->ctx->xs = e->saved_xs; e->ctx->idx = e->saved_idx; e->ctx->w = e->saved_w;
    cudaFree(e->x); cudaFree(e->step); cudaFree(e->dev);
    delete e;
    return MOEXB_OK;
}

int moexb_ep_own_tokens(const moexb_ep* e, int* first, int* count) {
    REQUIRE(e, "ep_own_tokens: null pointer");
    if (first) *first = e->g.tok0[e->g.rank];
    if (count) *count = e->g.tok0[e->g.rank + 1] - e->g.tok0[e->g.rank];
    return MOEXB_OK;
}

int moexb_ep_read_routing(moexb_ep* e, int* idx_out, float* w_out, void* stream) {
    REQUIRE(e, "ep_read_routing: null pointer");
    const size_t n = (size_t)e->g.T * e->g.K;
    if (idx_out) CUDA_TRY(cudaMemcpyAsync(idx_out, e->ctx->idx, n * sizeof(int), cudaMemcpyDeviceToDevice, S(stream)));
    if (w_out) CUDA_TRY(cudaMemcpyAsync(w_out, e->ctx->w, n * sizeof(float), cudaMemcpyDeviceToDevice, S(stream)));
    return MOEXB_OK;
}

int moexb_ep_begin_step(moexb_ep* e, void* stream) {
    REQUIRE(e, "ep_begin_step: null pointer");
    ep_step_k<<<1, 1, 0, S(stream)>>>(e->step);
    LAUNCHED("ep_step");
    return MOEXB_OK;
}

}  // extern "C"

static int ep_check_layer(const moexb_ep* e, const moexb_layer* L, int l, const char* who) {
    REQUIRE(e && L, "%s: null pointer", who);
    REQUIRE(L->ctx == e->ctx, "%s: layer belongs to another context", who);
    REQUIRE(l >= 0 && l + 1 < (int)EP_PHASES, "%s: layer index %d", who, l);
    REQUIRE(L->n_routed == e->n_routed && L->first_local == e->g.exp0[e->g.rank] && L->n_local == e->g.exp0[e->g.rank + 1] - e->g.exp0[e->g.rank],
            "%s: the layer holds experts [%d, %d) of %d, this rank's share is [%d, %d) of %d", who, L->first_local, L->first_local + L->n_local,
            L->n_routed, e->g.exp0[e->g.rank], e->g.exp0[e->g.rank + 1], e->n_routed);
    REQUIRE(L->loaded[L->n_routed], "%s: the shared expert of this layer was never loaded", who);
    return MOEXB_OK;
}

// The owner's side of the combine of layer `l - 1` (l >= 1), leaving the next layer's input (or, with `out`, the result).
static int ep_combine(moexb_ep* e, bool f16, bool residual, unsigned phase, float* out, bool next, bool split, void* stream) {
    moexb_ctx* c = e->ctx;
    const int n_own = e->g.tok0[e->g.rank + 1] - e->g.tok0[e->g.rank];
    const float* extra = c->ypair + (size_t)e->g.T * e->g.K * EH;   // the shared expert's rows, by absolute token
    float* x = residual ? e->x : nullptr;
    float* xn = next ? c->xn : nullptr;
    uint16_t* xs = next && split ? c->xs : nullptr;
    PROF(c, MOEXB_PROF_COMBINE, stream);
    if (f16) CUDA_TRY(launch_dep(ep_combine_norm_k<true>, n_own, 256, 0, S(stream), e->g, (const uint8_t*)e->peers.base[e->g.rank], e->lay, extra, x, out, xn, xs, residual ? 1 : 0, 1e-6f, (const unsigned*)e->step, phase, c->err));
    else CUDA_TRY(launch_dep(ep_combine_norm_k<false>, n_own, 256, 0, S(stream), e->g, (const uint8_t*)e->peers.base[e->g.rank], e->lay, extra, x, out, xn, xs, residual ? 1 : 0, 1e-6f, (const unsigned*)e->step, phase, c->err));
    LAUNCHED("ep_combine_norm");
    return MOEXB_OK;
}

extern "C" {

int moexb_ep_dispatch(moexb_ep* e, moexb_layer* L, int l, const void* X, int x_dtype, int residual, void* stream) {
    int rc = ep_check_layer(e, L, l, "ep_dispatch");
    if (rc != MOEXB_OK) return rc;
    REQUIRE(l > 0 || X, "ep_dispatch: layer 0 needs the input");
    REQUIRE(x_dtype == MOEXB_F32 || x_dtype == MOEXB_BF16, "ep_dispatch: x_dtype=%d", x_dtype);
    moexb_ctx* c = e->ctx;
    cudaStream_t st = S(stream);
    const int T = e->g.T, K = e->g.K, t0 = e->g.tok0[e->g.rank], n_own = e->g.tok0[e->g.rank + 1] - t0;
    const bool tiled = L->layout == MOEXB_LAYOUT_TILED;
    REQUIRE(tiled || c->path == 0, "ep_dispatch: expert parallelism runs on the streaming kernels");
    const bool prefill = tiled && L->fmt == FMT_SYM_F16 && T >= c->prefill_min_tokens;
    const bool f16 = tiled && L->fmt != FMT_ZP && !prefill;
    // activation columns per token: the grouped GEMM takes one when the layer input is exactly bf16, else hi + lo
    const int parts = prefill && x_dtype == MOEXB_BF16 && !residual && l == 0 ? 1 : 2;
    e->prefill = prefill; e->parts = parts;
    float* xn_own = c->xn + (size_t)t0 * EH;
    if (l == 0) {
        // the own rows of the input as fp32: into the residual rows (blocks) or straight into the layer input (plain layers)
        float* dst = residual ? e->x : xn_own;
        const size_t n = (size_t)n_own * EH;
        PROF(c, MOEXB_PROF_OTHER, stream);
        if (x_dtype == MOEXB_BF16) {
            bf16_to_f32_k<<<(unsigned)((n / 2 + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(X) + (size_t)t0 * EH, dst, n);
            LAUNCHED("bf16_to_f32");
        } else CUDA_TRY(cudaMemcpyAsync(dst, static_cast<const float*>(X) + (size_t)t0 * EH, n * sizeof(float), cudaMemcpyDeviceToDevice, st));
        if (residual && !prefill) {
            if (f16) rmsnorm_split_k<true><<<n_own, 256, 0, st>>>(e->x, xn_own, c->xs + (size_t)t0 * 2 * EH, 1e-6f);
            else rmsnorm_split_k<false><<<n_own, 256, 0, st>>>(e->x, xn_own, c->xs + (size_t)t0 * 2 * EH, 1e-6f);
            LAUNCHED("rmsnorm_split");
        } else if (residual) {
            rmsnorm_rows_k<<<n_own, 256, 0, st>>>(e->x, xn_own, EH, 1e-6f);
            LAUNCHED("rmsnorm_rows");
        } else if (!prefill) {
            if (f16) split_rows_k<true><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(xn_own, c->xs + (size_t)t0 * 2 * EH, EH, n);
            else split_rows_k<false><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(xn_own, c->xs + (size_t)t0 * 2 * EH, EH, n);
            LAUNCHED("split_rows");
        }
    } else {
        rc = ep_combine(e, f16, residual != 0, (unsigned)l, nullptr, true, !prefill, stream);
        if (rc != MOEXB_OK) return rc;
    }
    if (prefill) {
        PROF(c, MOEXB_PROF_OTHER, stream);
        const size_t n = (size_t)n_own * EH;
        split8_rows_k<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(xn_own, c->xs + (size_t)t0 * parts * EH, EH, parts, n);
        LAUNCHED("split8_rows");
    }
    // the routing kernel sends each token to the peers as soon as its experts are selected and raises the tokens' flags
    const RouteEp rep{e->dev, parts * EH * 2, (unsigned)(l + 1), e->step};
    return layer_route(c, L, xn_own, n_own, K, stream, false, t0, &rep);
}

int moexb_ep_experts(moexb_ep* e, moexb_layer* L, int l, void* stream) {
    int rc = ep_check_layer(e, L, l, "ep_experts");
    if (rc != MOEXB_OK) return rc;
    moexb_ctx* c = e->ctx;
    cudaStream_t st = S(stream);
    const int T = e->g.T, K = e->g.K, E = L->n_routed, t0 = e->g.tok0[e->g.rank], t1 = e->g.tok0[e->g.rank + 1];
    const bool tiled = L->layout == MOEXB_LAYOUT_TILED, prefill = e->prefill;
    const int maxp = prefill ? PF_NMAX / e->parts : (tiled ? tiled_maxp(c, L->fmt, T) : ST_MAXP);
    const unsigned* flags = reinterpret_cast<const unsigned*>(e->peers.base[e->g.rank] + e->lay.flag_a);
    const bool in_kernel = tiled && !prefill && plan_in_kernel(c, L->fmt, T, K, E, true);
    // the dispatch flags of all tokens are waited for by whoever makes the work list: the gate/up CTAs, or the planning kernel
    const PlanArgs plan{c->idx, c->w, T, K, E, L->slot_table, L->first_local, L->first_local + L->n_local, c->logits + E, E + 1, t0, t1, maxp, c->subs, c->pairs, c->nsub, flags, e->step, (unsigned)(l + 1)};
    if (!in_kernel) {
        PROF(c, MOEXB_PROF_GROUP, stream);
        constexpr int PLAN_STAGE_MAX = 196608;
        static PerDeviceOnce plan_once;
        const cudaError_t plan_attr = plan_once.run([] { return cudaFuncSetAttribute(group_plan1_k<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PLAN_STAGE_MAX); });
        const int stage_pairs = plan_attr == cudaSuccess && (size_t)T * K * 12 <= PLAN_STAGE_MAX ? T * K : 0;
        CUDA_TRY(launch_dep(group_plan1_k<true>, 1, 1024, (size_t)stage_pairs * 12, st, (const int*)c->idx, (const float*)c->w, T, K, E, L->slot_table, c->items, c->pairs, c->nitems,
                            c->subs, c->nsub, maxp, prefill ? c->subs2 : nullptr, c->nsub2, PF_NMAX / 2, (const float*)(c->logits + E), E + 1, t0, t1, stage_pairs,
                            flags, (const unsigned*)e->step, (unsigned)(l + 1), e->g.world, e->g.rank, c->err));
        LAUNCHED("group_plan");
    }
    rc = prefill ? prefill_experts(c, L->fmt, c->pairs, nullptr, T, e->parts, c->ypair, stream, true)
       : tiled ? tiled_experts(c, L->fmt, c->pairs, nullptr, c->ypair, T, stream, in_kernel ? &plan : nullptr)
               : stream_experts(c, L->fmt, c->pairs, nullptr, c->ypair, stream);
    if (rc != MOEXB_OK) return rc;
    PROF(c, MOEXB_PROF_COMBINE, stream);
    CUDA_TRY(launch_dep(ep_partial_push_k, T, 256, 0, st, e->g, e->peers, e->lay, (const float*)c->ypair, (const unsigned*)e->step, (unsigned)(l + 1)));
    LAUNCHED("ep_partial_push");
    return MOEXB_OK;
}

int moexb_ep_finish(moexb_ep* e, int n_layers, int residual, float* out_own, void* stream) {
    REQUIRE(e && out_own, "ep_finish: null pointer");
    REQUIRE(n_layers >= 1 && n_layers < (int)EP_PHASES, "ep_finish: %d layers", n_layers);
    return ep_combine(e, true, residual != 0, (unsigned)n_layers, out_own, false, false, stream);
}

// One whole step on `stream`: begin, per layer dispatch + experts, finish. X [T][H] of x_dtype (every rank passes the whole
// batch and uses its own rows), out_own [own tokens][H].
int moexb_ep_step(moexb_ep* e, moexb_layer* const* layers, int n_layers, const void* X, int x_dtype, int residual, float* out_own, void* stream) {
    REQUIRE(e && layers && X && out_own, "ep_step: null pointer");
    int rc = moexb_ep_begin_step(e, stream);
    for (int l = 0; l < n_layers && rc == MOEXB_OK; l++) {
        rc = moexb_ep_dispatch(e, layers[l], l, X, x_dtype, residual, stream);
        if (rc == MOEXB_OK) rc = moexb_ep_experts(e, layers[l], l, stream);
    }
    if (rc == MOEXB_OK) rc = moexb_ep_finish(e, n_layers, residual, out_own, stream);
    return rc;
}

int moexb_ep_stack_create(moexb_ep* e, moexb_layer* const* layers, int n_layers, int x_dtype, int residual, moexb_stack** out) {
    REQUIRE(e && layers && out, "ep_stack_create: null pointer");
    REQUIRE(n_layers >= 1 && n_layers < (int)EP_PHASES, "ep_stack_create: %d layers", n_layers);
    REQUIRE(residual || n_layers == 1, "ep_stack_create: plain (non-residual) layers are chained one at a time");
    moexb_ctx* c = e->ctx;
    REQUIRE(!c->profiling, "ep_stack_create: switch profiling off before capturing a graph");
    CUDA_TRY(cudaSetDevice(c->device));
    moexb_stack* s = new (std::nothrow) moexb_stack;
    if (!s) return fail(MOEXB_ERR_NOMEM, "out of host memory");
    const int T = e->g.T;
    s->ctx = c; s->T = T; s->K = e->g.K; s->x_dtype = x_dtype; s->n_layers = n_layers;
    s->out_rows = e->g.tok0[e->g.rank + 1] - e->g.tok0[e->g.rank];
    const size_t n = (size_t)T * EH;
    cudaError_t err = cudaMalloc(&s->x_in, n * (x_dtype == MOEXB_BF16 ? 2 : 4));
    if (err == cudaSuccess) err = cudaMalloc((void**)&s->buf[0], (size_t)e->g.n_own_max * EH * 4);
    if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&s->cap, cudaStreamNonBlocking);
    if (err != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_NOMEM, "ep_stack_create: %s", cudaGetErrorString(err)); }
    const long long before = g_launches.load();
    err = cudaStreamBeginCapture(s->cap, cudaStreamCaptureModeThreadLocal);
    if (err != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_CUDA, "ep_stack_create: begin capture: %s", cudaGetErrorString(err)); }
    const int rc = moexb_ep_step(e, layers, n_layers, s->x_in, x_dtype, residual, s->buf[0], s->cap);
    err = cudaStreamEndCapture(s->cap, &s->graph);
    s->kernels = (int)(g_launches.load() - before);
    g_launches.store(before);
    if (rc != MOEXB_OK) { moexb_stack_destroy(s); return rc; }
    if (err == cudaSuccess) err = cudaGraphInstantiate(&s->exec, s->graph, 0);
    if (err != cudaSuccess) { moexb_stack_destroy(s); return fail(MOEXB_ERR_CUDA, "ep_stack_create: graph: %s", cudaGetErrorString(err)); }
    s->result = s->buf[0];
    *out = s;
    return MOEXB_OK;
}

// ---- instrumentation ------------------------------------------------------------------------------------------------------

long long moexb_launch_count(void) { return g_launches.load(); }

int moexb_ctx_profile(moexb_ctx* c, int on) {
    REQUIRE(c, "ctx_profile: null context");
    c->profiling = on != 0;
    return MOEXB_OK;
}

int moexb_ctx_profile_read(moexb_ctx* c, float* ms, int* launches) {
    REQUIRE(c && ms && launches, "ctx_profile_read: null pointer");
    CUDA_TRY(cudaDeviceSynchronize());
    for (int i = 0; i < MOEXB_PROF_TAGS; i++) { ms[i] = 0.f; launches[i] = 0; }
    for (auto& r : c->recs) {
        float t = 0.f;
        CUDA_TRY(cudaEventElapsedTime(&t, r.a, r.b));
        ms[r.tag] += t; launches[r.tag]++;
        c->spare.push_back(r.a); c->spare.push_back(r.b);
    }
    c->recs.clear();
    return MOEXB_OK;
}

}  // extern "C"

// ---- one-token experts with built-in scratch ------------------------------------------------------------------------------
//
// moexb_experts_forward_static is for callers that cannot allocate device memory: an engine that sizes its expert cache
// from whatever memory is free at load time has no bytes left to ask for afterwards, and code on a latency-critical
// decode thread must not call cudaMalloc at all, because an allocation can block on the whole device.
// moexb_experts_forward asks such a caller for an `act` buffer; this variant brings its own.

namespace {
constexpr int STATIC_MAX_K = 16;  // experts per call: the scratch holds STATIC_MAX_K x I floats = 32 KB
constexpr int STATIC_MAX_DEVICES = 64;
// act[k][I] of the call in flight. Every GPU that loads the library holds these 32 KB until the process exits.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address to hand to a kernel.
static __device__ __align__(256) float g_static_act[STATIC_MAX_K * EI];
std::mutex g_static_lock;
float* g_static_ptr[STATIC_MAX_DEVICES];  // device address of g_static_act per device, resolved on first use
}  // namespace

extern "C" int moexb_experts_forward_static(int fmt, const uint8_t* const* slots, const float* w, int K, const float* x, float* out,
                                            void* stream, const int* nh) {
    REQUIRE(slots && w && x && out, "experts_forward_static: null pointer");
    REQUIRE(K >= 1 && K <= STATIC_MAX_K, "experts_forward_static: K=%d exceeds the built-in scratch (at most %d experts per call)", K, STATIC_MAX_K);
    REQUIRE(fmt_ok(fmt), "experts_forward_static: unknown expert format %d", fmt);
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    REQUIRE(dev >= 0 && dev < STATIC_MAX_DEVICES, "experts_forward_static: device %d out of range", dev);
    float* act;
    {
        // Set-up, once per device and with that device current: ask the runtime where the array lives on this GPU.
        std::lock_guard<std::mutex> lock(g_static_lock);
        if (!g_static_ptr[dev]) {
            void* p = nullptr;
            CUDA_TRY(cudaGetSymbolAddress(&p, g_static_act));
            REQUIRE(p, "experts_forward_static: the scratch array has no address on device %d", dev);
            g_static_ptr[dev] = static_cast<float*>(p);
        }
        act = g_static_ptr[dev];
    }
    // Nothing in the array has to start at zero: the first kernel writes rows k < K (or < *nh), the second reads only those.
    return by_fmt(fmt, [&]<int FMT>() {
        constexpr int WARPS = 8;
        decode_gate_up_k<FMT, WARPS><<<dim3(EI / WARPS, K), WARPS * 32, 0, S(stream)>>>(slots, K, nh, x, act);
        LAUNCHED("decode_gate_up (static scratch)");
        decode_down_k<FMT, WARPS, STATIC_MAX_K><<<EH / WARPS, WARPS * 32, K * pad32_size(EI) * sizeof(float), S(stream)>>>(slots, w, K, nh, act, out);
        LAUNCHED("decode_down (static scratch)");
        return (int)MOEXB_OK;
    });
}
