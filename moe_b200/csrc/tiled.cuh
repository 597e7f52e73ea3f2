// The resident ("tiled") expert layout and the streaming kernels that read it.
//
// Why a second layout: cp.async.bulk has a per-instruction cost. Streaming the reference layout needs one copy per row
// piece (256 bytes, because rows must be padded apart in shared memory to avoid bank conflicts), and 256-byte copies top
// out near 2 TB/s on a B200; 1 KB copies reach 4 TB/s, 4 KB copies 5.7 TB/s, 16 KB copies 6.4 TB/s (measured with the
// math switched off). So the resident image stores every expert as a sequence of self-contained 4-5 KB slices, each one
// contiguous copy, already in the order the tensor-core lanes consume it. The bytes are the same as in the reference
// blob (sizes are identical); only their order changes, and tile_expert_k / untile_expert_k convert in both directions.
//
// A slice is the weights of one MMA row tile (16 rows) over 512 inputs = 8 scale groups:
//   gate/up: rows 8*wt..8*wt+7 of gate (MMA rows 0-7) and of up (MMA rows 8-15), inputs 512*ks..512*ks+511; slice index
//            wt*4 + ks, wt < 64, ks < 4.
//   down   : rows 16*wt..16*wt+15, all 512 inputs; slice index 256 + wt, wt < 128.
// Inside a slice, for each group G: 512 bytes of nibbles, 16 bytes per lane l = 4*g + t: bytes 0-7 = row A(g)'s
// 16 nibbles for inputs 64*G + 16*t .. +15, bytes 8-15 = row B(g)'s (A = MMA row g, B = MMA row g + 8); then the group's
// scale bytes: fp16 (sA, sB) per g (32 bytes), or f32 (64 bytes), or zero point [scA0 mnA0 scA1 mnA1 | scB0 mnB0 scB1 mnB1]
// per g (64 bytes). Zero-point slices end with 128 bytes of half2 (d, dm): per g [A block 0, A block 1, B block 0,
// B block 1] for the two 256-input super-blocks of the slice.
#pragma once
#include "common.cuh"
#include "stream.cuh"

namespace moexb {

constexpr int TL_SLICES = 384;  // 256 gate/up + 128 down
template <int FMT> constexpr int tl_scale_group() { return FMT == FMT_SYM_F16 ? 32 : 64; }
template <int FMT> constexpr int tl_group_bytes() { return 512 + tl_scale_group<FMT>(); }
template <int FMT> constexpr int tl_slice_bytes() { return 8 * tl_group_bytes<FMT>() + (FMT == FMT_ZP ? 128 : 0); }
static_assert(TL_SLICES * tl_slice_bytes<FMT_SYM_F16>() == expert_bytes(FMT_SYM_F16), "tiled size");
static_assert(TL_SLICES * tl_slice_bytes<FMT_SYM_F32>() == expert_bytes(FMT_SYM_F32), "tiled size");
static_assert(TL_SLICES * tl_slice_bytes<FMT_ZP>() == expert_bytes(FMT_ZP), "tiled size");

// Rows (in the blob's merged [gate | up | down] row space) and first input of slice si, MMA row m (0..15).
__device__ __forceinline__ void tl_row_of(int si, int m, size_t& qoff, size_t& c0) {
    if (si < 256) {
        const int wt = si >> 2, ks = si & 3;
        const size_t row = (size_t)(m < 8 ? 0 : EI) + 8 * wt + (m & 7);
        qoff = row * (EH / 2) + ks * 256;     // byte offset of the row's 512 inputs in the nibble area
        c0 = row * (EH / 32) + ks * 16;       // their first 32-weight chunk
    } else {
        const int d = 16 * (si - 256) + m;
        qoff = DOWN_Q_OFF + (size_t)d * (EI / 2);
        c0 = DOWN_C_OFF + (size_t)d * (EI / 32);
    }
}

// One block per slice, blockIdx.y = expert of the batch (both sides advance by the blob size): reference-layout blob <->
// tiled blob (TO_TILED = direction). 256 threads.
template <int FMT, bool TO_TILED>
__global__ void __launch_bounds__(256) tile_expert_k(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst) {
    constexpr int GB = tl_group_bytes<FMT>(), SB = tl_slice_bytes<FMT>();
    const int si = blockIdx.x, tid = threadIdx.x;
    src += (size_t)blockIdx.y * expert_bytes(FMT); dst += (size_t)blockIdx.y * expert_bytes(FMT);
    const uint8_t* ref = TO_TILED ? src : dst;   // the reference-layout side
    uint8_t* til = const_cast<uint8_t*>(TO_TILED ? dst : src) + (size_t)si * SB;
    uint8_t* refw = const_cast<uint8_t*>(ref);
    auto move = [&](uint8_t* t, size_t roff, int n) {  // n bytes between tiled address t and reference offset roff
        for (int i = 0; i < n; i++) { if (TO_TILED) t[i] = ref[roff + i]; else refw[roff + i] = t[i]; }
    };
    {   // nibbles: thread = (group G, lane l)
        const int G = tid >> 5, l = tid & 31, g = l >> 2, t = l & 3;
        size_t qa, qb, ca, cb;
        tl_row_of(si, g, qa, ca); tl_row_of(si, g + 8, qb, cb);
        move(til + G * GB + 16 * l, qa + G * 32 + 8 * t, 8);
        move(til + G * GB + 16 * l + 8, qb + G * 32 + 8 * t, 8);
    }
    if (tid < 128) {  // scales: thread = (group G, MMA row m)
        const int G = tid >> 4, j = tid & 15, g = j >> 1, ab = j & 1;
        size_t q, c0;
        tl_row_of(si, g + 8 * ab, q, c0);
        uint8_t* sc = til + G * GB + 512;
        if constexpr (FMT == FMT_SYM_F16) move(sc + 4 * g + 2 * ab, Q_BYTES + (c0 / 2 + G) * 2, 2);
        else if constexpr (FMT == FMT_SYM_F32) move(sc + 8 * g + 4 * ab, Q_BYTES + (c0 / 2 + G) * 4, 4);
        else {
            move(sc + 8 * g + 4 * ab, Q_BYTES + (c0 + 2 * G) * 2, 4);  // [sc, mn] of the group's two chunks
            if (G < 2) move(til + 8 * GB + 16 * g + 8 * ab + 4 * G, Q_BYTES + CHUNKS * 2 + (c0 / 8 + G) * 4, 4);  // (d, dm) of super-block G
        }
    }
}

// ---- the work list made inside the gate/up kernel (no planning launch) ------------------------------------------------------
//
// For batches of up to PL_MAX_TOKENS tokens every CTA of the gate/up kernel builds the whole work list itself, in shared memory,
// from the router's ids and weights (at most 512 pairs: two microseconds of redundant work per CTA, against a separate one-block
// launch that the whole grid would wait for). The list is the one group_plan1_k makes - pairs bucketed by expert, sub-items of
// at most maxp pairs with the wide ones first, the shared expert's pairs appended for tokens [sh0, sh1) - except that an
// expert's pairs are in token order here, so every CTA derives the same list: a pair's place is (pairs of its expert in
// earlier 32-pair chunks) + (its rank among the equal ids of its own chunk, from one warp match). CTA 0 also writes the list
// to global memory, for the down kernel.
constexpr int PL_MAX_TOKENS = 64, PL_MAX_K = 8, PL_MAX_PAIRS = PL_MAX_TOKENS * PL_MAX_K, PL_MAX_E = 256;
constexpr int PL_MAX_SUBS = PL_MAX_E + PL_MAX_PAIRS / 4 + PL_MAX_TOKENS / 4 + 2;
struct PlanArgs {
    const int* idx; const float* w; int T, K, E;
    const uint8_t* const* slot_table;   // E + 1 blob pointers, null = expert not held here
    int e_lo, e_hi;                     // the routed experts held here are [e_lo, e_hi) (the same fact, without a load per pair)
    const float* gate_logits; int gl_stride, sh0, sh1, maxp;
    moexb_pair_item* subs_out; moexb_pair* pairs_out; int* nsub_out;   // the list in global memory (written by CTA 0)
    const unsigned* ep_flags; const unsigned* ep_step; unsigned ep_phase;   // expert parallelism: per-token dispatch flags to wait for, or null
};
// The list as the CTA keeps it (10 KB): a sub-item as (expert id, first pair, pairs), a pair as (p, weight) with the token
// derived from p (routed pairs p = t * K + rank, the shared expert's p = T * K + t).
struct PlanSub { uint16_t e, start, count, pad; };
struct PlanSmem {
    const uint8_t* slot[PL_MAX_E + 1];   // the layer's blob pointers (copied before the wait for the kernel before this one)
    PlanSub subs[PL_MAX_SUBS];
    uint2 pairs[PL_MAX_PAIRS + PL_MAX_TOKENS];
    int nsub[2], npairs, n, K;
    __device__ __forceinline__ moexb_pair pair_at(int i) const {
        const uint2 v = pairs[i];
        const int p = (int)v.x;
        return {p < n ? p / K : p - n, p, __uint_as_float(v.y)};
    }
};
// Scratch of the planning itself (8 KB): lives where the weight ring will be, whose first copy is requested after planning.
struct PlanTmp {
    int cnt[PL_MAX_E], start[PL_MAX_E], wat[PL_MAX_E], nat[PL_MAX_E];
    uint8_t chunk[PL_MAX_PAIRS / 32][PL_MAX_E];   // pairs of expert e in chunk c; then the exclusive prefix over the chunks
    int np, nw, nn;
};

// What does not depend on the router: cleared tables and the layer's blob pointers. Runs before the wait for the kernel
// before this one; a CTA barrier must follow before plan_in_cta.
__device__ __forceinline__ void plan_prepare(PlanSmem& L, PlanTmp& P, const PlanArgs& a) {
    const int tid = threadIdx.x, NT = blockDim.x;
    for (int i = tid; i < PL_MAX_E; i += NT) P.cnt[i] = 0;
    for (int i = tid; i < (int)sizeof(P.chunk) / 4; i += NT) reinterpret_cast<uint32_t*>(P.chunk)[i] = 0;
    for (int i = tid; i <= a.E; i += NT) L.slot[i] = a.slot_table[i];
}

__device__ __forceinline__ void plan_in_cta(PlanSmem& L, PlanTmp& P, const PlanArgs& a, int* err) {
    const int tid = threadIdx.x, NT = blockDim.x, lane = tid & 31;
    const int n = a.T * a.K, E = a.E, maxp = a.maxp, lgp = __ffs(maxp) - 1;   // maxp is 4 or 8
    if (a.ep_flags) {
        const unsigned target = *a.ep_step * EP_PHASES + a.ep_phase;
        for (int t = tid; t < a.T; t += NT)
            if (t < a.sh0 || t >= a.sh1) ep_wait_flag(a.ep_flags + t, target, err, EP_ERR_DISPATCH_WAIT);
        __syncthreads();   // the peers' ids are read by other threads than the ones that saw the flags
    }
    // the shared expert's gate logits: requested now, used when the list is written
    const int Ts = (a.gate_logits && L.slot[E] && a.sh1 > a.sh0) ? a.sh1 - a.sh0 : 0;
    const float gl = tid < Ts ? __ldcg(a.gate_logits + (size_t)(a.sh0 + tid) * a.gl_stride) : 0.f;
    constexpr int MAXPT = PL_MAX_PAIRS / 128;   // pairs per thread with the smallest CTA (4 warps)
    int ex[MAXPT], rk[MAXPT];
    float wv[MAXPT];
#pragma unroll
    for (int k = 0; k < MAXPT; k++) {
        const int p = tid + k * NT;   // a warp's 32 pairs are consecutive: one chunk
        ex[k] = -1; rk[k] = 0; wv[k] = 0.f;
        if (k * NT < n) {             // the whole warp takes part in the match
            int e = p < n ? __ldcg(a.idx + p) : -1;
            if (e < a.e_lo || e >= a.e_hi) e = -1;   // experts that are not held here are dropped
            if (p < n) wv[k] = __ldcg(a.w + p);
            const unsigned m = __match_any_sync(0xffffffffu, e);
            ex[k] = e; rk[k] = __popc(m & ((1u << lane) - 1));
            if (e >= 0 && rk[k] == 0) P.chunk[p >> 5][e] = (uint8_t)__popc(m);
        }
    }
    __syncthreads();
    const int nchunks = (n + 31) >> 5;
    for (int e = tid; e < E; e += NT) {
        int c = 0;
        for (int ch = 0; ch < nchunks; ch++) { const int v = P.chunk[ch][e]; P.chunk[ch][e] = (uint8_t)c; c += v; }
        P.cnt[e] = c;
    }
    __syncthreads();
    auto wide = [maxp, lgp](int c) { return (c >> lgp) + ((c & (maxp - 1)) > maxp / 2); };
    auto narrow = [maxp](int c) { return (int)((c & (maxp - 1)) > 0 && (c & (maxp - 1)) <= maxp / 2); };
    if (tid < 32) {   // exclusive scans over the experts: pairs, wide sub-items, narrow sub-items; a lane takes 8 experts
        int c[8], sp = 0, sw = 0, sn = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) { const int e = lane * 8 + j; c[j] = e < E ? P.cnt[e] : 0; sp += c[j]; sw += wide(c[j]); sn += narrow(c[j]); }
        int ip = sp, iw = sw, in = sn;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, ip, o), uw = __shfl_up_sync(0xffffffffu, iw, o), un = __shfl_up_sync(0xffffffffu, in, o);
            if (lane >= o) { ip += up; iw += uw; in += un; }
        }
        if (lane == 31) { P.np = ip; P.nw = iw; P.nn = in; }
        int bp = ip - sp, bw = iw - sw, bn = in - sn;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int e = lane * 8 + j;
            if (e < E) { P.start[e] = bp; P.wat[e] = bw; P.nat[e] = bn; }
            bp += c[j]; bw += wide(c[j]); bn += narrow(c[j]);
        }
    }
    __syncthreads();
    const int np = P.np, nw = P.nw, nn = P.nn, all_wide = nw + wide(Ts);
    for (int e = tid; e < E; e += NT) {
        const int c = P.cnt[e];
        if (!c) continue;
        const int cw = wide(c), at = P.start[e];
        for (int j = 0; j * maxp < c; j++)
            L.subs[j < cw ? P.wat[e] + j : all_wide + P.nat[e]] = {(uint16_t)e, (uint16_t)(at + j * maxp), (uint16_t)min(maxp, c - j * maxp), 0};
    }
#pragma unroll
    for (int k = 0; k < MAXPT; k++)
        if (ex[k] >= 0) {
            const int p = tid + k * NT;
            L.pairs[P.start[ex[k]] + P.chunk[p >> 5][ex[k]] + rk[k]] = make_uint2((unsigned)p, __float_as_uint(wv[k]));
        }
    if (Ts) {
        const int cw = wide(Ts), ns = all_wide + nn;
        if (tid < Ts) L.pairs[np + tid] = make_uint2((unsigned)(n + a.sh0 + tid), __float_as_uint(1.f / (1.f + expf(-gl))));   // Ts <= PL_MAX_TOKENS <= NT
        for (int j = tid; j * maxp < Ts; j += NT)
            L.subs[j < cw ? nw + j : ns] = {(uint16_t)E, (uint16_t)(np + j * maxp), (uint16_t)min(maxp, Ts - j * maxp), 0};
    }
    if (tid == 0) { L.nsub[0] = all_wide + nn + (Ts ? narrow(Ts) : 0); L.nsub[1] = all_wide; L.npairs = np + Ts; L.n = n; L.K = a.K; }
    __syncthreads();   // also: the scratch is free for the first weight copies
}

struct TiledArgs {
    const moexb_pair_item* subs;  // sub-items: at most 4 * NB pairs each, slot = tiled blob
    const int* nsub;
    const moexb_pair* pairs;
    const uint16_t* xs;           // gate/up: activations [token][2][H] (hi, lo: fp16 for the symmetric formats, bf16 for zero point), permuted; down: act [pair p][2][I]
    float* act32;                 // gate/up: optional fp32 copy of act [p][I]
    uint16_t* act_split;          // gate/up output [p][2][I], permuted
    float* ypair;                 // down output [p][H]
    int* err;
};

// Streaming expert kernel on the tiled layout. No producer warp: every warp is its own pipeline. A warp owns a ring of D
// slice buffers; lane 0 issues one cp.async.bulk per slice (4-5 KB, one contiguous run of the blob) D slices ahead and
// the warp waits on the slice's mbarrier before consuming it, so there is no cross-warp hand-off on the weight stream.
// Work is split in rounds of NW consecutive row tiles of one sub-item (warp w takes tile w of the round); a CTA walks a
// contiguous range of rounds, so its warps share the sub-item's 8 activation columns in shared memory and swap them
// together when the range crosses into the next sub-item.
// DOWN = false: row tile = 8 gate + 8 up rows, 4 slices (K = 2048); act = silu(gate) * up.
// DOWN = true : row tile = 16 down rows, 1 slice (K = 512); ypair = w * (down . act).
// NB = 8-column blocks of activations per sub-item (1: up to 4 pairs, 2: up to 8 pairs - the weights of an expert with 5-8
// pairs are then unpacked once instead of twice); CPS = CTAs per SM the launch is sized for.
// PLAN (gate/up only): the CTA makes the work list itself (plan_in_cta) from pa instead of reading a.subs / a.pairs / a.nsub.
template <int FMT, bool DOWN, int NW, int D, int NB = 1, int CPS = 2, bool PLAN = false>
__global__ void __launch_bounds__(NW * 32, CPS) stream_tiled_k(const TiledArgs a, const PlanArgs pa) {
    static_assert(NB == 1 || FMT != FMT_ZP, "two column blocks are built for the symmetric formats only");
    static_assert(!PLAN || !DOWN, "the down kernel reads the list the gate/up kernel left in global memory");
    constexpr int GB = tl_group_bytes<FMT>(), SB = tl_slice_bytes<FMT>();
    constexpr int KS = DOWN ? 1 : 4;                       // slices per row tile
    constexpr int RPS = (DOWN ? 128 : 64) / NW;            // rounds per sub-item
    constexpr int KB = DOWN ? EI : EH;
    constexpr int BCOL = st_bcol_bytes<DOWN>();
    constexpr bool Z = FMT == FMT_ZP;
    constexpr bool F16 = !Z;  // symmetric formats run on fp16 operands (cheaper unpacking, 22-bit activations); zero point on bf16
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* bsm = smem + NW * D * SB;                                 // 8 * NB activation columns
    uint64_t* bars = reinterpret_cast<uint64_t*>(bsm + 8 * NB * BCOL); // full[NW][D]
    PlanSmem& P = *reinterpret_cast<PlanSmem*>(bars + NW * D + 8);      // PLAN only (the launch adds the room)
    static_assert(!PLAN || sizeof(PlanTmp) <= NW * D * SB, "the planning scratch fits where the ring will be");
    // zero point: the sum of the activations over each 32-input chunk, per column: [K slice][group][chunk][8 columns]
    __shared__ __align__(16) float csum[Z ? KS * 8 * 2 * 8 : 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x < NW * D) mbar_init(smem_u32(bars + threadIdx.x), 1);
    if (threadIdx.x == 0) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if constexpr (PLAN) plan_prepare(P, *reinterpret_cast<PlanTmp*>(smem), pa);
    __syncthreads();
    // Gate/up: the sub-items come from the kernel before this one. Down: they are older (the gate/up kernel read them
    // too), so the weight copies start while gate/up still runs; only the activation columns wait for it.
    // The trigger comes after the wait so that the down kernel, which reads the sub-items before its own wait, cannot
    // start before the kernel that writes them has finished.
    if constexpr (PLAN) {
        pdl_wait();
        plan_in_cta(P, *reinterpret_cast<PlanTmp*>(smem), pa, a.err);
        if (blockIdx.x == 0) {
            // the list for the kernels that follow; the down kernel may read it as soon as every CTA here has triggered
            for (int i = threadIdx.x; i < P.nsub[0]; i += NW * 32) { const PlanSub su = P.subs[i]; pa.subs_out[i] = {P.slot[su.e], su.start, su.count}; }
            for (int i = threadIdx.x; i < P.npairs; i += NW * 32) pa.pairs_out[i] = P.pair_at(i);
            if (threadIdx.x < 2) pa.nsub_out[threadIdx.x] = P.nsub[threadIdx.x];
            __threadfence();
            __syncthreads();
        }
        pdl_trigger();
        // the planning scratch was written through the generic proxy where the bulk copies (async proxy) are about to land
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    } else if (!DOWN) { pdl_wait(); pdl_trigger(); }
    // the work list: the CTA's own (PLAN) or the one in global memory
    auto sub_at = [&](int i) -> moexb_pair_item {
        if constexpr (PLAN) { const PlanSub su = P.subs[i]; return {P.slot[su.e], su.start, su.count}; }
        else return a.subs[i];
    };
    auto pair_at = [&](int i) -> moexb_pair { if constexpr (PLAN) return P.pair_at(i); else return a.pairs[i]; };
    const int nsub0 = PLAN ? P.nsub[0] : a.nsub[0], nsub1 = PLAN ? P.nsub[1] : a.nsub[1];
    // This CTA's contiguous range of rounds: an equal share of the cost, a round of a wide sub-item (more than 4 pairs,
    // they come first in subs[]) counting CW and any other CN.
    constexpr int CN = 10, CW = NB == 2 ? 13 : 10;   // measured: a wide round takes 1.3 times a narrow one in both kernels
    const long long RW = NB == 2 ? (long long)nsub1 * RPS : 0, R = (long long)nsub0 * RPS;
    const long long C = RW * CW + (R - RW) * CN;
    auto round_at = [&](long long x) { return (int)(x < RW * CW ? x / CW : RW + (x - RW * CW) / CN); };
    const int r0 = round_at(C * blockIdx.x / gridDim.x), r1 = round_at(C * (blockIdx.x + 1) / gridDim.x);
    const int Q = (r1 - r0) * KS;  // slices this warp will consume
    uint8_t* ring = smem + warp * D * SB;
    uint64_t* full = bars + warp * D;

    // slice q of this warp: round r0 + q / KS, row tile rin*NW + warp, K slice q % KS
    auto issue = [&](int q) {
        const int r = r0 + q / KS, sub = r / RPS, rin = r % RPS, wt = rin * NW + warp;
        const uint8_t* src = sub_at(sub).slot + (size_t)(DOWN ? 256 + wt : wt * 4 + q % KS) * SB;
        const uint32_t bar = smem_u32(full + q % D);
        mbar_arrive_expect_tx(bar, SB);
        bulk_g2s(smem_u32(ring + (q % D) * SB), src, SB, bar);
    };
    // the activation columns of a sub-item: 2 * count columns of KB 16-bit values, requested with 16-byte asynchronous copies
    auto request_columns = [&](const moexb_pair_item& it) {
        constexpr int CHUNKS16 = KB * 2 / 16;
        for (int i = threadIdx.x; i < 2 * it.count * CHUNKS16; i += NW * 32) {
            const int col = i / CHUNKS16, ch = i % CHUNKS16;
            const moexb_pair pr = pair_at(it.start + (col >> 1));
            const size_t row = DOWN ? (size_t)pr.p : (size_t)pr.t;
            cp_async16(smem_u32(bsm + col * BCOL + ch * 16), a.xs + (row * 2 + (col & 1)) * KB + ch * 8);
        }
    };
    // Gate/up: the first sub-item's columns are requested before the weight copies (they take longer to set up than to arrive).
    // Down: the weight copies go out first, before the wait for the gate/up kernel whose output the columns are.
    bool columns_requested = false;
    if (!DOWN && Q > 0) { request_columns(sub_at(r0 / RPS)); columns_requested = true; }
    if (lane == 0)
        for (int q = 0; q < D && q < Q; q++) issue(q);
    if (DOWN) { pdl_wait(); pdl_trigger(); }

    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acd[4] = {0.f, 0.f, 0.f, 0.f};  // acd: the second column block
    int cur_sub = -1, n = 0, start = 0;
    int failed = -1;   // the slice this warp gave up waiting for
    const uint8_t* bcol = bsm + g * BCOL + t * 16;  // the lane's activation column (pair slot g >> 1, part g & 1)
    for (int q = 0; q < Q; q++) {
        const int r = r0 + q / KS, sub = r / RPS, rin = r % RPS, ks = q % KS;
        if (sub != cur_sub) {
            // new sub-item: the CTA's warps swap the activation columns together (their weight copies stay in flight)
            cur_sub = sub;
            const moexb_pair_item it = sub_at(sub);
            n = it.count; start = it.start;
            if (!columns_requested) {
                __syncthreads();   // every warp is done with the columns that are about to be overwritten
                request_columns(it);
            }
            columns_requested = false;
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncthreads();
            if constexpr (Z) {
                // the term m_c * sum(x) of a chunk does not depend on the weight row: sum(x) once per sub-item. Chunk hc of a
                // group is bytes [32 hc, 32 hc + 32) and [64 + 32 hc, 96 + 32 hc) of the group's 128 (lanes t = 2 hc, 2 hc + 1).
                for (int i = threadIdx.x; i < KS * 8 * 2 * 8; i += NW * 32) {
                    const uint8_t* grp = bsm + (i & 7) * BCOL + (i >> 4) * 128 + ((i >> 3) & 1) * 32;
                    float sum = 0.f;
#pragma unroll
                    for (int seg = 0; seg < 2; seg++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const uint4 v = *reinterpret_cast<const uint4*>(grp + 64 * seg + 16 * h);
                            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int j = 0; j < 4; j++) sum += __uint_as_float(wv[j] << 16) + __uint_as_float(wv[j] & 0xFFFF0000u);
                        }
                    csum[i] = sum;
                }
                __syncthreads();
            }
        }
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(full + q % D), (q / D) & 1, a.err, ST_ERR_FULL_WAIT))) { failed = q; break; }
        if (ks == 0) { acc[0] = acc[1] = acc[2] = acc[3] = 0.f; acd[0] = acd[1] = acd[2] = acd[3] = 0.f; }
        const uint8_t* sl = ring + (q % D) * SB;
        const uint8_t* bp = bcol + ks * 1024;  // 8 groups of 128 bytes per slice
        auto groups = [&]<bool WIDE>() {
#pragma unroll 4
        for (int G = 0; G < 8; G++) {
            const uint4 qq = *reinterpret_cast<const uint4*>(sl + G * GB + 16 * lane);
            const uint4 B0 = *reinterpret_cast<const uint4*>(bp + G * 128), B1 = *reinterpret_cast<const uint4*>(bp + G * 128 + 64);
            uint32_t Pa[2][4], Pb[2][4];
            if constexpr (F16) { dq_word_h(qq.x, Pa[0]); dq_word_h(qq.y, Pa[1]); dq_word_h(qq.z, Pb[0]); dq_word_h(qq.w, Pb[1]); }
            else { dq_word<false>(qq.x, Pa[0]); dq_word<false>(qq.y, Pa[1]); dq_word<false>(qq.z, Pb[0]); dq_word<false>(qq.w, Pb[1]); }
            if constexpr (!Z) {
                float sa, sb;
                if constexpr (FMT == FMT_SYM_F16) {
                    const float2 s2 = __half22float2(*reinterpret_cast<const __half2*>(sl + G * GB + 512 + 4 * g));
                    sa = s2.x; sb = s2.y;
                } else {
                    const float2 s2 = *reinterpret_cast<const float2*>(sl + G * GB + 512 + 8 * g);
                    sa = s2.x; sb = s2.y;
                }
                float c[4];  // one chain of four MMAs per group; the unrolled groups interleave
                mma_16<F16>(c, Pa[0][0], Pb[0][0], Pa[0][1], Pb[0][1], B0.x, B0.y, true);
                mma_16<F16>(c, Pa[0][2], Pb[0][2], Pa[0][3], Pb[0][3], B0.z, B0.w, false);
                mma_16<F16>(c, Pa[1][0], Pb[1][0], Pa[1][1], Pb[1][1], B1.x, B1.y, false);
                mma_16<F16>(c, Pa[1][2], Pb[1][2], Pa[1][3], Pb[1][3], B1.z, B1.w, false);
                acc[0] = fmaf(c[0], sa, acc[0]); acc[1] = fmaf(c[1], sa, acc[1]);
                acc[2] = fmaf(c[2], sb, acc[2]); acc[3] = fmaf(c[3], sb, acc[3]);
                if constexpr (WIDE) {
                    {  // the same weight fragments against columns 8-15
                        const uint4 C0 = *reinterpret_cast<const uint4*>(bp + 8 * BCOL + G * 128), C1 = *reinterpret_cast<const uint4*>(bp + 8 * BCOL + G * 128 + 64);
                        float d[4];
                        mma_16<F16>(d, Pa[0][0], Pb[0][0], Pa[0][1], Pb[0][1], C0.x, C0.y, true);
                        mma_16<F16>(d, Pa[0][2], Pb[0][2], Pa[0][3], Pb[0][3], C0.z, C0.w, false);
                        mma_16<F16>(d, Pa[1][0], Pb[1][0], Pa[1][1], Pb[1][1], C1.x, C1.y, false);
                        mma_16<F16>(d, Pa[1][2], Pb[1][2], Pa[1][3], Pb[1][3], C1.z, C1.w, false);
                        acd[0] = fmaf(d[0], sa, acd[0]); acd[1] = fmaf(d[1], sa, acd[1]);
                        acd[2] = fmaf(d[2], sb, acd[2]); acd[3] = fmaf(d[3], sb, acd[3]);
                    }
                }
            } else {
                // zero point: each 32-weight chunk has its own (s, m), w = s*u + m, so a group is two partial sums
                // s_c * sum(u x) + m_c * sum(x). Lanes t = 0,1 hold chunk 0 of the group, lanes t = 2,3 chunk 1, and an MMA
                // mixes the quad's k-slots, so the chunks are separated by zeroing the other half's nibbles; sum(x)
                // comes from the table made when the columns were loaded.
                const uint2 cm = *reinterpret_cast<const uint2*>(sl + G * GB + 512 + 8 * g);      // A: sc0 mn0 sc1 mn1 | B: ...
                const uint4 dd = *reinterpret_cast<const uint4*>(sl + 8 * GB + 16 * g);           // A sb0, A sb1, B sb0, B sb1
                const uint32_t da = (G >> 2) ? dd.y : dd.x, db = (G >> 2) ? dd.w : dd.z;
                const float2 dda = __half22float2(*reinterpret_cast<const __half2*>(&da)), ddb = __half22float2(*reinterpret_cast<const __half2*>(&db));
#pragma unroll
                for (int hc = 0; hc < 2; hc++) {
                    const bool mine = (t >> 1) == hc;
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_bf16(c, mine ? Pa[0][0] : 0u, mine ? Pb[0][0] : 0u, mine ? Pa[0][1] : 0u, mine ? Pb[0][1] : 0u, B0.x, B0.y);
                    mma_bf16(c, mine ? Pa[0][2] : 0u, mine ? Pb[0][2] : 0u, mine ? Pa[0][3] : 0u, mine ? Pb[0][3] : 0u, B0.z, B0.w);
                    mma_bf16(c, mine ? Pa[1][0] : 0u, mine ? Pb[1][0] : 0u, mine ? Pa[1][1] : 0u, mine ? Pb[1][1] : 0u, B1.x, B1.y);
                    mma_bf16(c, mine ? Pa[1][2] : 0u, mine ? Pb[1][2] : 0u, mine ? Pa[1][3] : 0u, mine ? Pb[1][3] : 0u, B1.z, B1.w);
                    const float2 sx = *reinterpret_cast<const float2*>(csum + (((ks * 8 + G) * 2 + hc) * 8 + 2 * t));  // columns 2t, 2t + 1
                    const float c1[4] = {sx.x, sx.y, sx.x, sx.y};
                    const uint32_t ca = (cm.x >> (16 * hc)) & 0xFFFFu, cb = (cm.y >> (16 * hc)) & 0xFFFFu;
                    const float s_a = dda.x * (float)(ca & 0xFF), m_a = dda.y * (float)(int8_t)(ca >> 8);
                    const float s_b = ddb.x * (float)(cb & 0xFF), m_b = ddb.y * (float)(int8_t)(cb >> 8);
                    acc[0] += fmaf(s_a, c[0], m_a * c1[0]); acc[1] += fmaf(s_a, c[1], m_a * c1[1]);
                    acc[2] += fmaf(s_b, c[2], m_b * c1[2]); acc[3] += fmaf(s_b, c[3], m_b * c1[3]);
                }
            }
        }
        };
        // one branch per slice, none inside the unrolled groups (their MMA chains interleave)
        if (NB == 2 && n > 4) groups.template operator()<NB == 2>(); else groups.template operator()<false>();
        // this slice is consumed: order the warp's reads before the copy that refills the buffer, then issue it
        __syncwarp();
        if (lane == 0 && q + D < Q) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(q + D);
        }
        if (ks == KS - 1) {
            // epilogue: the lane's columns 2t (hi) and 2t+1 (lo) of column block b belong to pair slot 4b + t
            const int wt = rin * NW + warp;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (4 * b + t >= n) break;
                const moexb_pair pr = pair_at(start + 4 * b + t);
                const float va = b ? acd[0] + acd[1] : acc[0] + acc[1], vb = b ? acd[2] + acd[3] : acc[2] + acc[3];
                if (DOWN) {
                    const int d = 16 * wt + g;
                    a.ypair[(size_t)pr.p * EH + d] = pr.w * va;
                    a.ypair[(size_t)pr.p * EH + d + 8] = pr.w * vb;
                } else {
                    const int row = 8 * wt + g;
                    const float v = va / (1.f + expf(-va)) * vb;
                    if (a.act32) a.act32[(size_t)pr.p * EI + row] = v;
                    uint16_t hi, lo;
                    split_hi_lo<F16>(v, hi, lo);
                    uint16_t* dst = a.act_split + (size_t)pr.p * 2 * EI + split_pos(row);
                    dst[0] = hi; dst[EI] = lo;
                }
            }
        }
    }
    if (failed >= 0) {
        // A wait ran out. The other warps of the CTA carry on, so this warp still takes part in every CTA barrier they will
        // reach (three per change of sub-item with zero-point blobs, else two), without computing; then it waits (bounded) for
        // the copies it has requested - slices [failed, failed + D) - so that none is in flight when the CTA leaves.
        for (int q = failed + 1; q < Q; q++) {
            const int sub = (r0 + q / KS) / RPS;
            if (sub != cur_sub) { cur_sub = sub; __syncthreads(); __syncthreads(); if (Z) __syncthreads(); }
        }
        for (int q = failed; q < min(Q, failed + D); q++) mbar_wait(smem_u32(full + q % D), (q / D) & 1, a.err, ST_ERR_FULL_WAIT);
    }
}

template <int FMT, bool DOWN, int NW, int D, int NB = 1, bool PLAN = false>
constexpr int tl_smem_bytes() { return NW * D * tl_slice_bytes<FMT>() + 8 * NB * st_bcol_bytes<DOWN>() + NW * D * 8 + 64 + (PLAN ? (int)sizeof(PlanSmem) + 16 : 0); }

}  // namespace moexb
