// One token through a whole stack of residual MoE blocks in ONE cooperative launch.
//
// A single token touches 17 MB per layer - 2.6 us of HBM time - so a layer made of separate launches is all latency: every
// kernel is a chain of dependent global round trips plus its launch. Here one persistent CTA per SM (all co-resident:
// cudaLaunchCooperativeKernel) walks the layers, and what every CTA needs of the token (the residual row, its rmsnorm, the
// fp16 hi + lo split, the selected experts) lives in its own shared memory, recomputed redundantly by every CTA instead of
// being passed through global memory. Per layer:
//   P1  router logits: CTA b computes rows b and b + grid of W . xn (one warp per row, the pinned summation order of
//       gemv_rows_k; the rows were copied into shared memory during the layer before) -> logits[E + 1] in global memory.                                        -- grid barrier --
//   P2  every CTA: which K experts - the logits that reach the K-th largest warp maximum (a few dozen) are compacted and
//       ranked among themselves (how many are larger, ties to the lower index; no sequential rounds); rank < K = selected. The softmax
//       weights are off this path: the last CTA takes no expert work and instead runs topk_token on the same logits
//       (the same experts by construction) and publishes the K + 1 weights, which are first needed in P5.
//   P3  gate/up: (expert, row tile of 8 gate + 8 up rows) units, two per CTA pass, the four K slices of a unit on four
//       warps (one 4.3 KB bulk copy each, issued as soon as P2 is done), partial sums added in shared memory, SiLU * up
//       -> act[K + 1][2][I] (fp16 hi, lo) in global memory. The warps' down slices (P4) are requested at the same time.
//                                                                                              -- grid barrier --
//   P4  down: a CTA takes a 16-row tile for all K + 1 experts (warp k the routed expert k; the shared expert's slice one
//       input group per warp), the experts' act rows come from L2; the tile's rows of x += sum of the weighted rows in
//       rank order (the products and the order of the down kernel + reduce_residual_norm_k) -> xnew[H] in global memory.
//                                                                                              -- grid barrier --
//   P5  every CTA: the new row from L2 (8 KB), rmsnorm and split for the next layer, all in shared memory.
// The grid barrier is a monotonic counter in global memory (zeroed by the host before the launch): one thread per CTA adds
// 1 and polls until the counter reaches (barriers so far) x grid. Every poll loop is bounded; a time-out sets the error
// word and an abort flag that all other loops watch, and the CTAs leave after waiting (bounded) for their copies in flight.
// The arithmetic of a slice is that of stream_tiled_k (exact fp16 nibbles, hi + lo activations, mma.sync, fp32 group
// scales), so results agree with the multi-launch path to rounding of the partial-sum order; logits, selected experts and
// the rmsnorm are bit-identical.
#pragma once
#include "common.cuh"
#include "router.cuh"
#include "stream.cuh"
#include "tiled.cuh"

namespace moexb {

struct DecodeLayer {
    const void* router;                   // [E + 1][H] f32 or f16
    const uint8_t* const* slot_table;     // E + 1 blob pointers (tiled layout)
};

struct DecodeStackArgs {
    const DecodeLayer* layers;
    int n_layers, E, K;
    const void* x_in;        // [H] f32 or bf16
    float* x_out;            // [H]
    float* logits;           // [E + 1]
    uint16_t* act;           // [K + 1][2][I] fp16 hi, lo in split_pos order
    float* ypair;            // [H] the new residual row, written tile by tile in P4
    float* wts;              // [K + 1] routing weights of the selected experts, then the shared expert's gate
    int* idx_out;            // optional [n_layers][K]
    float* w_out;            // optional [n_layers][K]
    unsigned* sync;          // [0] barrier counter, [1] abort flag; zero before the launch
    int* err;
};

constexpr int DS_WARPS = 8, DS_THREADS = DS_WARPS * 32;
constexpr int DS_D = 3;                       // slice buffers per warp
constexpr int DS_XCOL = EH * 2 + 64;          // stride between the hi and lo columns of the token (bytes)
constexpr int DS_ACOL = EI * 2 + 64;          // the same for an expert's act row
constexpr int DS_MAXK = 8;
constexpr int DS_MAXLAYERS = 128;
constexpr int DS_POLL_LIMIT = 1 << 21;       // polls of a grid barrier (an L2 round trip each: a second or two) before a CTA gives up
constexpr int DS_ERR_BARRIER = 5, DS_ERR_COPY = 6;

template <int FMT> constexpr int ds_smem_bytes() {
    return DS_WARPS * DS_D * tl_slice_bytes<FMT>() + 2 * DS_XCOL + DS_WARPS * 2 * DS_ACOL + 2 * EH * 4 /* xres, xn */ +
           2 * 4 * 16 * 2 * 4 /* partial sums */ + DS_WARPS * DS_D * 8 + 2 * EH * 4 /* router rows */ + (256 + 1) * 8 + 8 /* slot table */ +
           tl_slice_bytes<FMT>() + 2 * DS_ACOL /* the shared expert's down slice and act row */ + 2 * DS_WARPS * 16 * 4 /* down results */ + 256;
}

// 8 groups of one slice against the lane's two activation columns (bp: the lane's column pointer, already offset to the
// slice's first input); acc[0..1] += row g, acc[2..3] += row g + 8 (columns 2t, 2t + 1).
template <int FMT>
__device__ __forceinline__ void ds_slice(const uint8_t* __restrict__ sl, const uint8_t* __restrict__ bp, int lane, float (&acc)[4], int G0 = 0, int G1 = 8,
                                         const float* __restrict__ sums = nullptr) {
    constexpr int GB = tl_group_bytes<FMT>();
    const int g = lane >> 2, t = lane & 3;
#pragma unroll 4
    for (int G = G0; G < G1; G++) {
        const uint4 qq = *reinterpret_cast<const uint4*>(sl + G * GB + 16 * lane);
        const uint4 B0 = *reinterpret_cast<const uint4*>(bp + G * 128), B1 = *reinterpret_cast<const uint4*>(bp + G * 128 + 64);
        uint32_t Pa[2][4], Pb[2][4];
        if constexpr (FMT != FMT_ZP) {
            dq_word_h(qq.x, Pa[0]); dq_word_h(qq.y, Pa[1]); dq_word_h(qq.z, Pb[0]); dq_word_h(qq.w, Pb[1]);
            float sa, sb;
            if constexpr (FMT == FMT_SYM_F16) {
                const float2 s2 = __half22float2(*reinterpret_cast<const __half2*>(sl + G * GB + 512 + 4 * g));
                sa = s2.x; sb = s2.y;
            } else {
                const float2 s2 = *reinterpret_cast<const float2*>(sl + G * GB + 512 + 8 * g);
                sa = s2.x; sb = s2.y;
            }
            float c[4];
            mma_16<true>(c, Pa[0][0], Pb[0][0], Pa[0][1], Pb[0][1], B0.x, B0.y, true);
            mma_16<true>(c, Pa[0][2], Pb[0][2], Pa[0][3], Pb[0][3], B0.z, B0.w, false);
            mma_16<true>(c, Pa[1][0], Pb[1][0], Pa[1][1], Pb[1][1], B1.x, B1.y, false);
            mma_16<true>(c, Pa[1][2], Pb[1][2], Pa[1][3], Pb[1][3], B1.z, B1.w, false);
            acc[0] = fmaf(c[0], sa, acc[0]); acc[1] = fmaf(c[1], sa, acc[1]);
            acc[2] = fmaf(c[2], sb, acc[2]); acc[3] = fmaf(c[3], sb, acc[3]);
        } else {
            // zero point (bf16 operands): each 32-weight chunk has its own (s, m), w = s*u + m, so a group is two partial
            // sums s_c * sum(u x) + m_c * sum(x). The two chunks of a group are separated by zeroing the other half's
            // nibbles; sum(x) does not depend on the weight row and comes from `sums` ([group][chunk][hi, lo], made once
            // per activation row).
            dq_word<false>(qq.x, Pa[0]); dq_word<false>(qq.y, Pa[1]); dq_word<false>(qq.z, Pb[0]); dq_word<false>(qq.w, Pb[1]);
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
                const float2 sx = *reinterpret_cast<const float2*>(sums + G * 4 + hc * 2);   // the chunk's sum of the hi and of the lo column
                const float c1[4] = {sx.x, sx.y, sx.x, sx.y};   // columns 2t (hi), 2t + 1 (lo) of rows g and g + 8
                const uint32_t ca = (cm.x >> (16 * hc)) & 0xFFFFu, cb = (cm.y >> (16 * hc)) & 0xFFFFu;
                const float s_a = dda.x * (float)(ca & 0xFF), m_a = dda.y * (float)(int8_t)(ca >> 8);
                const float s_b = ddb.x * (float)(cb & 0xFF), m_b = ddb.y * (float)(int8_t)(cb >> 8);
                acc[0] += fmaf(s_a, c[0], m_a * c1[0]); acc[1] += fmaf(s_a, c[1], m_a * c1[1]);
                acc[2] += fmaf(s_b, c[2], m_b * c1[2]); acc[3] += fmaf(s_b, c[3], m_b * c1[3]);
            }
        }
    }
}

// Sum of the 32 bf16 values of one zero-point chunk of an activation column: chunk hc of a group is bytes
// [32 hc, 32 hc + 32) and [64 + 32 hc, 96 + 32 hc) of the group's 128 (the k-slots of lanes t = 2 hc, 2 hc + 1).
__device__ __forceinline__ float ds_chunk_sum(const uint8_t* group, int hc) {
    float s = 0.f;
#pragma unroll
    for (int seg = 0; seg < 2; seg++)
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const uint4 v = *reinterpret_cast<const uint4*>(group + 64 * seg + 32 * hc + 16 * q);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) s += __uint_as_float(w[i] << 16) + __uint_as_float(w[i] & 0xFFFF0000u);
        }
    return s;
}

// One thread per CTA: arrive at the grid barrier (sync[0], a monotonic counter) and poll until `target` arrivals have been
// counted. False when another CTA raised the abort flag (sync[1]) or after `limit` polls, in which case the error word and
// the abort flag are set.
__device__ __forceinline__ bool ds_barrier_arrive_wait(unsigned* sync, unsigned target, int* err, int limit = DS_POLL_LIMIT) {
    // release: the CTA's writes (ordered before this by the caller's block barrier) are visible to whoever sees the count
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(sync) : "memory");
    for (int i = 0; i < limit; i++) {
        unsigned seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(sync) : "memory");
        if (seen >= target) return true;
        if ((i & 63) == 63) {
            unsigned ab;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ab) : "l"(sync + 1) : "memory");
            if (ab) return false;
        }
    }
    atomicExch(err, DS_ERR_BARRIER);
    atomicExch(sync + 1, 1u);
    return false;
}

// WT: router weight type; XBF: the input row is bf16. Symmetric formats run on fp16 operands, zero point on bf16.
template <int FMT, typename WT, bool XBF>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_stack_k(const DecodeStackArgs a) {
    constexpr int SB = tl_slice_bytes<FMT>();
    constexpr bool F16 = FMT != FMT_ZP;   // element type of the split activations
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;                                               // [warp][DS_D][SB]
    uint8_t* xcol = ring + DS_WARPS * DS_D * SB;                        // token hi, lo columns (fp16, split_pos order)
    uint8_t* acol = xcol + 2 * DS_XCOL;                                 // [warp][2][DS_ACOL] act columns for the down slice
    float* xres = reinterpret_cast<float*>(acol + DS_WARPS * 2 * DS_ACOL);  // [H] the residual row
    float* xn = xres + EH;                                              // [H] its rmsnorm
    float* part = xn + EH;                                              // [2 units][4 k slices][16 rows][2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(part + 2 * 4 * 16 * 2);    // [warp][DS_D]
    uint8_t* rrow = reinterpret_cast<uint8_t*>(bars + DS_WARPS * DS_D);     // this CTA's (at most two) router rows of the coming layer
    const uint8_t** table = reinterpret_cast<const uint8_t**>(rrow + 2 * EH * 4);   // the coming layer's E + 1 blob pointers
    uint8_t* shbuf = reinterpret_cast<uint8_t*>(table) + (256 + 1) * 8 + 8;         // the shared expert's down slice of this CTA's row tile
    uint8_t* shcol = shbuf + SB;                                                    // the shared expert's act row (hi, lo)
    float* yrt = reinterpret_cast<float*>(shcol + 2 * DS_ACOL);                     // [warp][16] a routed expert's 16 down rows
    float* ysh = yrt + DS_WARPS * 16;                                               // [warp][16] the shared expert's, one input group per warp
    __shared__ __align__(8) uint64_t shbar;
    __shared__ int s_idx[DS_MAXK];
    __shared__ float s_w[DS_MAXK];
    __shared__ const uint8_t* s_slot[DS_MAXK + 1];
    __shared__ float s_wt[DS_MAXK + 1];
    __shared__ int s_abort;
    __shared__ unsigned s_keys[DS_THREADS];   // the candidates' logits as ordered integer keys
    __shared__ int s_cidx[DS_THREADS];        // and their expert ids
    __shared__ unsigned s_wmax[DS_WARPS];
    __shared__ unsigned s_tau;
    __shared__ int s_wcnt[DS_WARPS];
    __shared__ int s_idx2[DS_MAXK];
    __shared__ const uint8_t* s_slot2[DS_MAXK + 1];
    // zero point only: sum(x) per 32-input chunk of the token's columns, of each routed expert's act row, of the shared one's
    __shared__ __align__(16) float s_xsum[4 * 8 * 4], s_asum[DS_WARPS * 8 * 4], s_shsum[DS_WARPS * 4];
    __shared__ DecodeLayer s_layers[DS_MAXLAYERS];   // the layer descriptors: no global round trip when a layer is staged
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int grid = gridDim.x, b = blockIdx.x, E = a.E, K = a.K, O = E + 1;
    if (tid < DS_WARPS * DS_D) mbar_init(smem_u32(bars + tid), 1);
    if (tid == 0) mbar_init(smem_u32(&shbar), 1);
    if (tid == 0) { s_abort = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    for (int i = tid; i < a.n_layers; i += DS_THREADS) s_layers[i] = a.layers[i];
    // the token: residual row, rmsnorm, split (every CTA its own copy)
    float v[8];
    {
        float x8[8];
        if constexpr (XBF) {
            const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(a.x_in);
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int i = 0; i < 4; i++) x8[4 * h + i] = __bfloat162float(x[1024 * h + 4 * tid + i]);
        } else {
            const float* x = static_cast<const float*>(a.x_in);
            const float4 p = *reinterpret_cast<const float4*>(x + 4 * tid), q = *reinterpret_cast<const float4*>(x + 1024 + 4 * tid);
            x8[0] = p.x; x8[1] = p.y; x8[2] = p.z; x8[3] = p.w; x8[4] = q.x; x8[5] = q.y; x8[6] = q.z; x8[7] = q.w;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = x8[i];
#pragma unroll
        for (int h = 0; h < 2; h++)
            *reinterpret_cast<float4*>(xres + 1024 * h + 4 * tid) = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
    }
    __syncthreads();
    norm_split_row<F16>(v, xn, reinterpret_cast<uint16_t*>(xcol), 1e-6f, DS_XCOL / 2);
    __syncthreads();
    // [K slice][group][chunk][hi, lo]: thread = (column, K slice, group, chunk); read by P3 after later block barriers
    auto x_sums = [&]() {
        if (FMT == FMT_ZP && tid < 128) {
            const int col = tid >> 6, c = tid & 63;
            s_xsum[(c >> 1) * 4 + (c & 1) * 2 + col] = ds_chunk_sum(xcol + col * DS_XCOL + (c >> 1) * 128, c & 1);
        }
    };
    x_sums();

    // The router rows this CTA owns and the slot table of layer l: requested (cp.async) while the layer before still streams
    // its experts, so that P1 and P2 find them in shared memory.
    auto stage_layer = [&](int l) {
        const DecodeLayer Ln = s_layers[l];
        for (int w = 0; w < 2; w++) {
            const int r = b + w * grid;
            if (r < O) {
                const uint8_t* src = static_cast<const uint8_t*>(Ln.router) + (size_t)r * EH * sizeof(WT);
                for (int i = tid * 16; i < EH * (int)sizeof(WT); i += DS_THREADS * 16) cp_async16(smem_u32(rrow + w * EH * sizeof(WT) + i), src + i);
            }
        }
        for (int i = tid; i < O; i += DS_THREADS) cp_async8(smem_u32(table + i), Ln.slot_table + i);
    };
    stage_layer(0);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    unsigned barriers = 0;   // grid barriers passed
    // all CTAs have finished the phase before this call; false: time-out or abort
    auto grid_barrier = [&]() -> bool {
        __syncthreads();
        if (tid == 0 && !ds_barrier_arrive_wait(a.sync, (barriers + 1) * (unsigned)grid, a.err)) s_abort = 1;
        barriers++;
        __syncthreads();
        return !s_abort;
    };

    // slices of this warp per layer: n3 gate/up passes (unit = 2 * (pass * grid + b) + (warp >> 2), K slice warp & 3), then n4
    // down passes (unit = (pass * grid + b) * DS_WARPS + warp)
    // The last CTA computes the routing weights instead of expert work (a one-CTA grid does both, weights first).
    const bool weights_cta = b == grid - 1;
    const int wgrid = grid > 1 ? grid - 1 : 1;
    const bool worker = grid == 1 || !weights_cta;
    const int U3 = (K + 1) * 64, U4 = EH / 16;   // gate/up units; down row tiles (a CTA takes a tile for all K + 1 experts)
    const int n3 = (U3 + 2 * wgrid - 1) / (2 * wgrid), n4 = (U4 + wgrid - 1) / wgrid, nS = n3 + n4;
    uint8_t* myring = ring + warp * DS_D * SB;
    uint64_t* mybars = bars + warp * DS_D;
    long long S0 = 0;        // slices (list entries) of this warp in earlier layers
    // source of list entry s of this layer, or null when the entry is empty
    auto slice_src = [&](int s) -> const uint8_t* {
        if (!worker) return nullptr;
        if (s < n3) {
            const int u = 2 * (s * wgrid + b) + (warp >> 2);
            if (u >= U3) return nullptr;
            return s_slot[u >> 6] + (size_t)((u & 63) * 4 + (warp & 3)) * SB;
        }
        const int tt = (s - n3) * wgrid + b;   // down: routed expert `warp`, row tile tt
        if (tt >= U4 || warp >= K) return nullptr;
        return s_slot[warp] + (size_t)(256 + tt) * SB;
    };
    auto issue = [&](int s) {   // lane 0
        const uint8_t* src = slice_src(s);
        if (!src) return;
        const long long S = S0 + s;
        const uint32_t bar = smem_u32(mybars + S % DS_D);
        mbar_arrive_expect_tx(bar, SB);
        bulk_g2s(smem_u32(myring + (S % DS_D) * SB), src, SB, bar);
    };
    uint32_t sh_phase = 0;   // parity of the next completion of the shared expert's slice barrier
    bool sh_inflight = false;   // a copy into shbuf was requested and not yet waited for (every thread keeps track)
    auto issue_shared = [&](int pass) {   // thread 0: the shared expert's down slice of this CTA's row tile of the pass
        const int tt = pass * wgrid + b;
        if (!worker || tt >= U4) return;
        mbar_arrive_expect_tx(smem_u32(&shbar), SB);
        bulk_g2s(smem_u32(shbuf), s_slot[K] + (size_t)(256 + tt) * SB, SB, smem_u32(&shbar));
    };
    uint32_t phase = 0;      // bit j: parity of the next completion of buffer j's barrier (empty list entries skip a buffer)
    auto wait_slice = [&](int s) -> bool {
        const int j = (int)((S0 + s) % DS_D);
        const bool in = mbar_wait(smem_u32(mybars + j), (phase >> j) & 1u, a.err, DS_ERR_COPY);
        phase ^= 1u << j;
        if (!in) { atomicExch(a.sync + 1, 1u); s_abort = 1; }
        return in;
    };
    int issued = 0, consumed = 0;   // list entries of this layer (the warp's lanes agree)
    bool ok = true;

    for (int l = 0; l < a.n_layers && ok; l++) {
            // ---- P1: router logits of rows b, b + grid, .. (one warp each) ----
        if (warp < 2 && b + warp * grid < O) {
            const int r = b + warp * grid;
            const WT* wr = reinterpret_cast<const WT*>(rrow + warp * EH * sizeof(WT));
            float acc = 0.f;
#pragma unroll
            for (int u = 0; u < 16; u++) {
                float4 w;
                if constexpr (sizeof(WT) == 4) w = *reinterpret_cast<const float4*>(wr + 128 * u + 4 * lane);
                else {
                    const uint2 h = *reinterpret_cast<const uint2*>(wr + 128 * u + 4 * lane);
                    const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&h.x)), q = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
                    w = make_float4(p.x, p.y, q.x, q.y);
                }
                const float4 x = *reinterpret_cast<const float4*>(xn + 128 * u + 4 * lane);
                acc = fmaf(w.x, x.x, acc); acc = fmaf(w.y, x.y, acc); acc = fmaf(w.z, x.z, acc); acc = fmaf(w.w, x.w, acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) __stcg(a.logits + r, acc);
        }
        if (!(ok = grid_barrier())) break;
        // ---- P2: selection (every CTA). No sequential rounds: (1) a threshold that at least K logits reach - the K-th largest of
        // the warps' maxima; (2) the logits at or above it (a few dozen) are compacted into a list; (3) list entry j counts the
        // entries that come before it (larger, or equal with a lower expert id - the order of topk_token's rounds): those with
        // fewer than K before them are the selection, the count is their rank ----
        {
            const int nw = E >> 5;   // warps that hold logits
            unsigned key = 0u;
            if (tid < E) { const float x = __ldcg(a.logits + tid); key = f2key(x != x ? -INFINITY : x); }
            const unsigned wmax = __reduce_max_sync(0xffffffffu, key);
            if (lane == 0) s_wmax[warp] = wmax;
            __syncthreads();
            // the threshold: the warp maximum with exactly K - 1 maxima before it (lane w2 of warp 0 ranks maximum w2); with fewer
            // warps than K every logit is a candidate
            if (tid < 32) {
                if (tid == 0) s_tau = 0u;
                __syncwarp();
                if (nw >= K && tid < nw) {
                    const unsigned m2 = s_wmax[tid];
                    int before = 0;
                    for (int w3 = 0; w3 < nw; w3++) before += s_wmax[w3] > m2 || (s_wmax[w3] == m2 && w3 < tid);
                    if (before == K - 1) s_tau = m2;
                }
            }
            __syncthreads();
            const unsigned tau = s_tau;
            const bool cand = tid < E && key >= tau;
            const unsigned mask = __ballot_sync(0xffffffffu, cand);
            if (lane == 0) s_wcnt[warp] = __popc(mask);
            __syncthreads();
            int off = 0, C = 0;
            for (int w2 = 0; w2 < DS_WARPS; w2++) { const int c2 = s_wcnt[w2]; if (w2 < warp) off += c2; C += c2; }
            if (cand) { const int at = off + __popc(mask & ((1u << lane) - 1)); s_keys[at] = key; s_cidx[at] = tid; }
            __syncthreads();
            if (tid < C) {   // entries are in ascending expert order, so "lower expert id" is "earlier in the list"
                const unsigned kj = s_keys[tid];
                int cnt = 0;
                for (int c2 = 0; c2 < C; c2++) { const unsigned k2 = s_keys[c2]; cnt += k2 > kj || (k2 == kj && c2 < tid); }
                if (cnt < K) {
                    const int e = s_cidx[tid];
                    s_idx[cnt] = e; s_slot[cnt] = table[e];
                    if (b == 0 && a.idx_out) a.idx_out[(size_t)l * K + cnt] = e;
                }
            }
            if (tid == 0) s_slot[K] = table[E];
            __syncthreads();
        }
        if (weights_cta && warp == 0) {
            // the softmax weights, off the other CTAs' path: first read after two more grid barriers
            const TopkOut o{s_idx2, s_w, table, s_slot2, s_wt, nullptr, nullptr, nullptr};
            topk_token<8, true>(a.logits, 0, E, K, 1, lane, o);
            __syncwarp();
            if (lane <= K) __stcg(a.wts + lane, s_wt[lane]);
            if (lane < K && a.w_out) a.w_out[(size_t)l * K + lane] = s_w[lane];
        }
        // ---- P3: gate/up. All copies this layer needs that fit the ring are requested now, the down slices included ----
        // Only the gate/up slices are requested now: the down slices are not needed before the next grid barrier, and asked for
        // together with the others they would take a third of the HBM bandwidth that P3 is waiting on. They are requested as the
        // warp's gate/up passes complete (below), and land while the grid waits at the barrier.
        issued = 0; consumed = 0;
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the buffers were read by the warp in the layer before
            for (; issued < n3 && issued < DS_D; issued++) issue(issued);
        }
        issued = __shfl_sync(0xffffffffu, issued, 0);
        if (l + 1 < a.n_layers) stage_layer(l + 1);   // lands while the experts stream; waited for at the end of the layer
        for (int pass = 0; pass < n3 && ok; pass++) {
            const int u = worker ? 2 * (pass * wgrid + b) + (warp >> 2) : U3;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (u < U3) {
                if (!wait_slice(pass)) { ok = false; }
                else ds_slice<FMT>(myring + ((S0 + pass) % DS_D) * SB, xcol + (g & 1) * DS_XCOL + t * 16 + (warp & 3) * 1024, lane, acc, 0, 8, s_xsum + (warp & 3) * 32);
            }
            consumed = pass + 1;
            __syncwarp();
            if (lane == 0 && issued < nS) { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); issue(issued); }
            if (issued < nS) issued++;
            if (pass == 0) {   // the shared expert's down slice of this CTA's row tile: behind the first gate/up pass as well
                if (tid == 0) { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); issue_shared(0); }
                sh_inflight = worker && b < U4;
            }
            if (t == 0 && u < U3) {
                float* p = part + (((warp >> 2) * 4 + (warp & 3)) * 16 + g) * 2;
                p[0] = acc[0] + acc[1]; p[1] = acc[2] + acc[3];
            }
            __syncthreads();
            if ((warp & 3) == 0 && lane < 8 && u < U3) {   // rows 8*wt + lane of gate and up: add the four K slices, SiLU * up
                const float* p = part + ((warp >> 2) * 4 * 16 + lane) * 2;
                float G = 0.f, U = 0.f;
#pragma unroll
                for (int ks = 0; ks < 4; ks++) { G += p[ks * 32]; U += p[ks * 32 + 1]; }
                const float val = G / (1.f + expf(-G)) * U;
                uint16_t hi, lo;
                split_hi_lo<F16>(val, hi, lo);
                const int k = u >> 6, row = 8 * (u & 63) + lane;
                uint16_t* dst = a.act + (size_t)k * 2 * EI + split_pos(row);
                __stcg(dst, hi); __stcg(dst + EI, lo);
            }
            ok = __syncthreads_and(ok);   // also: every warp leaves the loop together when a copy timed out
        }
        if (!ok || !(ok = grid_barrier())) break;
        // ---- P4: down. A CTA takes a 16-row tile for all K + 1 experts: warp k the routed expert k, and the shared expert's
        // slice one input group per warp; the slices are (mostly) in shared memory already, the act rows come from L2. The
        // tile's rows of the new residual row are finished here: x += sum of the weighted rows in rank order ----
        if (tid <= K) s_wt[tid] = __ldcg(a.wts + tid);   // published by the last CTA before the barrier just passed
        for (int pass = 0; pass < n4 && ok; pass++) {
            const int tt = worker ? pass * wgrid + b : U4;
            if (tt < U4) {
                if (tid < 128) *reinterpret_cast<uint4*>(shcol + (tid >> 6) * DS_ACOL + (tid & 63) * 16) = __ldcg(reinterpret_cast<const uint4*>(a.act + (size_t)K * 2 * EI) + tid);
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                if (warp < K) {
                    uint8_t* ac = acol + warp * 2 * DS_ACOL;
                    const uint4* src = reinterpret_cast<const uint4*>(a.act + (size_t)warp * 2 * EI);   // 2 x 1024 bytes
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int c = lane + 32 * i;   // 16-byte chunk 0..127: column c >> 6, chunk c & 63
                        *reinterpret_cast<uint4*>(ac + (c >> 6) * DS_ACOL + (c & 63) * 16) = __ldcg(src + c);
                    }
                    __syncwarp();
                    if constexpr (FMT == FMT_ZP) {   // lane = (group, chunk, column)
                        s_asum[warp * 32 + lane] = ds_chunk_sum(ac + (lane & 1) * DS_ACOL + (lane >> 2) * 128, (lane >> 1) & 1);
                        __syncwarp();
                    }
                    if (!wait_slice(n3 + pass)) ok = false;
                    else ds_slice<FMT>(myring + ((S0 + n3 + pass) % DS_D) * SB, ac + (g & 1) * DS_ACOL + t * 16, lane, acc, 0, 8, s_asum + warp * 32);
                    if (t == 0) { yrt[warp * 16 + g] = acc[0] + acc[1]; yrt[warp * 16 + g + 8] = acc[2] + acc[3]; }
                }
                __syncthreads();   // the shared expert's act row is in
                if (!mbar_wait(smem_u32(&shbar), sh_phase, a.err, DS_ERR_COPY)) { atomicExch(a.sync + 1, 1u); s_abort = 1; ok = false; }
                else {
                    float as[4] = {0.f, 0.f, 0.f, 0.f};
                    if constexpr (FMT == FMT_ZP) {   // this warp's input group of the shared act row: lanes 0-3 = (chunk, column)
                        if (lane < 4) s_shsum[warp * 4 + lane] = ds_chunk_sum(shcol + (lane & 1) * DS_ACOL + warp * 128, lane >> 1);
                        __syncwarp();
                    }
                    ds_slice<FMT>(shbuf, shcol + (g & 1) * DS_ACOL + t * 16, lane, as, warp, warp + 1, s_shsum);
                    if (t == 0) { ysh[warp * 16 + g] = as[0] + as[1]; ysh[warp * 16 + g + 8] = as[2] + as[3]; }
                }
                sh_phase ^= 1u;
                sh_inflight = false;
            }
            consumed = n3 + pass + 1;
            __syncthreads();
            if (tt < U4 && tid < 16) {
                float acc = 0.f;
                for (int r = 0; r < K; r++) acc += __fmul_rn(s_wt[r], yrt[r * 16 + tid]);
                float sh = 0.f;
#pragma unroll
                for (int w = 0; w < DS_WARPS; w++) sh += ysh[w * 16 + tid];
                acc += __fmul_rn(s_wt[K], sh);
                __stcg(a.ypair + 16 * tt + tid, xres[16 * tt + tid] + acc);
            }
            if (lane == 0 && issued < nS) { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); issue(issued); }
            if (issued < nS) issued++;
            ok = __syncthreads_and(ok);
            if (tid == 0 && pass + 1 < n4) { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); issue_shared(pass + 1); }
            if (pass + 1 < n4) sh_inflight = worker && (pass + 1) * wgrid + b < U4;
        }
        S0 += nS;
        if (!__syncthreads_and(ok) || !(ok = grid_barrier())) { ok = false; break; }
        // ---- P5: the new residual row (every CTA its own copy), rmsnorm + split for the next layer ----
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int k0 = 1024 * h + 4 * tid;
            const float4 acc = __ldcg(reinterpret_cast<const float4*>(a.ypair + k0));
            *reinterpret_cast<float4*>(xres + k0) = acc;
            v[4 * h] = acc.x; v[4 * h + 1] = acc.y; v[4 * h + 2] = acc.z; v[4 * h + 3] = acc.w;
        }
        __syncthreads();   // part[] of norm_split_row and xn / xcol are free: every warp is past P1 and P3 of this layer
        if (l + 1 < a.n_layers) norm_split_row<F16>(v, xn, reinterpret_cast<uint16_t*>(xcol), 1e-6f, DS_XCOL / 2);
        asm volatile("cp.async.wait_all;" ::: "memory");   // the next layer's router rows and slot table
        __syncthreads();
        if (l + 1 < a.n_layers) x_sums();
    }
    // leave: no copy may still be in flight into this CTA's shared memory
    if (!ok) {
        for (int s = consumed; s < issued; s++)
            if (slice_src(s)) wait_slice(s);
        if (sh_inflight) mbar_wait(smem_u32(&shbar), sh_phase, a.err, DS_ERR_COPY);
        return;
    }
    if (b == 0) {
#pragma unroll
        for (int h = 0; h < 2; h++) *reinterpret_cast<float4*>(a.x_out + 1024 * h + 4 * tid) = *reinterpret_cast<const float4*>(xres + 1024 * h + 4 * tid);
    }
}

// Self-test of the grid barrier's time-out: a grid of ONE CTA arrives at a barrier that expects two arrivals.
__global__ void selftest_grid_barrier_timeout_k(unsigned* sync, int* err, int limit, int* result) {
    if (threadIdx.x == 0) *result = ds_barrier_arrive_wait(sync, 2u, err, limit) ? 1 : 0;
}

}  // namespace moexb
