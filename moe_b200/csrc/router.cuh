// Router kernels: logits in a pinned fp32 summation order, softmax + top-K selection, pair grouping by expert.
#pragma once
#include "common.cuh"

namespace moexb {

__device__ __forceinline__ float4 ld_w4(const float* W, size_t k) { return __ldg(reinterpret_cast<const float4*>(W + k)); }
__device__ __forceinline__ float4 ld_w4(const __half* W, size_t k) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(W + k));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// y[r][o] = W[o] . x[r]. One warp per (row r, output o): lane j accumulates elements 128c+4j .. 128c+4j+3 for
// c = 0, 1, .. with fused multiply-adds in ascending order, then a xor-butterfly (16, 8, 4, 2, 1) adds the 32 partial
// sums. The CPU oracle follows the same order, so the logits - and with them the selected experts - agree bit for bit.
// Stands behind gemv_f16_k (kernels.cuh:73-91). grid (ceil(O / WARPS), rows).
template <typename WT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) gemv_rows_k(const WT* __restrict__ W, const float* __restrict__ x,
                                                          float* __restrict__ y, int I, int O) {
    const int o = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (o >= O) return;
    const float* xr = x + (size_t)blockIdx.y * I;
    const WT* wr = W + (size_t)o * I;
    float acc = 0.f;
    constexpr int U = 16;  // loads of U steps are in flight before the first multiply-add; the summation order is unchanged
    auto steps = [&](int c0, const float4 (&w)[U]) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (c0 + u < I / 128) v[u] = __ldg(reinterpret_cast<const float4*>(xr + 128 * (c0 + u) + 4 * lane));
#pragma unroll
        for (int u = 0; u < U; u++)
            if (c0 + u < I / 128) { acc = fmaf(w[u].x, v[u].x, acc); acc = fmaf(w[u].y, v[u].y, acc); acc = fmaf(w[u].z, v[u].z, acc); acc = fmaf(w[u].w, v[u].w, acc); }
    };
    {   // the weights of the first U steps do not depend on the kernel before this one: they are requested before the wait
        float4 w[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (u < I / 128) w[u] = ld_w4(wr, (size_t)128 * u + 4 * lane);
        pdl_wait();
        pdl_trigger();
        steps(0, w);
    }
    for (int c0 = U; c0 < I / 128; c0 += U) {
        float4 w[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (c0 + u < I / 128) w[u] = ld_w4(wr, (size_t)128 * (c0 + u) + 4 * lane);
        steps(c0, w);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)blockIdx.y * O + o] = acc;
}

// The same result for many rows (a batch or a prefill chunk). A block stages TR activation rows in shared memory and its
// WARPS warps each own TO outputs; a lane still holds elements 128c+4j..4j+3 of every dot product, so every
// (row, output) sum is formed in exactly the order of gemv_rows_k and the two kernels agree bit for bit.
// grid (ceil(O / (WARPS*TO)), ceil(rows / TR)); dynamic shared memory TR * I floats.
template <typename WT, int WARPS, int TO, int TR>
__global__ void __launch_bounds__(WARPS * 32) gemm_rows_k(const WT* __restrict__ W, const float* __restrict__ x,
                                                          float* __restrict__ y, int I, int O, int rows) {
    extern __shared__ __align__(16) float xsm[];  // [TR][I]
    const int r0 = blockIdx.y * TR, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    for (int i = threadIdx.x * 4; i < TR * I; i += WARPS * 128) {
        const int r = min(r0 + i / I, rows - 1);
        *reinterpret_cast<float4*>(xsm + i) = __ldg(reinterpret_cast<const float4*>(x + (size_t)r * I + i % I));
    }
    __syncthreads();
    const int o0 = (blockIdx.x * WARPS + (threadIdx.x >> 5)) * TO;
    if (o0 >= O) return;
    float acc[TR][TO];
#pragma unroll
    for (int r = 0; r < TR; r++)
#pragma unroll
        for (int o = 0; o < TO; o++) acc[r][o] = 0.f;
    float4 wn[TO];  // the next step's weights are loaded while this step's products run
#pragma unroll
    for (int o = 0; o < TO; o++) wn[o] = ld_w4(W + (size_t)min(o0 + o, O - 1) * I, (size_t)4 * lane);
    for (int c = 0; c < I / 128; c++) {
        float4 w[TO];
#pragma unroll
        for (int o = 0; o < TO; o++) w[o] = wn[o];
        if (c + 1 < I / 128) {
#pragma unroll
            for (int o = 0; o < TO; o++) wn[o] = ld_w4(W + (size_t)min(o0 + o, O - 1) * I, (size_t)128 * (c + 1) + 4 * lane);
        }
#pragma unroll
        for (int r = 0; r < TR; r++) {
            const float4 v = *reinterpret_cast<const float4*>(xsm + r * I + 128 * c + 4 * lane);
#pragma unroll
            for (int o = 0; o < TO; o++) {
                float a = acc[r][o];
                a = fmaf(w[o].x, v.x, a); a = fmaf(w[o].y, v.y, a); a = fmaf(w[o].z, v.z, a); a = fmaf(w[o].w, v.w, a);
                acc[r][o] = a;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < TR; r++)
#pragma unroll
        for (int o = 0; o < TO; o++) {
            const float sum = warp_sum(acc[r][o]);
            if (lane == 0 && r0 + r < rows && o0 + o < O) y[(size_t)(r0 + r) * O + o0 + o] = sum;
        }
}

// Softmax over E logits and the K largest by one warp (kernels.cuh:373-406 does it with a block per token).
// Lane l holds logits l, l+32, ..; each round every lane offers its best remaining value as an order-preserving
// integer key, one warp reduction finds the largest key and a second the lowest index that holds it (ties go to the
// lower index), and the winner is struck from its owner's mask. Selection compares logits (softmax is monotone). NaN
// logits count as -inf. Optional decode outputs: slots_out / wts_out [K+1] = the selected experts' blob pointers and
// weights followed by the shared expert with weight sigmoid(logits[E]); dsubs / dpairs / dnsub = the same K+1 experts as
// one-pair sub-items for the streaming kernels (T = 1).
struct TopkOut {
    int* idx; float* w;
    const uint8_t* const* slot_table; const uint8_t** slots_out; float* wts_out;
    moexb_pair_item* dsubs; moexb_pair* dpairs; int* dnsub;
    // expert parallelism (ep.cuh): the warp that selected a token's experts also sends the token to the peers - ids and
    // weights to every rank, the activation row (ep_row_bytes at [token] of the exchange buffer's row area) to the ranks that
    // hold one of the selected experts - and the block then raises the tokens' dispatch flags
    const EpDevice* ep = nullptr; int ep_row_bytes = 0; unsigned ep_phase = 0; const unsigned* ep_step = nullptr;
};
__device__ __forceinline__ unsigned f2key(float v) { const unsigned u = __float_as_uint(v); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }
__device__ __forceinline__ float key2f(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// CG: the logits were written by other blocks of the same launch - read them past L1.
template <int NJ, bool CG>
__device__ __forceinline__ void topk_token(const float* __restrict__ l, int t, int E, int K, int norm, int lane, const TopkOut& o) {
    const int nj = E >> 5;  // <= NJ
    float v[NJ];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        v[j] = -INFINITY;
        if (j < nj) { const float a = CG ? __ldcg(l + lane + 32 * j) : l[lane + 32 * j]; v[j] = a != a ? -INFINITY : a; }
        m = fmaxf(m, v[j]);
    }
    const float gate_logit = (o.slots_out && lane == K) ? (CG ? __ldcg(l + E) : l[E]) : 0.f;
#pragma unroll
    for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    unsigned key[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) key[j] = j < nj ? f2key(v[j]) : 0u;  // 0 = not a candidate (below every real key)
    // K rounds, each two warp reductions: the largest remaining key, then the lowest index that holds it. Between them a lane
    // only has to know its own best remaining key, kept by a tree of comparisons that every lane runs without branching (the
    // lower slot wins among equals). The softmax denominator is summed inside the rounds, where the reductions leave issue
    // slots free: one term per round, the rest after the last one.
    int mine_i = 0;
    unsigned mine_key = 0u;
    unsigned bk; int bj;
    auto best = [&] {   // (bk, bj) = the lane's largest key and its lowest slot
        unsigned k2[NJ / 2 > 0 ? NJ / 2 : 1]; int j2[NJ / 2 > 0 ? NJ / 2 : 1];
#pragma unroll
        for (int j = 0; j < NJ / 2; j++) { const bool l = key[2 * j] >= key[2 * j + 1]; k2[j] = l ? key[2 * j] : key[2 * j + 1]; j2[j] = l ? 2 * j : 2 * j + 1; }
#pragma unroll
        for (int w = NJ / 2; w > 1; w >>= 1)
#pragma unroll
            for (int j = 0; j < w / 2; j++) { const bool l = k2[2 * j] >= k2[2 * j + 1]; k2[j] = l ? k2[2 * j] : k2[2 * j + 1]; j2[j] = l ? j2[2 * j] : j2[2 * j + 1]; }
        bk = k2[0]; bj = j2[0];
    };
    best();
    float sum = 0.f;
    for (int k = 0; k < K; k++) {
        const unsigned top = __reduce_max_sync(0xffffffffu, bk);
        const unsigned win = __reduce_min_sync(0xffffffffu, bk == top ? (unsigned)(lane + 32 * bj) : 0x7fffffffu);
        const bool won = (int)(win & 31) == lane;
#pragma unroll
        for (int j = 0; j < NJ; j++) if (won && j == (int)(win >> 5)) key[j] = 0u;
        best();
        if (lane == k) { mine_key = top; mine_i = (int)win; }
#pragma unroll
        for (int j = 0; j < NJ; j++) if (j == k && j < nj) sum += expf(v[j] - m);
    }
#pragma unroll
    for (int j = 0; j < NJ; j++) if (j >= K && j < nj) sum += expf(v[j] - m);
    sum = warp_sum(sum);
    // the K probabilities at once, and their sum in selection order
    float mine = 0.f, total = 0.f;  // lane k keeps the k-th probability
    if (lane < K) mine = expf(key2f(mine_key) - m) / sum;
    for (int k = 0; k < K; k++) total += __shfl_sync(0xffffffffu, mine, k);
    if (lane < K) {
        const float wk = norm ? mine / total : mine;
        o.idx[(size_t)t * K + lane] = mine_i;
        o.w[(size_t)t * K + lane] = wk;
        if (o.slots_out) { o.slots_out[(size_t)t * (K + 1) + lane] = o.slot_table[mine_i]; o.wts_out[(size_t)t * (K + 1) + lane] = wk; }
        if (o.dsubs) { o.dsubs[lane] = {o.slot_table[mine_i], lane, 1}; o.dpairs[lane] = {0, lane, wk}; }  // one token: expert k = sub-item k
    }
    if (o.slots_out && lane == K) {
        const float gate = 1.f / (1.f + expf(-gate_logit));
        o.slots_out[(size_t)t * (K + 1) + K] = o.slot_table[E];
        o.wts_out[(size_t)t * (K + 1) + K] = gate;
        if (o.dsubs) { o.dsubs[K] = {o.slot_table[E], K, 1}; o.dpairs[K] = {0, K, gate}; o.dnsub[0] = K + 1; o.dnsub[1] = 0; }
    }
    if (o.ep) {
        const EpDevice& ep = *o.ep;
        const int rank = ep.g.rank, ta = ep.g.tok0[rank] + t;   // t counts from this rank's first token
        unsigned need = 0;
        if (lane < K)
            for (int s = 0; s < ep.g.world; s++) if (mine_i >= ep.g.exp0[s] && mine_i < ep.g.exp0[s + 1]) need = 1u << s;
        need = __reduce_or_sync(0xffffffffu, need);
        const float wk = norm ? mine / total : mine;
        // the row (at most 8 KB = 16 x 16 bytes per lane) is read once, every load in flight before the first store
        const uint4* src = reinterpret_cast<const uint4*>(ep.p.base[rank] + ep.lay.xs + (size_t)ta * o.ep_row_bytes);
        const int n16 = o.ep_row_bytes / 16;
        uint4 v[16];
        if (need & ~(1u << rank)) {
#pragma unroll
            for (int j = 0; j < 16; j++) if (lane + 32 * j < n16) v[j] = src[lane + 32 * j];
        }
        for (int d = 0; d < ep.g.world; d++) {
            if (d == rank) continue;
            uint8_t* db = ep.p.base[d];
            if (lane < K) {
                reinterpret_cast<int*>(db + ep.lay.idx)[(size_t)ta * K + lane] = mine_i;
                reinterpret_cast<float*>(db + ep.lay.w)[(size_t)ta * K + lane] = wk;
            }
            if (need >> d & 1) {
                uint4* out = reinterpret_cast<uint4*>(db + ep.lay.xs + (size_t)ta * o.ep_row_bytes);
#pragma unroll
                for (int j = 0; j < 16; j++) if (lane + 32 * j < n16) out[lane + 32 * j] = v[j];
            }
        }
    }
}

// After the warps of a block have sent tokens [t_first, t_first + n) of this rank (topk_token with o.ep): one system-scope
// fence by one thread behind the block barrier, then the tokens' dispatch flags on every peer.
__device__ __forceinline__ void ep_raise_dispatch_flags(const TopkOut& o, int t_first, int n) {
    if (!o.ep) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        const EpDevice& ep = *o.ep;
        const unsigned value = *o.ep_step * EP_PHASES + o.ep_phase;
        __threadfence_system();
        for (int d = 0; d < ep.g.world; d++) {
            if (d == ep.g.rank) continue;
            unsigned* flags = reinterpret_cast<unsigned*>(ep.p.base[d] + ep.lay.flag_a) + ep.g.tok0[ep.g.rank] + t_first;
            for (int i = 0; i < n; i++) st_relaxed_sys(flags + i, value);
        }
    }
}

// One warp per token.
template <int WARPS, int NJ>
__global__ void __launch_bounds__(WARPS * 32) router_topk_k(const float* __restrict__ logits, int E, int K, int norm, int ld, int T, const TopkOut o) {
    const int t = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_trigger();
    if (t >= T) return;
    topk_token<NJ, false>(logits + (size_t)t * ld, t, E, K, norm, lane, o);
}

// Whether this block is the last of `expected` blocks to reach this point for counter *cnt (every block calls it once,
// after its global writes); the last one sees the writes of all the others and resets the counter for the next launch.
__device__ __forceinline__ bool last_block_done(int* cnt, int expected) {
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();   // one fence per block: the barrier orders the block's writes before it, and it is cumulative
        const int ticket = atomicAdd(cnt, 1);
        s_last = ticket == expected - 1;
        if (s_last) { *cnt = 0; __threadfence(); }
    }
    __syncthreads();
    return s_last;
}

// Router logits and top-K selection of a few tokens in one launch: gemv_rows_k's grid (ceil(O / WARPS) blocks per
// token, O = E + 1), and the last block of a token to finish selects that token's experts - no second launch, no wait:
// the block that comes last simply does the extra work. done[t] must be zero before the first launch.
template <typename WT, int WARPS, int NJ>
__global__ void __launch_bounds__(WARPS * 32) route_gemv_k(const WT* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int I,
                                                           int E, int K, int norm, int* __restrict__ done, const TopkOut o) {
    const int O = E + 1, t = blockIdx.y;
    const int out = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const float* xr = x + (size_t)t * I;
    const WT* wr = W + (size_t)min(out, O - 1) * I;
    float acc = 0.f;
    constexpr int U = 16;
    auto steps = [&](int c0, const float4 (&w)[U]) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (c0 + u < I / 128) v[u] = __ldg(reinterpret_cast<const float4*>(xr + 128 * (c0 + u) + 4 * lane));
#pragma unroll
        for (int u = 0; u < U; u++)
            if (c0 + u < I / 128) { acc = fmaf(w[u].x, v[u].x, acc); acc = fmaf(w[u].y, v[u].y, acc); acc = fmaf(w[u].z, v[u].z, acc); acc = fmaf(w[u].w, v[u].w, acc); }
    };
    {
        float4 w[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (u < I / 128) w[u] = ld_w4(wr, (size_t)128 * u + 4 * lane);
        pdl_wait();
        pdl_trigger();
        steps(0, w);
    }
    for (int c0 = U; c0 < I / 128; c0 += U) {
        float4 w[U];
#pragma unroll
        for (int u = 0; u < U; u++)
            if (c0 + u < I / 128) w[u] = ld_w4(wr, (size_t)128 * (c0 + u) + 4 * lane);
        steps(c0, w);
    }
    acc = warp_sum(acc);
    if (lane == 0 && out < O) y[(size_t)t * O + out] = acc;
    if (!last_block_done(done + t, gridDim.x)) return;
    if (threadIdx.x < 32) topk_token<NJ, true>(y + (size_t)t * O, t, E, K, norm, lane, o);
    ep_raise_dispatch_flags(o, t, 1);
}

// The same for a batch: gemm_rows_k's tiling (a block stages TR token rows in shared memory, each of its WARPS warps owns
// TO outputs, every dot product in gemv_rows_k's summation order) with the weights of U steps requested at a time and
// the next U already in flight; the last block of a token tile to finish selects the experts of its TR tokens (warp r
// takes tokens r, r + WARPS, ..). grid (ceil((E + 1) / (WARPS * TO)), ceil(T / TR)); dynamic shared memory TR * I floats;
// done[tile] zero before the first launch.
template <typename WT, int WARPS, int TO, int TR, int NJ>
__global__ void __launch_bounds__(WARPS * 32) route_gemm_k(const WT* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int I,
                                                           int E, int K, int norm, int T, int* __restrict__ done, const TopkOut o) {
    extern __shared__ __align__(16) float xsm[];  // [TR][I]
    // steps per batch of weights: the small tile takes 8 (half of I = 2048) - the first batch, requested before the wait,
    // arrives while the kernel before this one still runs (all 16 at once would spill)
    constexpr int U = TO <= 2 ? 8 : 4;
    const int O = E + 1, r0 = blockIdx.y * TR, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o0 = (blockIdx.x * WARPS + warp) * TO;
    const WT* wr[TO];
#pragma unroll
    for (int i = 0; i < TO; i++) wr[i] = W + (size_t)min(o0 + i, O - 1) * I;
    float4 wn[TO][U];  // the weights of the next U steps
    auto load_w = [&](int c0) {
#pragma unroll
        for (int i = 0; i < TO; i++)
#pragma unroll
            for (int u = 0; u < U; u++)
                if (c0 + u < I / 128) wn[i][u] = ld_w4(wr[i], (size_t)128 * (c0 + u) + 4 * lane);
    };
    load_w(0);  // weights do not depend on the kernel before this one
    pdl_wait();
    pdl_trigger();
    for (int r = 0; r < TR; r++) {   // the tile's token rows: 16-byte asynchronous copies, all in flight at once
        const float* src = x + (size_t)min(r0 + r, T - 1) * I;
        for (int c = threadIdx.x * 4; c < I; c += WARPS * 128) cp_async16(smem_u32(xsm + r * I + c), src + c);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    float acc[TR][TO];
#pragma unroll
    for (int r = 0; r < TR; r++)
#pragma unroll
        for (int i = 0; i < TO; i++) acc[r][i] = 0.f;
    for (int c0 = 0; c0 < I / 128; c0 += U) {
        float4 w[TO][U];
#pragma unroll
        for (int i = 0; i < TO; i++)
#pragma unroll
            for (int u = 0; u < U; u++) w[i][u] = wn[i][u];
        if (c0 + U < I / 128) load_w(c0 + U);
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (c0 + u >= I / 128) break;
#pragma unroll
            for (int r = 0; r < TR; r++) {
                const float4 v = *reinterpret_cast<const float4*>(xsm + r * I + 128 * (c0 + u) + 4 * lane);
#pragma unroll
                for (int i = 0; i < TO; i++) {
                    float a = acc[r][i];
                    a = fmaf(w[i][u].x, v.x, a); a = fmaf(w[i][u].y, v.y, a); a = fmaf(w[i][u].z, v.z, a); a = fmaf(w[i][u].w, v.w, a);
                    acc[r][i] = a;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < TR; r++)
#pragma unroll
        for (int i = 0; i < TO; i++) {
            const float sum = warp_sum(acc[r][i]);
            if (lane == 0 && r0 + r < T && o0 + i < O) y[(size_t)(r0 + r) * O + o0 + i] = sum;
        }
    if (!last_block_done(done + blockIdx.y, gridDim.x)) return;
    for (int r = warp; r < TR && r0 + r < T; r += WARPS) topk_token<NJ, true>(y + (size_t)(r0 + r) * O, r0 + r, E, K, norm, lane, o);
    ep_raise_dispatch_flags(o, r0, min(TR, T - r0));
}

// The same for a prefill chunk, register-tiled. A block of 8 warps owns 32 tokens x 16 outputs; warp (wm, wn) the 8 tokens
// 8*wm.. and the 8 outputs 8*wn.., every lane the same 4 of each 128 inputs as in gemv_rows_k, so a lane holds 64 partial
// sums and each (token, output) sum is formed in the pinned order. Token rows and weight rows come through shared memory in
// chunks of 256 inputs (cp.async, two stages; two blocks per SM): per 128 inputs a warp reads 16 x 16 bytes per lane and does 256 fused
// multiply-adds, which makes the kernel FMA-bound where route_gemm_k is bound by re-reading the weights from L2. The last
// block of a token tile selects the experts of its 32 tokens. grid (ceil((E + 1) / 16), ceil(T / 32)); I = 2048.
constexpr int RG2_TM = 32, RG2_TN = 16, RG2_KC = 256;
template <typename WT> constexpr int rg2_stage_bytes() { return RG2_TM * RG2_KC * 4 + RG2_TN * RG2_KC * (int)sizeof(WT); }
template <typename WT, int NJ>
__global__ void __launch_bounds__(256, 2) route_gemm2_k(const WT* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int E, int K,
                                                     int norm, int T, int* __restrict__ done, const TopkOut o) {
    constexpr int I = EH, NCH = I / RG2_KC, STAGE = rg2_stage_bytes<WT>();
    extern __shared__ __align__(16) uint8_t rsm[];   // 2 stages x ([32 tokens][512] f32 | [16 outputs][512] WT)
    const int O = E + 1, r0 = blockIdx.y * RG2_TM, o0 = blockIdx.x * RG2_TN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp >> 1, wn = warp & 1;
    auto fill_w = [&](int ch) {
        uint8_t* ws = rsm + (ch & 1) * STAGE + RG2_TM * RG2_KC * 4;
        constexpr int PER_ROW = RG2_KC * (int)sizeof(WT) / 16;   // 16-byte pieces per row chunk
        for (int i = tid; i < RG2_TN * PER_ROW; i += 256) {
            const int r = i / PER_ROW, c = i % PER_ROW;
            cp_async16(smem_u32(ws + (size_t)i * 16), reinterpret_cast<const uint8_t*>(W + (size_t)min(o0 + r, O - 1) * I + ch * RG2_KC) + c * 16);
        }
    };
    auto fill_x = [&](int ch) {
        uint8_t* xs = rsm + (ch & 1) * STAGE;
        constexpr int PER_ROW = RG2_KC * 4 / 16;
        for (int i = tid; i < RG2_TM * PER_ROW; i += 256) {
            const int r = i / PER_ROW, c = i % PER_ROW;
            cp_async16(smem_u32(xs + (size_t)i * 16), reinterpret_cast<const uint8_t*>(x + (size_t)min(r0 + r, T - 1) * I + ch * RG2_KC) + c * 16);
        }
    };
    fill_w(0);   // weights do not depend on the kernel before this one
    pdl_wait();
    pdl_trigger();
    fill_x(0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
    for (int ch = 0; ch < NCH; ch++) {
        if (ch + 1 < NCH) { fill_w(ch + 1); fill_x(ch + 1); }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const float* xs = reinterpret_cast<const float*>(rsm + (ch & 1) * STAGE) + (size_t)(8 * wm) * RG2_KC;
        const WT* ws = reinterpret_cast<const WT*>(rsm + (ch & 1) * STAGE + RG2_TM * RG2_KC * 4) + (size_t)(8 * wn) * RG2_KC;
#pragma unroll
        for (int c = 0; c < RG2_KC / 128; c++) {
            float4 wv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if constexpr (sizeof(WT) == 4) wv[j] = *reinterpret_cast<const float4*>(ws + (size_t)j * RG2_KC + 128 * c + 4 * lane);
                else {
                    const uint2 h = *reinterpret_cast<const uint2*>(ws + (size_t)j * RG2_KC + 128 * c + 4 * lane);
                    const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&h.x)), q = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
                    wv[j] = make_float4(p.x, p.y, q.x, q.y);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 v = *reinterpret_cast<const float4*>(xs + (size_t)i * RG2_KC + 128 * c + 4 * lane);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float a = acc[i][j];
                    a = fmaf(wv[j].x, v.x, a); a = fmaf(wv[j].y, v.y, a); a = fmaf(wv[j].z, v.z, a); a = fmaf(wv[j].w, v.w, a);
                    acc[i][j] = a;
                }
            }
        }
        __syncthreads();   // the stage is refilled by the copies of chunk ch + 2
    }
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float sum = warp_sum(acc[i][j]);
            const int r = r0 + 8 * wm + i, oo = o0 + 8 * wn + j;
            if (lane == 0 && r < T && oo < O) y[(size_t)r * O + oo] = sum;
        }
    if (!last_block_done(done + blockIdx.y, gridDim.x)) return;
    for (int r = warp; r < RG2_TM && r0 + r < T; r += 8) topk_token<NJ, true>(y + (size_t)(r0 + r) * O, r0 + r, E, K, norm, lane, o);
    ep_raise_dispatch_flags(o, r0, min(RG2_TM, T - r0));
}

// ---- pair grouping: bucket the T*K (token, rank) pairs by expert (moex.cu:1466-1486; kernels.cuh:1030-1045) ----------

// counts[e] = number of pairs that selected expert e. One warp per expert.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) group_count_k(const int* __restrict__ idx, int n, int E, int* __restrict__ counts) {
    const int e = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= E) return;
    int c = 0;
    for (int p = lane; p < n; p += 32) c += __ldg(idx + p) == e;
#pragma unroll
    for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (lane == 0) counts[e] = c;
}

// Items in ascending expert id over the experts that are held (slot_table[e] != null) and selected; the pairs of an
// expert in token order, p = t*K + rank. Every block rebuilds the (tiny) exclusive scan over experts, then one warp per
// expert walks the pair list once and writes its matches in order. Optional shared expert: one more item holding every
// token, p = T*K + t, w = sigmoid(gate logit of t). E <= 1024.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) group_scatter_k(const int* __restrict__ idx, const float* __restrict__ w, int T, int K, int E,
                                                              const uint8_t* const* __restrict__ slot_table, const int* __restrict__ counts,
                                                              moexb_pair_item* __restrict__ items, moexb_pair* __restrict__ pairs,
                                                              int* __restrict__ nitems, const float* __restrict__ gate_logits, int gl_stride) {
    __shared__ int start[1024], item_of[1024];
    __shared__ int s_ni, s_np;
    if (threadIdx.x == 0) {
        int ni = 0, np = 0;
        for (int e = 0; e < E; e++) {
            const int c = slot_table[e] ? counts[e] : 0;
            start[e] = np; item_of[e] = c ? ni : -1;
            np += c; ni += c != 0;
        }
        s_ni = ni; s_np = np;
    }
    __syncthreads();
    const int n = T * K, lane = threadIdx.x & 31;
    const int e = blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (e < E && item_of[e] >= 0) {
        int at = start[e];
        if (lane == 0) items[item_of[e]] = {slot_table[e], at, counts[e]};
        for (int p0 = 0; p0 < n; p0 += 32) {
            const int p = p0 + lane;
            const bool hit = p < n && __ldg(idx + p) == e;
            const unsigned b = __ballot_sync(0xffffffffu, hit);
            if (hit) pairs[at + __popc(b & ((1u << lane) - 1))] = {p / K, p, __ldg(w + p)};
            at += __popc(b);
        }
    }
    if (blockIdx.x == 0) {
        if (gate_logits && slot_table[E]) {
            if (threadIdx.x == 0) { items[s_ni] = {slot_table[E], s_np, T}; *nitems = s_ni + 1; }
            for (int t = threadIdx.x; t < T; t += blockDim.x)
                pairs[s_np + t] = {t, n + t, 1.f / (1.f + expf(-gate_logits[(size_t)t * gl_stride]))};
        } else if (threadIdx.x == 0) *nitems = s_ni;
    }
}

}  // namespace moexb
