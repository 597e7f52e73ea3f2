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
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; j++) if (j < nj) sum += expf(v[j] - m);
    sum = warp_sum(sum);
    unsigned key[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) key[j] = j < nj ? f2key(v[j]) : 0u;  // 0 = not a candidate (below every real key)
    float mine = 0.f, total = 0.f;  // lane k keeps the k-th probability
    int mine_i = 0;
    for (int k = 0; k < K; k++) {
        unsigned bk = 0; int bj = 0;
#pragma unroll
        for (int j = 0; j < NJ; j++) if (key[j] > bk) { bk = key[j]; bj = j; }
        const unsigned top = __reduce_max_sync(0xffffffffu, bk);
        const unsigned win = __reduce_min_sync(0xffffffffu, bk == top ? (unsigned)(lane + 32 * bj) : 0x7fffffffu);
        if ((int)(win & 31) == lane) {
#pragma unroll
            for (int j = 0; j < NJ; j++) if (j == (int)(win >> 5)) key[j] = 0u;
        }
        const float p = expf(key2f(top) - m) / sum;
        total += p;
        if (lane == k) { mine = p; mine_i = (int)win; }
    }
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
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(cnt, 1);
        s_last = ticket == expected - 1;
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (s_last) __threadfence();
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
    constexpr int U = 4;
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
    for (int i = threadIdx.x * 4; i < TR * I; i += WARPS * 128) {
        const int r = min(r0 + i / I, T - 1);
        *reinterpret_cast<float4*>(xsm + i) = __ldg(reinterpret_cast<const float4*>(x + (size_t)r * I + i % I));
    }
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

// Exclusive prefix sums of N per-thread values over a block of 256 threads; totals returned through tot[].
template <int N>
__device__ __forceinline__ void block_scan_256(int (&v)[N], int (&tot)[N]) {
    __shared__ int ws[N][8];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int inc[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        inc[i] = v[i];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, inc[i], o); if (lane >= o) inc[i] += u; }
        if (lane == 31) ws[i][w] = inc[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < N; i++) {
        int before = 0, all = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) { const int x = ws[i][j]; all += x; if (j < w) before += x; }
        v[i] = inc[i] - v[i] + before;
        tot[i] = all;
    }
}

// Grouping and planning in one launch (the work of group_count_k + group_scatter_k, plus the sub-items of at most MAXP
// pairs that the streaming kernels walk). Every block builds the per-expert histogram of the T*K pairs in shared memory
// and scans it; then one warp per expert writes that expert's item, its sub-items and its pairs in token order.
// Sub-items of more than MAXP / 2 pairs ("wide") come first in subs[], the others after them, and nsub[1] receives the
// number of wide ones: a pass over a wide sub-item costs the streaming kernels more, and with the two kinds apart a kernel
// can split the work evenly from nsub[0] and nsub[1] alone. (An expert's sub-items are all wide except possibly its last.)
// Optional shared expert as in group_scatter_k, for the tokens [sh0, sh1). E <= 1024; 256 threads; grid ceil(E / 8).
__host__ __device__ constexpr int plan_wide(int c, int maxp) { return c / maxp + (c % maxp > maxp / 2); }
__host__ __device__ constexpr int plan_narrow(int c, int maxp) { return c % maxp > 0 && c % maxp <= maxp / 2; }
template <int MAXP>
__global__ void __launch_bounds__(256) group_plan_k(const int* __restrict__ idx, const float* __restrict__ w, int T, int K, int E,
                                                    const uint8_t* const* __restrict__ slot_table, moexb_pair_item* __restrict__ items,
                                                    moexb_pair* __restrict__ pairs, int* __restrict__ nitems, moexb_pair_item* __restrict__ subs,
                                                    int* __restrict__ nsub, const float* __restrict__ gate_logits, int gl_stride,
                                                    int sh0, int sh1) {
    __shared__ int cnt[1024], start[1024], item_of[1024], wide_at[1024], narrow_at[1024];
    __shared__ int s_tot[4];
    const int n = T * K, tid = threadIdx.x, lane = tid & 31;
    for (int e = tid; e < E; e += 256) cnt[e] = 0;
    __syncthreads();
    pdl_wait();
    pdl_trigger();
    for (int p = tid; p < n; p += 256) atomicAdd(&cnt[__ldg(idx + p)], 1);
    __syncthreads();
    {
        const int per = (E + 255) / 256, e0 = tid * per;
        int c[4], v[4] = {0, 0, 0, 0}, tot[4];
        for (int i = 0; i < per; i++) {
            const int e = e0 + i;
            c[i] = (e < E && slot_table[e]) ? cnt[e] : 0;
            v[0] += c[i]; v[1] += c[i] != 0; v[2] += plan_wide(c[i], MAXP); v[3] += plan_narrow(c[i], MAXP);
        }
        block_scan_256<4>(v, tot);
        for (int i = 0; i < per; i++) {
            const int e = e0 + i;
            if (e < E) {
                start[e] = v[0]; item_of[e] = c[i] ? v[1] : -1; wide_at[e] = v[2]; narrow_at[e] = v[3];
                cnt[e] = c[i];
            }
            v[0] += c[i]; v[1] += c[i] != 0; v[2] += plan_wide(c[i], MAXP); v[3] += plan_narrow(c[i], MAXP);
        }
        if (tid == 0) { s_tot[0] = tot[0]; s_tot[1] = tot[1]; s_tot[2] = tot[2]; s_tot[3] = tot[3]; }
    }
    __syncthreads();
    const bool with_shared = gate_logits && slot_table[E] && sh1 > sh0;
    const int Ts = with_shared ? sh1 - sh0 : 0;
    const int nw = s_tot[2] + plan_wide(Ts, MAXP);   // all wide sub-items: the routed experts', then the shared expert's
    const int e = blockIdx.x * 8 + (tid >> 5);
    if (e < E && item_of[e] >= 0) {
        const uint8_t* slot = slot_table[e];
        int at = start[e];
        const int c = cnt[e], cw = plan_wide(c, MAXP);
        if (lane == 0) items[item_of[e]] = {slot, at, c};
        for (int j = lane; j * MAXP < c; j += 32)
            subs[j < cw ? wide_at[e] + j : nw + narrow_at[e]] = {slot, at + j * MAXP, min(MAXP, c - j * MAXP)};
        for (int p0 = 0; p0 < n; p0 += 32) {
            const int p = p0 + lane;
            const bool hit = p < n && __ldg(idx + p) == e;
            const unsigned b = __ballot_sync(0xffffffffu, hit);
            if (hit) pairs[at + __popc(b & ((1u << lane) - 1))] = {p / K, p, __ldg(w + p)};
            at += __popc(b);
        }
    }
    if (blockIdx.x == 0) {
        const int np = s_tot[0], ni = s_tot[1], ns = nw + s_tot[3];  // ns: where the shared expert's narrow sub-item goes
        if (with_shared) {
            // the shared expert for tokens [sh0, sh1) (all of them on one GPU; a slice per rank under expert parallelism)
            const uint8_t* slot = slot_table[E];
            const int cw = plan_wide(Ts, MAXP);
            if (tid == 0) { items[ni] = {slot, np, Ts}; *nitems = ni + 1; nsub[0] = ns + plan_narrow(Ts, MAXP); nsub[1] = nw; }
            for (int t = tid; t < Ts; t += 256) pairs[np + t] = {sh0 + t, n + sh0 + t, 1.f / (1.f + expf(-gate_logits[(size_t)(sh0 + t) * gl_stride]))};
            for (int j = tid; j * MAXP < Ts; j += 256) subs[j < cw ? s_tot[2] + j : ns] = {slot, np + j * MAXP, min(MAXP, Ts - j * MAXP)};
        } else if (tid == 0) { *nitems = ni; nsub[0] = ns; nsub[1] = nw; }
    }
}

}  // namespace moexb
