// Expert parallelism over the GPUs of one NVLink node: the token all-to-all done by the path's own kernels over peer memory.
//
// Rank r of R holds the routed experts [exp0[r], exp0[r+1]) of every layer (router and shared expert replicated) and OWNS
// the tokens [tok0[r], tok0[r+1]): it alone keeps their residual rows, normalises and routes them, runs the shared expert
// for them and produces their outputs. Every rank has one "exchange buffer" of the same layout, mapped into all the others
// (peer pointers), holding for ALL T tokens the normalised activation rows in the 16-bit split form the expert kernels
// read, the selected expert ids and routing weights, and per source rank one partial output row for each own token.
// One layer on rank r:
//   dispatch  r's routing kernel selects the experts of its own tokens, and the warp that selected a token's experts stores
//             the token's ids and weights into every peer's buffer and its activation row into the buffers of the ranks
//             that hold one of its selected experts (plain st.global through the peer mapping; topk_token in router.cuh);
//             the block then raises the tokens' dispatch flags on every peer;
//   experts   the planner waits for the dispatch flags of all T tokens, groups the (token, expert) pairs of the experts held here, the
//             gate/up and down kernels run as on one GPU (all their reads are local HBM);
//   combine   ep_partial_push_k adds, per token, the weighted rows of the experts held here in router-rank order and stores
//             that ONE partial row into the owner's buffer (only where this rank had a selected expert), then raises the
//             token's combine flag there; ep_combine_norm_k on the owner waits for the token's R combine flags and adds the
//             partial rows in rank order 0..R-1, the shared expert's row and the residual, normalises, and the next
//             layer's dispatch follows.
// A flag is a 32-bit word (dispatch: per token; combine: per source rank and token) holding step * EP_PHASES + layer + 1 of
// the last completed push (monotonic; the
// step counter lives in device memory so that a captured graph can be replayed). Writers order data before flag with
// __threadfence_system() and a release store at system scope; readers poll with acquire loads at system scope and read the
// peer-written data past L1. Every poll loop is bounded: on a time-out the kernel records EP_ERR_* in the context's error
// word and carries on with whatever is in the buffer (always valid ids and finite numbers from an earlier layer), so
// nothing hangs or faults and the host sees the failure in moexb_ctx_status.
// Why a rank can never overwrite data a peer still reads: the owner of a token sends the token's row and ids of layer l+1
// only after its combine of layer l for that token, which waited for the token's combine flag of EVERY rank (raised whether
// or not that rank had a row to send), and a rank raises it only after its planner, gate/up, down and partial-sum kernels of
// layer l are done with the token; the partial rows a rank writes for layer l+1 come after its planner of layer l+1, which
// waited for every token's dispatch flag, which the owner raises after its combine has read the partial rows of layer l.
#pragma once
#include "common.cuh"
#include "stream.cuh"

namespace moexb {

__host__ __device__ inline size_t ep_align(size_t x) { return (x + 255) & ~(size_t)255; }
__host__ inline EpLayout ep_layout(int T, int K, int world) {
    EpLayout l;
    const size_t n_own_max = (T + world - 1) / world;
    size_t at = 0;
    l.xs = at; at = ep_align(at + (size_t)T * 2 * EH * 2);
    l.idx = at; at = ep_align(at + (size_t)T * K * 4);
    l.w = at; at = ep_align(at + (size_t)T * K * 4);
    l.part = at; at = ep_align(at + (size_t)world * n_own_max * EH * 4);
    l.flag_a = at; at = ep_align(at + (size_t)T * 4);
    l.flag_b = at; at = ep_align(at + (size_t)world * n_own_max * 4);
    l.bytes = at;
    return l;
}

__global__ void ep_step_k(unsigned* step) { *step += 1; }

// Combine, sending side. grid T, 256 threads: block t adds the rows ypair[t*K + r] of the ranks r whose expert is held
// here, in rank order (the sum reduce_residual_norm_k forms for a rank's share), and stores the one partial row into the
// token owner's buffer at [this rank][token's place among the owner's tokens]. Tokens none of whose experts are held here
// send nothing; the owner derives the same from the ids.
__global__ void __launch_bounds__(256) ep_partial_push_k(const EpGeom g, const EpPeers p, const EpLayout lay, const float* __restrict__ ypair,
                                                         const unsigned* __restrict__ step, unsigned phase) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, K = g.K;
    const int* idx = reinterpret_cast<const int*>(p.base[g.rank] + lay.idx) + (size_t)t * K;
    unsigned have = 0;
    for (int r = 0; r < K; r++) { const int e = __ldcg(idx + r); if (e >= g.exp0[g.rank] && e < g.exp0[g.rank + 1]) have |= 1u << r; }
    int owner = 0;
    while (t >= g.tok0[owner + 1]) owner++;
    if (have) {
        float* dst = reinterpret_cast<float*>(p.base[owner] + lay.part) + ((size_t)g.rank * g.n_own_max + (t - g.tok0[owner])) * EH;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int k0 = 1024 * h + 4 * threadIdx.x;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int rb = 0; rb < K; rb += 8) {  // eight rows in flight, added in rank order
                float4 y[8];
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (rb + u < K && (have >> (rb + u) & 1)) y[u] = *reinterpret_cast<const float4*>(ypair + ((size_t)t * K + rb + u) * EH + k0);
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (rb + u < K && (have >> (rb + u) & 1)) { acc.x += y[u].x; acc.y += y[u].y; acc.z += y[u].z; acc.w += y[u].w; }
            }
            *reinterpret_cast<float4*>(dst + k0) = acc;
        }
    }
    // the token's flag on its owner, raised whether or not a row went out: it also tells the owner that this rank is done with
    // the token's row and ids of this layer. One system-scope fence, by one thread after the block barrier (the barrier orders
    // the block's stores before it and the fence is cumulative).
    if (owner != g.rank) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            st_relaxed_sys(reinterpret_cast<unsigned*>(p.base[owner] + lay.flag_b) + (size_t)g.rank * g.n_own_max + (t - g.tok0[owner]), *step * EP_PHASES + phase);
        }
    }
}

// Combine, owner's side. grid own tokens, 256 threads: waits for all ranks' combine flags of own token i, then:
// value = sum over source ranks 0..R-1 (those that hold one of the token's experts) of their partial row, + the shared
// expert's row, + the residual row x[i] when x is given. x[i] and out[i] receive the value when given. When xn is given the
// next layer's input is left there (absolute token index): rmsnorm(value) if norm, else the value itself, with its 16-bit
// split in xs when xs is given.
template <bool F16>
__global__ void __launch_bounds__(256) ep_combine_norm_k(const EpGeom g, const uint8_t* __restrict__ local, const EpLayout lay,
                                                         const float* __restrict__ extra, float* __restrict__ x, float* __restrict__ out,
                                                         float* __restrict__ xn, uint16_t* __restrict__ xs, int norm, float eps,
                                                         const unsigned* __restrict__ step, unsigned phase, int* err) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x, t = g.tok0[g.rank] + i, K = g.K;
    if ((int)threadIdx.x < g.world && (int)threadIdx.x != g.rank)
        ep_wait_flag(reinterpret_cast<const unsigned*>(local + lay.flag_b) + (size_t)threadIdx.x * g.n_own_max + i, *step * EP_PHASES + phase, err, EP_ERR_COMBINE_WAIT);
    __syncthreads();   // the polling threads' acquire loads, then the barrier: the peers' rows are visible to the whole block
    // the ids of the layer whose partial rows these are: the routing kernel of the next layer has not run yet
    const int* idx = reinterpret_cast<const int*>(local + lay.idx) + (size_t)t * K;
    unsigned need = 0;
    for (int r = 0; r < K; r++) {
        const int e = idx[r];
        for (int s = 0; s < g.world; s++) if (e >= g.exp0[s] && e < g.exp0[s + 1]) need |= 1u << s;
    }
    const float* part = reinterpret_cast<const float*>(local + lay.part);
    float v[8];
    // both halves of the row in one round trip: every load is requested before the first addition
    float4 ye[2], yx[2], y[2][EP_MAX_RANKS];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int k0 = 1024 * h + 4 * threadIdx.x;
        ye[h] = yx[h] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (extra) ye[h] = *reinterpret_cast<const float4*>(extra + (size_t)t * EH + k0);
        if (x) yx[h] = *reinterpret_cast<const float4*>(x + (size_t)i * EH + k0);
#pragma unroll
        for (int s = 0; s < EP_MAX_RANKS; s++)
            if (s < g.world && (need >> s & 1)) y[h][s] = __ldcg(reinterpret_cast<const float4*>(part + ((size_t)s * g.n_own_max + i) * EH + k0));
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int k0 = 1024 * h + 4 * threadIdx.x;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < EP_MAX_RANKS; s++)
            if (s < g.world && (need >> s & 1)) { acc.x += y[h][s].x; acc.y += y[h][s].y; acc.z += y[h][s].z; acc.w += y[h][s].w; }
        if (extra) { acc.x += ye[h].x; acc.y += ye[h].y; acc.z += ye[h].z; acc.w += ye[h].w; }
        if (x) { acc.x = yx[h].x + acc.x; acc.y = yx[h].y + acc.y; acc.z = yx[h].z + acc.z; acc.w = yx[h].w + acc.w; }
        if (x) *reinterpret_cast<float4*>(x + (size_t)i * EH + k0) = acc;
        if (out) *reinterpret_cast<float4*>(out + (size_t)i * EH + k0) = acc;
        v[4 * h] = acc.x; v[4 * h + 1] = acc.y; v[4 * h + 2] = acc.z; v[4 * h + 3] = acc.w;
    }
    if (xn) {
        const float r = norm ? row_rms_scale(v, eps) : 1.f;
        scaled_split_row<F16>(v, r, xn + (size_t)t * EH, xs ? xs + (size_t)t * 2 * EH : nullptr);
    }
}

// Self-test of the flag wait's time-out: one thread waits for a flag nobody raises.
__global__ void selftest_ep_wait_timeout_k(const unsigned* flag, int* err, int limit, int* result) {
    if (threadIdx.x == 0) *result = ep_wait_flag(flag, 1u, err, EP_ERR_COMBINE_WAIT, limit) ? 1 : 0;
}

}  // namespace moexb
