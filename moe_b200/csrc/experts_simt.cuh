// Routed-expert kernels in fp32 SIMT arithmetic: one-token decode and the per-pair multi-token path.
// Weights are streamed with 16-byte loads (32 int4 each), unpacked in registers and reduced with warp shuffles; the
// dequantised value of every weight is exact, products and sums are fp32 fused multiply-adds.
#pragma once
#include "common.cuh"

namespace moexb {

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + expf(-g)) * u; }

// Stage n floats of x into padded shared memory (see pad32).
__device__ __forceinline__ void stage_padded(float* __restrict__ xs, const float* __restrict__ x, int n) {
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4)
        *reinterpret_cast<float4*>(xs + pad32(i)) = __ldg(reinterpret_cast<const float4*>(x + i));
}

// One token. act[k][row] = silu(gate_k[row] . x) * (up_k[row] . x). Block (row block, expert k): a warp owns one
// (gate, up) row pair = 2 x 1024 bytes, all four 16-byte loads of a lane are issued before x is staged, so the DRAM
// latency overlaps the staging. Stands behind expert_gate_up_k (kernels.cuh:597-622).
template <int FMT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) decode_gate_up_k(const uint8_t* const* __restrict__ slots, int K, const int* __restrict__ nh,
                                                               const float* __restrict__ x, float* __restrict__ act) {
    __shared__ __align__(16) float xs[pad32_size(EH)];
    const int k = blockIdx.y;
    if (k >= (nh ? *nh : K)) return;
    const int row = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const uint8_t* blob = slots[k];
    const uint4* g = reinterpret_cast<const uint4*>(blob + (size_t)row * (EH / 2));
    const uint4* u = reinterpret_cast<const uint4*>(blob + (size_t)(EI + row) * (EH / 2));
    uint4 qg[2], qu[2]; float2 sg[2], su[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int c = lane + 32 * i;
        qg[i] = ld_stream(g + c); qu[i] = ld_stream(u + c);
        sg[i] = chunk_scale<FMT>(blob, (size_t)row * (EH / 32) + c);
        su[i] = chunk_scale<FMT>(blob, (size_t)(EI + row) * (EH / 32) + c);
    }
    stage_padded(xs, x, EH);
    __syncthreads();
    float ag = 0.f, au = 0.f;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int c = lane + 32 * i;
        ag += dot32<FMT>(qg[i], xs + 36 * c, sg[i]);
        au += dot32<FMT>(qu[i], xs + 36 * c, su[i]);
    }
    ag = warp_sum(ag); au = warp_sum(au);
    if (lane == 0) act[(size_t)k * EI + row] = silu_mul(ag, au);
}

// One token. out[d] = sum_k w[k] * (down_k[d] . act_k). A down row is 256 bytes = 16 lanes x 16 bytes, so each half
// warp takes every other expert; all loads of a row are in flight before the first product. Stands behind
// expert_down_k (kernels.cuh:624-657). Dynamic shared memory: K * pad32_size(EI) floats.
template <int FMT, int WARPS, int KMAX>
__global__ void __launch_bounds__(WARPS * 32) decode_down_k(const uint8_t* const* __restrict__ slots, const float* __restrict__ w, int K,
                                                            const int* __restrict__ nh, const float* __restrict__ act, float* __restrict__ out) {
    extern __shared__ __align__(16) float as[];
    if (nh) K = min(K, max(*nh, 0));   // the launch sized shared memory for K experts: a larger device count is clamped
    const int d = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31, hf = lane >> 4, c = lane & 15;
    uint4 q[KMAX / 2]; float2 sm[KMAX / 2]; float wk[KMAX / 2];
#pragma unroll
    for (int i = 0; i < KMAX / 2; i++) {
        const int k = 2 * i + hf;
        if (k < K) {
            const uint8_t* blob = slots[k];
            q[i] = ld_stream(reinterpret_cast<const uint4*>(blob + DOWN_Q_OFF + (size_t)d * (EI / 2)) + c);
            sm[i] = chunk_scale<FMT>(blob, DOWN_C_OFF + (size_t)d * (EI / 32) + c);
            wk[i] = w[k];
        }
    }
    for (int i = threadIdx.x * 4; i < K * EI; i += blockDim.x * 4)
        *reinterpret_cast<float4*>(as + (i / EI) * pad32_size(EI) + pad32(i % EI)) = __ldg(reinterpret_cast<const float4*>(act + i));
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < KMAX / 2; i++) {
        const int k = 2 * i + hf;
        if (k < K) acc = fmaf(wk[i], dot32<FMT>(q[i], as + k * pad32_size(EI) + 36 * c, sm[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[d] = acc;
}

// T tokens grouped by expert. act[p][row] for every pair of item blockIdx.y: the warp keeps its (gate, up) row pair
// in registers and walks the item's tokens, whose activations the block stages one at a time. Stands behind
// pairs_gate_up_k (kernels.cuh:691-720).
template <int FMT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) pairs_gate_up_k(const moexb_pair_item* __restrict__ items, const moexb_pair* __restrict__ pairs,
                                                              const float* __restrict__ X, float* __restrict__ act, const int* __restrict__ nitems) {
    __shared__ __align__(16) float xs[pad32_size(EH)];
    if (nitems && (int)blockIdx.y >= *nitems) return;
    const moexb_pair_item it = items[blockIdx.y];
    const int row = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const uint4* g = reinterpret_cast<const uint4*>(it.slot + (size_t)row * (EH / 2));
    const uint4* u = reinterpret_cast<const uint4*>(it.slot + (size_t)(EI + row) * (EH / 2));
    uint4 qg[2], qu[2]; float2 sg[2], su[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int c = lane + 32 * i;
        qg[i] = ld_stream(g + c); qu[i] = ld_stream(u + c);
        sg[i] = chunk_scale<FMT>(it.slot, (size_t)row * (EH / 32) + c);
        su[i] = chunk_scale<FMT>(it.slot, (size_t)(EI + row) * (EH / 32) + c);
    }
    for (int j = 0; j < it.count; j++) {
        const moexb_pair pr = pairs[it.start + j];
        __syncthreads();
        stage_padded(xs, X + (size_t)pr.t * EH, EH);
        __syncthreads();
        float ag = 0.f, au = 0.f;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int c = lane + 32 * i;
            ag += dot32<FMT>(qg[i], xs + 36 * c, sg[i]);
            au += dot32<FMT>(qu[i], xs + 36 * c, su[i]);
        }
        ag = warp_sum(ag); au = warp_sum(au);
        if (lane == 0) act[(size_t)pr.p * EI + row] = silu_mul(ag, au);
    }
}

// ypair[p][d] = w_p * (down[d] . act[p]). One warp per output row, the two half warps take alternate pairs.
// Stands behind pairs_down_k (kernels.cuh:722-740).
template <int FMT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) pairs_down_k(const moexb_pair_item* __restrict__ items, const moexb_pair* __restrict__ pairs,
                                                           const float* __restrict__ act, float* __restrict__ ypair, const int* __restrict__ nitems) {
    if (nitems && (int)blockIdx.y >= *nitems) return;
    const moexb_pair_item it = items[blockIdx.y];
    const int d = blockIdx.x * WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31, hf = lane >> 4, c = lane & 15;
    const uint4 q = ld_stream(reinterpret_cast<const uint4*>(it.slot + DOWN_Q_OFF + (size_t)d * (EI / 2)) + c);
    const float2 sm = chunk_scale<FMT>(it.slot, DOWN_C_OFF + (size_t)d * (EI / 32) + c);
    for (int j0 = 0; j0 < it.count; j0 += 2) {
        const int j = j0 + hf;
        const bool on = j < it.count;
        const moexb_pair pr = pairs[it.start + (on ? j : j0)];
        float v = on ? dot32<FMT>(q, act + (size_t)pr.p * EI + 32 * c, sm) : 0.f;
        v = half_warp_sum(v);
        if (c == 0 && on) ypair[(size_t)pr.p * EH + d] = pr.w * v;
    }
}

// moe[t][d] = sum_{r<K} ypair[t*K+r][d] in rank order, + extra[t][d] when given (kernels.cuh:744-753, where the
// extra term is the CPU experts' share; here it also carries the shared expert's rows).
__global__ void pairs_reduce_k(const float* __restrict__ ypair, const float* __restrict__ extra, float* __restrict__ moe, int K, int D,
                               const int* __restrict__ use_extra) {
    if (use_extra && !*use_extra) extra = nullptr;
    const int t = blockIdx.y, d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (d >= D) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < K; r++) {
        const float4 v = *reinterpret_cast<const float4*>(ypair + ((size_t)t * K + r) * D + d);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (extra) {
        const float4 v = *reinterpret_cast<const float4*>(extra + (size_t)t * D + d);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(moe + (size_t)t * D + d) = acc;
}

// out[t][d] += sh[t][d] / (1 + exp(-gl[t])) (kernels.cuh:973-977, 1101-1106)
__global__ void gated_add_rows_k(float* __restrict__ out, const float* __restrict__ sh, const float* __restrict__ gl, int gl_stride, int D) {
    const int t = blockIdx.y, d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d < D) out[(size_t)t * D + d] += sh[(size_t)t * D + d] / (1.f + expf(-gl[(size_t)t * gl_stride]));
}

// One item over all T tokens with weight 1 and p = t: the work list of an expert applied to every token.
__global__ void identity_pairs_k(const uint8_t* blob, int T, moexb_pair_item* item, moexb_pair* pairs) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t == 0) *item = {blob, 0, T};
    if (t < T) pairs[t] = {t, t, 1.f};
}

// ---- glue of the layer-level calls ------------------------------------------------------------------------------------

__global__ void bf16_to_f32_k(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i < n) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(in + i));
        out[i] = v.x; out[i + 1] = v.y;
    }
}

// y = x / sqrt(mean(x^2) + eps), unit weight (kernels.cuh:48-64 with w = 0). One block of 256 per row; D % 4 == 0.
// The sum of squares has a pinned order (thread i takes elements 4i..4i+3, 1024+4i.., with fused multiply-adds; a
// xor-butterfly per warp; the 8 warp sums added in order) and the square root and divisions are IEEE, so the CPU
// oracle reproduces the normalised row bit for bit and a chained stack routes identically on both sides.
__global__ void __launch_bounds__(256) rmsnorm_rows_k(const float* __restrict__ x, float* __restrict__ y, int D, float eps) {
    __shared__ float part[8];
    const float* xr = x + (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < D; i += 1024) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float r = 1.f / sqrtf(tot / (float)D + eps);
    for (int i = threadIdx.x * 4; i < D; i += 1024) {
        float4 v = *reinterpret_cast<const float4*>(xr + i);
        v.x *= r; v.y *= r; v.z *= r; v.w *= r;
        *reinterpret_cast<float4*>(y + (size_t)blockIdx.x * D + i) = v;
    }
}

// out = x + moe (the residual add the reference folds into the next layer's RMSNorm, moex.cu:1082)
__global__ void residual_add_k(const float* __restrict__ x, const float* __restrict__ moe, float* __restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i < n) {
        const float4 a = *reinterpret_cast<const float4*>(x + i), b = *reinterpret_cast<const float4*>(moe + i);
        *reinterpret_cast<float4*>(out + i) = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
    }
}

}  // namespace moexb
