// Shared device helpers of the expert-FFN kernels: geometry, blob accessors, nibble unpacking, warp reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "moexb.h"

namespace moexb {

// Geometry of one expert, fixed like the reference's constexprs (kernels.cuh:422-426).
constexpr int EH = 2048;                                  // hidden size: inputs of gate/up, outputs of down
constexpr int EI = 512;                                   // expert intermediate size
constexpr int EGS = 64;                                   // weights per scale group
constexpr size_t Q_BYTES = (size_t)3 * EH * EI / 2;       // 1,572,864 bytes of packed nibbles
constexpr size_t CHUNKS = (size_t)3 * EH * EI / 32;       // 98,304 chunks of 32 weights (one 16-byte load each)
constexpr size_t DOWN_Q_OFF = (size_t)2 * EI * (EH / 2);  // byte offset of the down matrix in the nibble area
constexpr size_t DOWN_C_OFF = (size_t)2 * EI * (EH / 32); // first chunk of the down matrix

enum : int { FMT_SYM_F32 = 0, FMT_SYM_F16 = 1, FMT_ZP = 2 };

__host__ __device__ constexpr size_t expert_bytes(int fmt) {
    return fmt == FMT_SYM_F32 ? Q_BYTES + CHUNKS / 2 * 4 : fmt == FMT_SYM_F16 ? Q_BYTES + CHUNKS / 2 * 2
         : fmt == FMT_ZP ? Q_BYTES + CHUNKS * 2 + CHUNKS / 8 * 4 : 0;
}

// Programmatic dependent launch. A kernel started with the programmatic-serialization launch attribute may begin while
// its predecessor in the stream still runs: pdl_wait() blocks until the predecessor has finished and its writes are
// visible, so everything a kernel does before it must touch only data the predecessor does not write (weights, shared
// memory set-up). pdl_trigger() lets the successor's blocks be scheduled as soon as every block of this grid has
// called it; every kernel here calls it after its own pdl_wait(), so a successor never runs (not even its part before the
// wait) until the kernel two places ahead of it has finished. Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- expert parallelism (ep.cuh): geometry, exchange-buffer layout, flags that another GPU raises ----
constexpr int EP_MAX_RANKS = 8;
struct EpGeom {
    int rank, world, T, K, n_own_max;
    int tok0[EP_MAX_RANKS + 1];   // rank r owns tokens [tok0[r], tok0[r+1])
    int exp0[EP_MAX_RANKS + 1];   // and holds routed experts [exp0[r], exp0[r+1])
};
// byte offsets inside an exchange buffer: activation rows [T][2][H] 16-bit, ids [T][K], weights [T][K], partial rows
// [world][n_own_max][H] f32, dispatch flags [T] (one per token), combine flags [world][n_own_max] (one per source rank and own token)
struct EpLayout { size_t xs, idx, w, part, flag_a, flag_b, bytes; };
struct EpPeers { uint8_t* base[EP_MAX_RANKS]; };   // exchange buffer of every rank, as mapped in this process
struct EpDevice { EpGeom g; EpPeers p; EpLayout lay; };
constexpr unsigned EP_PHASES = 256;           // a flag holds step * EP_PHASES + layer + 1: layers of a step must stay below this
constexpr int EP_POLL_LIMIT = 1 << 21;        // polls (a local L2 round trip and a short sleep each: a second or two in all) before a wait gives up
constexpr int EP_ERR_DISPATCH_WAIT = 7, EP_ERR_COMBINE_WAIT = 8;
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for *flag >= target; false (and the error word set) when it ran out of polls.
__device__ __forceinline__ bool ep_wait_flag(const unsigned* flag, unsigned target, int* err, int code, int limit = EP_POLL_LIMIT) {
    for (int i = 0; i < limit; i++) {
        if ((int)(ld_acquire_sys(flag) - target) >= 0) return true;
        if (i > 64) __nanosleep(200);
    }
    atomicExch(err, code);
    return false;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Streaming 16-byte load: expert weights are read once per step, so they should not displace the activations and
// router weights that stay hot in L1/L2.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// (scale, zero) of 32-weight chunk g32 of a blob: symmetric formats (s, 0) with s shared by chunks 2g, 2g+1;
// zero point (d*sc, dm*mn) with [sc u8, mn i8] per chunk and half2 (d, dm) per 8 chunks (kernels.cuh:416-421).
template <int FMT>
__device__ __forceinline__ float2 chunk_scale(const uint8_t* __restrict__ blob, size_t g32) {
    const uint8_t* sp = blob + Q_BYTES;
    if constexpr (FMT == FMT_SYM_F32) return make_float2(__ldg(reinterpret_cast<const float*>(sp) + (g32 >> 1)), 0.f);
    else if constexpr (FMT == FMT_SYM_F16) return make_float2(__half2float(__ldg(reinterpret_cast<const __half*>(sp) + (g32 >> 1))), 0.f);
    else {
        const uchar2 cm = __ldg(reinterpret_cast<const uchar2*>(sp) + g32);
        const float2 dd = __half22float2(__ldg(reinterpret_cast<const __half2*>(sp + CHUNKS * 2) + (g32 >> 3)));
        return make_float2(dd.x * (float)cm.x, dd.y * (float)(int8_t)cm.y);
    }
}

// Nibble n (0..7) of word q as an exact float: the integer is or-ed into the mantissa of 2^23 and 2^23 (+8 for the
// two's-complement formats, whose nibbles were xor-ed with 8 beforehand) is subtracted again. No int->float converts.
template <bool SIGNED>
__device__ __forceinline__ float nib(uint32_t q, int n) {
    return __uint_as_float(0x4B000000u | ((q >> (4 * n)) & 0xFu)) - (SIGNED ? 8388616.f : 8388608.f);
}

// Activations in shared memory are read 32 consecutive floats per lane (the 32 inputs of one 16-byte weight load);
// 4 floats of padding after every 32 rotate the lanes over the banks, so the float4 reads do not conflict.
__host__ __device__ constexpr int pad32(int i) { return i + (i >> 5) * 4; }
__host__ __device__ constexpr int pad32_size(int n) { return n + n / 8; }

// 32 weights of one 16-byte load times 32 consecutive inputs at x (16-byte aligned; padded shared or global memory),
// fp32 fused multiply-adds, scaled: s * sum(q x) for the symmetric formats, s * sum(u x) + m * sum(x) for zero point.
template <int FMT>
__device__ __forceinline__ float dot32(uint4 q, const float* __restrict__ x, float2 sm) {
    constexpr bool Z = FMT == FMT_ZP;
    uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float acc = 0.f, sx = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (!Z) w[j] ^= 0x88888888u;
        const float4 a = *reinterpret_cast<const float4*>(x + 8 * j), b = *reinterpret_cast<const float4*>(x + 8 * j + 4);
        const float xs[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int n = 0; n < 8; n++) {
            acc = fmaf(nib<!Z>(w[j], n), xs[n], acc);
            if (Z) sx += xs[n];
        }
    }
    return Z ? fmaf(sm.x, acc, sm.y * sx) : acc * sm.x;
}

}  // namespace moexb
