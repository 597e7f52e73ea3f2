// Grouped expert GEMM for prefill-size batches on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA of 512 threads owns a 256-row weight block of one expert (gate rows r..r+127 and the same up rows; or 256
// consecutive down rows) and one tile of up to 128 activation columns (tokens of that expert, as bf16: one column per
// token when the input is exactly bf16, hi + lo columns when it is fp32). Per 64-input scale group:
//   1. every thread reads one 16-byte lane unit of the tiled weight image (16 nibbles of two rows), turns it into exact
//      bf16 integers in registers and stores four 16-byte rows of the K-major canonical core-matrix layout in shared
//      memory; the group's activation rows arrive with cp.async;
//   2. one thread issues 2 x 4 tcgen05.mma (M = 128, N = columns, K = 16) into a per-group accumulator in TMEM and
//      commits them to an mbarrier;
//   3. when the barrier flips, every thread pulls its row's partial sums out of TMEM (tcgen05.ld) and adds them, times the
//      row's fp32 group scale, to fp32 accumulators in registers - weights stay exact, exactly as in the streaming
//      kernels.
// Steps 1 and 3 of neighbouring groups run while the tensor core works on step 2 (two shared-memory stages, two TMEM
// accumulators per weight half). Every mbarrier wait is bounded; on a time-out the CTA still frees its TMEM and leaves.
//
// Inputs are permuted inside every block of 8: position 8b + j holds input 8b + p(j), p = (0,4,1,5,2,6,3,7) - the order in
// which dq_word produces weights - for the activations as well, so no shuffling is needed at run time.
#pragma once
#include "common.cuh"
#include "stream.cuh"
#include "tiled.cuh"

namespace moexb {

constexpr int PF_THREADS = 512;
constexpr int PF_NMAX = 128;            // activation columns per tile (MMA N)
constexpr int PF_A_STAGE = 256 * 128;   // 256 rows x 64 inputs x 2 bytes
constexpr int PF_B_STAGE = PF_NMAX * 128;

__host__ __device__ constexpr int perm8_pos(int k) { return (k & ~7) | (((k & 3) << 1) | ((k >> 2) & 1)); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // K-major, no swizzle: core matrices of 8 rows x 16 bytes; LBO = step between the two K halves of an MMA, SBO = step
    // between 8-row groups; bits 46-47 = descriptor version 1
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint32_t umma_idesc_bf16(int M, int N) {
    // D = f32 (bits 4-5 = 1), A = B = bf16 (bits 7-9, 10-12 = 1), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, bool accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

struct PrefillArgs {
    const moexb_pair_item* tiles;  // sub-items: an expert blob (tiled layout) and up to `ntok` of its pairs
    const int* ntiles;
    const moexb_pair* pairs;
    const uint16_t* xs;            // gate/up: activations [token][parts][H] bf16, perm8 order; down: act [pair p][2][I]
    uint16_t* act_out;             // gate/up output: act [p][2][I] bf16 hi, lo, perm8 order
    float* act32;                  // optional fp32 copy of act
    float* ypair;                  // down output [p][H]
    int* err;
    int parts;                     // activation columns per pair in xs: 1 (exact bf16) or 2 (hi + lo)
};

// DOWN = false: weight block = gate rows 128*rt..+127 (half 0) and the same up rows (half 1); K = 2048 = 32 groups.
// DOWN = true : weight block = down rows 256*rt..+127 (half 0) and +128..+255 (half 1); K = 512 = 8 groups; parts = 2.
template <int FMT, bool DOWN>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_k(const PrefillArgs a) {
    static_assert(FMT == FMT_SYM_F16 || FMT == FMT_SYM_F32, "zero-point experts use the streaming kernels");
    constexpr int GB = tl_group_bytes<FMT>(), SB = tl_slice_bytes<FMT>();
    constexpr int NG = DOWN ? EI / 64 : EH / 64;   // scale groups along K
    constexpr int RT = DOWN ? EH / 256 : EI / 128; // row blocks per expert
    constexpr int KB = DOWN ? EI : EH;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;                                 // 2 stages x [half][k-block 8][row 128][16 B]
    uint8_t* sB = smem + 2 * PF_A_STAGE;                // 2 stages x [k-block 8][column 128][16 B]
    float* sS = reinterpret_cast<float*>(sB + 2 * PF_B_STAGE);   // group scales [NG][256 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sS) + NG * 256 * 4);  // MMA-done barriers of the two stages
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 2);
    int* s_fail = reinterpret_cast<int*>(s_tmem + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { mbar_init(smem_u32(bars), 1); mbar_init(smem_u32(bars + 1), 1); *s_fail = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;

    // this thread's lane unit of the weight image: slice j of the 16 in the block, lane l = 4*g + t of the slice's group
    const int uj = tid >> 5, ul = tid & 31, ug = ul >> 2, ut = ul & 3;
    // rows (within their half) of the unit's two 8-byte pieces, and the halves they belong to
    const int rowA = DOWN ? (uj & 7) * 16 + ug : uj * 8 + ug, rowB = DOWN ? rowA + 8 : rowA;
    const int halfA = DOWN ? uj >> 3 : 0, halfB = DOWN ? uj >> 3 : 1;
    // this thread's accumulator slice: TMEM lanes 32*(warp & 3) .. +31 (row = that + lane), weight half, column half
    const int e_half = warp >> 3, e_ch = (warp >> 2) & 1, e_row = 32 * (warp & 3) + lane;
    uint32_t phase[2] = {0, 0};
    const int ntiles = *a.ntiles * RT;

    for (int tile = blockIdx.x; tile < ntiles && !*s_fail; tile += gridDim.x) {
        const moexb_pair_item it = a.tiles[tile / RT];
        const int rt = tile % RT;
        const int ncol = it.count * a.parts;                 // real activation columns
        const int N = (ncol + 31) & ~31;                     // MMA N: a multiple of 32, so each column half is a multiple of 16
        const uint32_t idesc = umma_idesc_bf16(128, N);
        // slices of this block in the tiled image: gate/up slice (wt, ks) = wt*4 + ks with wt = 16*rt + j; down slice 256 + 16*rt + j
        const uint8_t* blob = it.slot;
        // group scales of the block's 256 rows: the unit owner of (j, g) copies both rows' scales for all groups
        if (ut == 0) {
            for (int G = 0; G < NG; G++) {
                const uint8_t* sl = blob + (size_t)(DOWN ? 256 + 16 * rt + uj : (16 * rt + uj) * 4 + (G >> 3)) * SB + (G & 7) * GB + 512;
                float s0, s1;
                if constexpr (FMT == FMT_SYM_F16) { const float2 s2 = __half22float2(*reinterpret_cast<const __half2*>(sl + 4 * ug)); s0 = s2.x; s1 = s2.y; }
                else { const float2 s2 = *reinterpret_cast<const float2*>(sl + 8 * ug); s0 = s2.x; s1 = s2.y; }
                sS[G * 256 + halfA * 128 + rowA] = s0;
                sS[G * 256 + halfB * 128 + rowB] = s1;
            }
        }
        // activation rows of this tile's columns
        const uint16_t* xcol0 = nullptr; const uint16_t* xcol1 = nullptr;  // the (up to) two 16-byte copies per group this thread makes
        int c0 = -1, c1 = -1;
        {
            // copy unit u = (column, k-block of 8): 8 per column per group; N*8 units, threads take u = tid and tid + 512
            const int u0 = tid, u1 = tid + PF_THREADS;
            if (u0 < N * 8) {
                c0 = u0 >> 3;
                if (c0 < ncol) { const moexb_pair pr = a.pairs[it.start + c0 / a.parts]; xcol0 = a.xs + ((size_t)(DOWN ? pr.p : pr.t) * a.parts + c0 % a.parts) * KB + (u0 & 7) * 8; }
            }
            if (u1 < N * 8) {
                c1 = u1 >> 3;
                if (c1 < ncol) { const moexb_pair pr = a.pairs[it.start + c1 / a.parts]; xcol1 = a.xs + ((size_t)(DOWN ? pr.p : pr.t) * a.parts + c1 % a.parts) * KB + (u1 & 7) * 8; }
            }
        }
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; i++) acc[i] = 0.f;

        // fill stage (G & 1) with group G: weights (dequantised) and activations
        auto fill = [&](int G) {
            const int st = G & 1;
            const uint8_t* sl = blob + (size_t)(DOWN ? 256 + 16 * rt + uj : (16 * rt + uj) * 4 + (G >> 3)) * SB + (G & 7) * GB;
            const uint4 q = ld_stream(reinterpret_cast<const uint4*>(sl) + ul);
            uint32_t P[4];
            uint8_t* base = sA + st * PF_A_STAGE;
            // piece A: 16 nibbles of rowA, inputs 16*ut .. +15 of the group = k-blocks 2*ut, 2*ut + 1
            dq_word<true>(q.x, P); *reinterpret_cast<uint4*>(base + halfA * 16384 + (2 * ut) * 2048 + rowA * 16) = make_uint4(P[0], P[1], P[2], P[3]);
            dq_word<true>(q.y, P); *reinterpret_cast<uint4*>(base + halfA * 16384 + (2 * ut + 1) * 2048 + rowA * 16) = make_uint4(P[0], P[1], P[2], P[3]);
            dq_word<true>(q.z, P); *reinterpret_cast<uint4*>(base + halfB * 16384 + (2 * ut) * 2048 + rowB * 16) = make_uint4(P[0], P[1], P[2], P[3]);
            dq_word<true>(q.w, P); *reinterpret_cast<uint4*>(base + halfB * 16384 + (2 * ut + 1) * 2048 + rowB * 16) = make_uint4(P[0], P[1], P[2], P[3]);
            uint8_t* bb = sB + st * PF_B_STAGE;
            if (c0 >= 0) {
                const uint32_t dst = smem_u32(bb + (tid & 7) * (N * 16) + c0 * 16);
                if (xcol0) cp_async16(dst, xcol0 + G * 64); else *reinterpret_cast<uint4*>(bb + (tid & 7) * (N * 16) + c0 * 16) = make_uint4(0, 0, 0, 0);
            }
            if (c1 >= 0) {
                const uint32_t dst = smem_u32(bb + (tid & 7) * (N * 16) + c1 * 16);
                if (xcol1) cp_async16(dst, xcol1 + G * 64); else *reinterpret_cast<uint4*>(bb + (tid & 7) * (N * 16) + c1 * 16) = make_uint4(0, 0, 0, 0);
            }
        };
        // issue the 8 MMAs of group G (one thread)
        auto issue = [&](int G) {
            const int st = G & 1;
            const uint32_t aB = smem_u32(sA + st * PF_A_STAGE), bB = smem_u32(sB + st * PF_B_STAGE);
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    umma_bf16(tmem + (uint32_t)((h * 2 + st) * PF_NMAX), umma_desc(aB + h * 16384 + ks * 4096, 2048, 128),
                              umma_desc(bB + ks * 2 * (N * 16), N * 16, 128), idesc, ks > 0);
            umma_commit(smem_u32(bars + st));
        };
        // add group G's partial sums, scaled, to the accumulators
        auto drain = [&](int G) {
            const int st = G & 1;
            const float s = sS[G * 256 + e_half * 128 + e_row];
            const uint32_t t0 = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)((e_half * 2 + st) * PF_NMAX + e_ch * (N >> 1));
#pragma unroll
            for (int cb = 0; cb < 4; cb++) {
                if (cb * 16 < (N >> 1)) {
                    float v[16];
                    tmem_ld16(t0 + cb * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; i++) acc[cb * 16 + i] = fmaf(v[i], s, acc[cb * 16 + i]);
                }
            }
        };

        __syncthreads();  // the previous tile's readers are done with the stages, scales and TMEM
        fill(0);
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue(0); }
        for (int G = 0; G < NG; G++) {
            // MMAs of group G-1 are done: its stage is free for group G+1 and its sums can be drained
            if (G >= 1) {
                if (!mbar_wait(smem_u32(bars + ((G - 1) & 1)), phase[(G - 1) & 1], a.err, 3)) *s_fail = 1;
                phase[(G - 1) & 1] ^= 1;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (G + 1 < NG) fill(G + 1);
            if (G >= 1) drain(G - 1);
            asm volatile("cp.async.wait_all;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (*s_fail) break;
            if (G + 1 < NG && tid == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue(G + 1); }
        }
        if (*s_fail) break;
        if (!mbar_wait(smem_u32(bars + ((NG - 1) & 1)), phase[(NG - 1) & 1], a.err, 3)) *s_fail = 1;
        phase[(NG - 1) & 1] ^= 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        drain(NG - 1);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (*s_fail) break;

        // epilogue. The thread holds row e_row of half e_half, columns e_ch*N/2 .. +N/2-1. (All loops over acc are fully
        // unrolled with constant indices so the accumulators stay in registers.)
        const int cbase = e_ch * (N >> 1);
        if (DOWN) {
            const int d = 256 * rt + 128 * e_half + e_row;
#pragma unroll
            for (int i = 0; i < 64; i += 2) {   // parts == 2: columns (2j, 2j+1) = (hi, lo) of pair j
                const int j = (cbase + i) >> 1;
                if (i < (N >> 1) && j < it.count) {
                    const moexb_pair pr = a.pairs[it.start + j];
                    a.ypair[(size_t)pr.p * EH + d] = pr.w * (acc[i] + acc[i + 1]);
                }
            }
        } else {
            // up half hands its sums to the gate half through shared memory (the stages are free now)
            float* ex = reinterpret_cast<float*>(sA);  // [row 128][column PF_NMAX]
            if (e_half == 1) {
#pragma unroll
                for (int i = 0; i < 64; i++)
                    if (i < (N >> 1)) ex[e_row * PF_NMAX + cbase + i] = acc[i];
            }
            __syncthreads();
            if (e_half == 0) {
                const int row = 128 * rt + e_row;
                const bool two = a.parts == 2;
#pragma unroll
                for (int i = 0; i < 64; i++) {
                    const int j = two ? (cbase + i) >> 1 : cbase + i;
                    if (i < (N >> 1) && j < it.count && !(two && (i & 1))) {
                        float g = acc[i], u = ex[e_row * PF_NMAX + cbase + i];
                        if (two) { g += acc[(i + 1) & 63]; u += ex[e_row * PF_NMAX + cbase + i + 1]; }
                        const float v = g / (1.f + expf(-g)) * u;
                        const moexb_pair pr = a.pairs[it.start + j];
                        if (a.act32) a.act32[(size_t)pr.p * EI + row] = v;
                        uint16_t hi, lo;
                        split_hi_lo<false>(v, hi, lo);
                        uint16_t* dst = a.act_out + (size_t)pr.p * 2 * EI + perm8_pos(row);
                        dst[0] = hi; dst[EI] = lo;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

template <int FMT, bool DOWN>
constexpr int pf_smem_bytes() { return 2 * PF_A_STAGE + 2 * PF_B_STAGE + (DOWN ? EI / 64 : EH / 64) * 256 * 4 + 64 + 1024; }

// x [rows][K] fp32 -> xs [rows][parts][K] bf16 in perm8 order: parts = 1 keeps bf16(x) (exact when x came from bf16),
// parts = 2 adds lo = bf16(x - hi).
__global__ void split8_rows_k(const float* __restrict__ x, uint16_t* __restrict__ xs, int K, int parts, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t r = i / K; const int k = (int)(i % K);
    uint16_t hi, lo;
    split_hi_lo<false>(x[i], hi, lo);
    uint16_t* dst = xs + r * parts * K + perm8_pos(k);
    dst[0] = hi;
    if (parts == 2) dst[K] = lo;
}

}  // namespace moexb
