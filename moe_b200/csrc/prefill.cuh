// Grouped expert GEMM for prefill-size batches on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA of 512 threads owns a 256-row weight block of one expert (gate rows r..r+127 and the same up rows; or 256
// consecutive down rows) and one tile of up to 128 activation columns (tokens of that expert, as fp16: one column per
// token when the input is exactly bf16, hi + lo columns when it is fp32). Per 64-input scale group:
//   1. every thread takes one 16-byte lane unit of the tiled weight image (16 nibbles of two rows; the raw bytes were
//      requested five groups earlier with cp.async), unpacks it to exact fp16 integers, multiplies by the group's fp16
//      scale and splits the product into hi = fp16(q*s) and lo = q*s - hi (one fused multiply-add; both halves together
//      are the exact weight), and stores them as K-major canonical core matrices in shared memory; the group's
//      activation rows arrive with cp.async;
//   2. one thread issues 16 tcgen05.mma (M = 128, N = columns, K = 16; hi and lo weights x two weight halves x four K
//      steps) that accumulate over all groups in TMEM, and commits them to an mbarrier, which frees the stage.
// The unpacking of group G+1 runs while the tensor core works on group G. After the last group every thread reads its
// row's sums out of TMEM (tcgen05.ld) for the epilogue. Every mbarrier wait is bounded; on a time-out the CTA still
// frees its TMEM and leaves.
//
// Inputs are permuted inside every block of 8: position 8b + j holds input 8b + p(j), p = (0,4,1,5,2,6,3,7) - the order in
// which the unpacking produces weights - for the activations as well, so no shuffling is needed at run time.
#pragma once
#include "common.cuh"
#include "stream.cuh"
#include "tiled.cuh"

namespace moexb {

constexpr int PF_THREADS = 512;
constexpr int PF_NMAX = 128;            // activation columns per tile (MMA N)
constexpr int PF_A_STAGE = 2 * 256 * 128;   // hi and lo x 256 rows x 64 inputs x 2 bytes
constexpr int PF_B_STAGE = PF_NMAX * 128;

__host__ __device__ constexpr int perm8_pos(int k) { return (k & ~7) | (((k & 3) << 1) | ((k >> 2) & 1)); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // K-major, no swizzle: core matrices of 8 rows x 16 bytes; LBO = step between the two K halves of an MMA, SBO = step
    // between 8-row groups; bits 46-47 = descriptor version 1
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint32_t umma_idesc_f16(int M, int N) {
    // D = f32 (bits 4-5 = 1), A = B = fp16 (bits 7-9, 10-12 = 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, bool accumulate) {
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

constexpr int PF_RING = 5;      // raw weight groups in flight (cp.async), each 8 KB of nibbles + the group's scales
constexpr int PF_AHEAD = 3;     // a group's raw bytes are requested this many groups before they are unpacked
constexpr int PF_RAW = 256 * 32 + 512;  // bytes of one ring slot

// DOWN = false: weight block = gate rows 128*rt..+127 (half 0) and the same up rows (half 1); K = 2048 = 32 groups.
// DOWN = true : weight block = down rows 256*rt..+127 (half 0) and +128..+255 (half 1); K = 512 = 8 groups; parts = 2.
template <int FMT, bool DOWN>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_k(const PrefillArgs a) {
    static_assert(FMT == FMT_SYM_F16, "the grouped GEMM takes fp16 group scales; other formats use the streaming kernels");
    constexpr int GB = tl_group_bytes<FMT>(), SB = tl_slice_bytes<FMT>();
    constexpr int NG = DOWN ? EI / 64 : EH / 64;   // scale groups along K
    constexpr int RT = DOWN ? EH / 256 : EI / 128; // row blocks per expert
    constexpr int KB = DOWN ? EI : EH;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;                                 // 2 stages x [hi, lo][half][k-block 8][row 128][16 B]
    uint8_t* sB = sA + 2 * PF_A_STAGE;                  // 3 stages x [k-block 8][column N][16 B]
    uint8_t* sR = sB + 3 * PF_B_STAGE;                  // ring of raw groups: [slot][512 units x 16 B | 128 scale pairs x 4 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sR + PF_RING * PF_RAW);  // MMA-done barriers of the two A stages
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 2);
    int* s_fail = reinterpret_cast<int*>(s_tmem + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { mbar_init(smem_u32(bars), 1); mbar_init(smem_u32(bars + 1), 1); *s_fail = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;

    // this thread's lane unit of the weight image: slice j of the 16 in the block, unit l = 4*g + t of the slice's group.
    // Lanes are spread as g = lane & 7, t = lane >> 3, so that eight consecutive lanes hold eight consecutive rows of one
    // k-block: their 16-byte stores into the core-matrix layout are one contiguous 128 bytes (no bank conflicts).
    const int uj = tid >> 5, ug = tid & 7, ut = (tid >> 3) & 3, ul = 4 * ug + ut;
    // rows (within their half) of the unit's two 8-byte pieces, and the halves they belong to
    const int rowA = DOWN ? (uj & 7) * 16 + ug : uj * 8 + ug, rowB = DOWN ? rowA + 8 : rowA;
    const int halfA = DOWN ? uj >> 3 : 0, halfB = DOWN ? uj >> 3 : 1;
    // this thread's slice of the result: TMEM lanes 32*(warp & 3) .. +31 (row = that + lane), weight half, column half
    const int e_half = warp >> 3, e_ch = (warp >> 2) & 1, e_row = 32 * (warp & 3) + lane;
    uint32_t ph0 = 0, ph1 = 0;
    const int ntiles = *a.ntiles * RT;

    for (int tile = blockIdx.x; tile < ntiles && !*s_fail; tile += gridDim.x) {
        const moexb_pair_item it = a.tiles[tile / RT];
        const int rt = tile % RT;
        const int ncol = it.count * a.parts;                 // real activation columns
        const int N = (ncol + 31) & ~31;                     // MMA N: a multiple of 32, so each column half is a multiple of 16
        const uint32_t idesc = umma_idesc_f16(128, N);
        const uint8_t* blob = it.slot;
        // activation rows of this tile's columns: copy unit u = (column c, k-block kb of 8 inputs), N*8 units, threads take
        // u = tid and tid + 512. kb = (u & 1) + 2 * ((u >> 1) / N), c = (u >> 1) % N: a lane pair reads one 32-byte sector of a
        // column, consecutive pairs write consecutive 16-byte rows of the core-matrix layout.
        const uint16_t* xcol0 = nullptr; const uint16_t* xcol1 = nullptr;
        int d0 = -1, d1 = -1;  // byte offsets inside a B stage
        {
            const int u0 = tid, u1 = tid + PF_THREADS;
            if (u0 < N * 8) {
                const int c = (u0 >> 1) % N, kb = (u0 & 1) + 2 * ((u0 >> 1) / N);
                d0 = kb * (N * 16) + c * 16;
                if (c < ncol) { const moexb_pair pr = a.pairs[it.start + c / a.parts]; xcol0 = a.xs + ((size_t)(DOWN ? pr.p : pr.t) * a.parts + c % a.parts) * KB + kb * 8; }
            }
            if (u1 < N * 8) {
                const int c = (u1 >> 1) % N, kb = (u1 & 1) + 2 * ((u1 >> 1) / N);
                d1 = kb * (N * 16) + c * 16;
                if (c < ncol) { const moexb_pair pr = a.pairs[it.start + c / a.parts]; xcol1 = a.xs + ((size_t)(DOWN ? pr.p : pr.t) * a.parts + c % a.parts) * KB + kb * 8; }
            }
        }

        // request group G's raw bytes: this thread's 16-byte unit, and (one thread per row pair) the pair's two scales
        auto prefetch = [&](int G) {
            const uint8_t* gb = blob + (size_t)(DOWN ? 256 + 16 * rt + uj : (16 * rt + uj) * 4 + (G >> 3)) * SB + (G & 7) * GB;
            uint8_t* slot = sR + (G % PF_RING) * PF_RAW;
            cp_async16(smem_u32(slot + tid * 16), gb + ul * 16);
            if (ut == 0) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(slot + 8192 + (uj * 8 + ug) * 4)), "l"(gb + 512 + 4 * ug) : "memory");
        };
        // request group G's activation rows into B stage G % 3
        auto fill_b = [&](int G) {
            uint8_t* bb = sB + (G % 3) * PF_B_STAGE;
            if (d0 >= 0) { if (xcol0) cp_async16(smem_u32(bb + d0), xcol0 + G * 64); else *reinterpret_cast<uint4*>(bb + d0) = make_uint4(0, 0, 0, 0); }
            if (d1 >= 0) { if (xcol1) cp_async16(smem_u32(bb + d1), xcol1 + G * 64); else *reinterpret_cast<uint4*>(bb + d1) = make_uint4(0, 0, 0, 0); }
        };
        // unpack group G (its raw bytes have landed) into A stage G & 1: exact weight q*s as fp16 hi + lo
        auto unpack = [&](int G) {
            const uint8_t* slot = sR + (G % PF_RING) * PF_RAW;
            const uint4 q = *reinterpret_cast<const uint4*>(slot + tid * 16);
            const uint32_t sc = *reinterpret_cast<const uint32_t*>(slot + 8192 + (uj * 8 + ug) * 4);   // (scale of row A, scale of row B)
            const uint32_t sA2 = __byte_perm(sc, sc, 0x1010), sB2 = __byte_perm(sc, sc, 0x3232);         // each doubled into an f16x2
            uint8_t* base = sA + (G & 1) * PF_A_STAGE;
            auto put = [&](uint32_t word, uint32_t s2, int half, int kb, int row) {
                uint32_t P[4], hi[4], lo[4];
                dq_word_h(word, P);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(hi[i]) : "r"(P[i]), "r"(s2));
                    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(lo[i]) : "r"(P[i]), "r"(s2), "r"(hi[i] ^ 0x80008000u));
                }
                *reinterpret_cast<uint4*>(base + half * 16384 + kb * 2048 + row * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(base + 32768 + half * 16384 + kb * 2048 + row * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            };
            // piece A: 16 nibbles of rowA, inputs 16*ut .. +15 of the group = k-blocks 2*ut, 2*ut + 1; piece B likewise
            put(q.x, sA2, halfA, 2 * ut, rowA); put(q.y, sA2, halfA, 2 * ut + 1, rowA);
            put(q.z, sB2, halfB, 2 * ut, rowB); put(q.w, sB2, halfB, 2 * ut + 1, rowB);
        };
        // issue the 16 MMAs of group G (one thread): D[half] += (A_hi + A_lo)[half] * B over the group's four K steps
        auto issue = [&](int G) {
            const int st = G & 1;
            const uint32_t aB = smem_u32(sA + st * PF_A_STAGE), bB = smem_u32(sB + (G % 3) * PF_B_STAGE);
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int hl = 0; hl < 2; hl++)
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_f16(tmem + (uint32_t)(h * PF_NMAX), umma_desc(aB + hl * 32768 + h * 16384 + ks * 4096, 2048, 128),
                                 umma_desc(bB + ks * 2 * (N * 16), N * 16, 128), idesc, G > 0 || hl > 0 || ks > 0);
            umma_commit(smem_u32(bars + st));
        };
        auto wait_mma = [&](int G) {  // MMAs of group G (and all before) done (bounded)
            uint32_t& ph = (G & 1) ? ph1 : ph0;
            if (!mbar_wait(smem_u32(bars + (G & 1)), ph, a.err, 3)) *s_fail = 1;
            ph ^= 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        };

        __syncthreads();  // the previous tile's readers are done with the stages, the ring and TMEM
        // prologue: raw groups 0..AHEAD and activations of groups 0, 1 on their way; group 0 unpacked and issued
        for (int G = 0; G <= PF_AHEAD && G < NG; G++) prefetch(G);
        fill_b(0); fill_b(1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // the scale pairs of group 0 were copied by other threads
        unpack(0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue(0); }
        for (int G = 0; G < NG; G++) {
            // group G is on the tensor core. Meanwhile: unpack group G+1, request what comes later.
            if (G >= 1) wait_mma(G - 1);   // frees A stage (G+1)&1 and B stage (G+2)%3
            if (G + 2 < NG) fill_b(G + 2);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (G + 1 + PF_AHEAD < NG) prefetch(G + 1 + PF_AHEAD);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 2;" ::: "memory");   // everything requested before this iteration has landed
            if (G + 1 < NG) unpack(G + 1);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (*s_fail) break;
            if (G + 1 < NG && tid == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue(G + 1); }
        }
        if (*s_fail) break;
        wait_mma(NG - 1);
        asm volatile("cp.async.wait_group 0;" ::: "memory");

        // epilogue. The thread reads row e_row of half e_half, columns e_ch*N/2 .. +N/2-1, 16 at a time.
        const int cbase = e_ch * (N >> 1);
        const uint32_t t0 = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(e_half * PF_NMAX + cbase);
        if (DOWN) {
            const int d = 256 * rt + 128 * e_half + e_row;
#pragma unroll
            for (int cb = 0; cb < 4; cb++) {
                if (cb * 16 < (N >> 1)) {
                    float v[16];
                    tmem_ld16(t0 + cb * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {   // parts == 2: columns (2j, 2j+1) = (hi, lo) of pair j
                        const int j = (cbase + cb * 16 + i) >> 1;
                        if (j < it.count) {
                            const moexb_pair pr = a.pairs[it.start + j];
                            a.ypair[(size_t)pr.p * EH + d] = pr.w * (v[i] + v[i + 1]);
                        }
                    }
                }
            }
        } else {
            // the up half hands its sums to the gate half through shared memory (the A stages are free now)
            float* ex = reinterpret_cast<float*>(sA);  // [column PF_NMAX][row 128]
            const bool two = a.parts == 2;
            if (e_half == 1) {
#pragma unroll
                for (int cb = 0; cb < 4; cb++) {
                    if (cb * 16 < (N >> 1)) {
                        float v[16];
                        tmem_ld16(t0 + cb * 16, v);
#pragma unroll
                        for (int i = 0; i < 16; i++) ex[(cbase + cb * 16 + i) * 128 + e_row] = v[i];
                    }
                }
            }
            __syncthreads();
            if (e_half == 0) {
                const int row = 128 * rt + e_row;
#pragma unroll
                for (int cb = 0; cb < 4; cb++) {
                    if (cb * 16 < (N >> 1)) {
                        float v[16];
                        tmem_ld16(t0 + cb * 16, v);
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const int col = cbase + cb * 16 + i;
                            const int j = two ? col >> 1 : col;
                            if (j < it.count && !(two && (i & 1))) {
                                float g = v[i], u = ex[col * 128 + e_row];
                                if (two) { g += v[(i + 1) & 15]; u += ex[(col + 1) * 128 + e_row]; }
                                const float val = g / (1.f + expf(-g)) * u;
                                const moexb_pair pr = a.pairs[it.start + j];
                                if (a.act32) a.act32[(size_t)pr.p * EI + row] = val;
                                uint16_t hi, lo;
                                split_hi_lo<true>(val, hi, lo);
                                uint16_t* dst = a.act_out + (size_t)pr.p * 2 * EI + perm8_pos(row);
                                dst[0] = hi; dst[EI] = lo;
                            }
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
}

template <int FMT, bool DOWN>
constexpr int pf_smem_bytes() { return 2 * PF_A_STAGE + 3 * PF_B_STAGE + PF_RING * PF_RAW + 64 + 1024; }

// x [rows][K] fp32 -> xs [rows][parts][K] fp16 in perm8 order: parts = 1 keeps fp16(x) (exact when x came from bf16 and is
// in fp16's normal range), parts = 2 adds lo = fp16(x - hi).
__global__ void split8_rows_k(const float* __restrict__ x, uint16_t* __restrict__ xs, int K, int parts, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t r = i / K; const int k = (int)(i % K);
    uint16_t hi, lo;
    split_hi_lo<true>(x[i], hi, lo);
    uint16_t* dst = xs + r * parts * K + perm8_pos(k);
    dst[0] = hi;
    if (parts == 2) dst[K] = lo;
}

}  // namespace moexb
