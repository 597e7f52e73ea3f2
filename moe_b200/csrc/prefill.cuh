// Grouped expert GEMM for prefill-size batches on the 5th-generation tensor cores (tcgen05.mma, weights and accumulators
// in tensor memory).
//
// One CTA of 512 threads owns a 256-row weight block of one expert (gate rows r..r+127 and the same up rows; or 256
// consecutive down rows) and one tile of up to 128 activation columns (tokens of that expert, as fp16: one column per
// token when the input is exactly bf16, hi + lo columns when it is fp32). Per 64-input scale group:
//   1. every thread takes 32 weights of one row (16 bytes of the tiled weight image, requested several groups earlier
//      with cp.async into a ring in shared memory), unpacks them to exact fp16 integers, multiplies by the group's fp16
//      scale and splits the product into hi = fp16(q*s) and lo = q*s - hi (one fused multiply-add; both halves together
//      are the exact weight), and writes them with tcgen05.st into tensor memory, where a thread's TMEM lane is its
//      weight row - the A operand never passes through shared memory; the group's activation rows (B operand) arrive in
//      shared memory with cp.async;
//   2. one thread issues 16 tcgen05.mma (M = 128, N = columns, K = 16, A from tensor memory; hi and lo weights x two
//      weight halves x four K steps) that accumulate over all groups in TMEM, and commits them to an mbarrier, which
//      frees the stage.
// The unpacking of group G+1 runs while the tensor core works on group G. After the last group every thread reads its
// row's sums out of TMEM (tcgen05.ld) for the epilogue. Every mbarrier wait is bounded; on a time-out the CTA still
// frees its TMEM and leaves. Tensor memory: columns 0-255 the two accumulators (128 columns each), 256-511 two stages of
// A (per stage: weight half x (hi, lo) x 32 columns = 64 inputs, two fp16 per column).
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
// The same with the A operand in tensor memory (lane = row, two fp16 per 32-bit column).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, bool accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
constexpr uint32_t UMMA_NEGATE_A = 1u << 13;
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
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

constexpr int PF_RING = 8;      // raw weight groups in flight (cp.async), each 8 KB of nibbles + the group's scales
constexpr int PF_AHEAD = 6;     // a group's raw bytes are requested this many groups before they are unpacked (2 <= AHEAD < RING)
constexpr int PF_RAW = 256 * 32 + 512;  // bytes of one ring slot: [slice 16][row 16][32 bytes = 64 nibbles] | [slice 16][row pair 8] x (fp16, fp16)
constexpr int PF_TMEM_COLS = 512;
constexpr int PF_TMEM_A = 256;  // first column of the A stages

// DOWN = false: weight block = gate rows 128*rt..+127 (half 0) and the same up rows (half 1); K = 2048 = 32 groups.
// DOWN = true : weight block = down rows 256*rt..+127 (half 0) and +128..+255 (half 1); K = 512 = 8 groups; parts = 2.
// One CTA per SM (the launch asks for more than half of the shared memory, and the CTA takes all 512 TMEM columns).
template <int FMT, bool DOWN>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_k(const PrefillArgs a) {
    static_assert(FMT == FMT_SYM_F16, "the grouped GEMM takes fp16 group scales; other formats use the streaming kernels");
    static_assert(PF_AHEAD >= 2 && PF_AHEAD < PF_RING, "ring depth");
    constexpr int GB = tl_group_bytes<FMT>(), SB = tl_slice_bytes<FMT>();
    constexpr int NG = DOWN ? EI / 64 : EH / 64;   // scale groups along K
    constexpr int RT = DOWN ? EH / 256 : EI / 128; // row blocks per expert
    constexpr int KB = DOWN ? EI : EH;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sB = smem;                                 // 3 stages x [k-block 8][column N][16 B]
    uint8_t* sR = sB + 3 * PF_B_STAGE;                  // ring of raw groups
    uint64_t* bars = reinterpret_cast<uint64_t*>(sR + PF_RING * PF_RAW);  // MMA-done barriers of the two A stages
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 2);
    int* s_fail = reinterpret_cast<int*>(s_tmem + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { mbar_init(smem_u32(bars), 2); mbar_init(smem_u32(bars + 1), 2); *s_fail = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "n"(PF_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;

    // copy role: slice cj of the 16 in the block, 16-byte unit cl = 4*g + t of the slice's group = 8 bytes of row g (inputs
    // 16t..16t+15 of the group) and 8 bytes of row g + 8
    const int cj = tid >> 5, cg = (tid & 31) >> 2, ct = tid & 3;
    // unpack role: a warp reaches only the TMEM lanes 32*(warp & 3)..+31, lane = weight row inside its half; the four
    // warps of a lane quarter split the two weight halves and the two 32-input halves of the group
    const int uq = warp & 3, uh = warp >> 3, ukh = (warp >> 2) & 1, ui = 32 * uq + lane;
    const int uj = DOWN ? 8 * uh + (ui >> 4) : ui >> 3, um = DOWN ? ui & 15 : (ui & 7) + 8 * uh;   // slice and row of the slice
    const uint32_t lane_base = (uint32_t)(32 * uq) << 16;
    // epilogue role: row ui of both halves, column quarter ecq
    const int ecq = warp >> 2;
    uint32_t ph0 = 0, ph1 = 0;
    pdl_wait();
    pdl_trigger();
    const int ntiles = *a.ntiles * RT;

    // What a tile's copies, MMAs and epilogue need to know. The first groups of the NEXT tile are requested before the epilogue
    // of the current one (the ring and the activation stages are free by then), so that the start of a tile does not wait for
    // a memory round trip with nothing else to do; hence two of these are alive at a time.
    struct Tile {
        moexb_pair_item it; int rt, ncol, N;
        const uint16_t* xcol0; const uint16_t* xcol1;   // the thread's two copy units of an activation stage (null = padding column)
        int d0, d1;                                     // their byte offsets inside a B stage, -1 = none
    };
    auto setup = [&](int tile) {
        Tile p;
        p.it = a.tiles[tile / RT];
        p.rt = tile % RT;
        p.ncol = p.it.count * a.parts;                 // real activation columns
        p.N = (p.ncol + 31) & ~31;                     // MMA N: a multiple of 32, so each column quarter is a multiple of 8
        // activation rows of this tile's columns: copy unit u = (column c, k-block kb of 8 inputs), N*8 units, threads take
        // u = tid and tid + 512. kb = (u & 1) + 2 * ((u >> 1) / N), c = (u >> 1) % N: a lane pair reads one 32-byte sector of a
        // column, consecutive pairs write consecutive 16-byte rows of the core-matrix layout.
        p.xcol0 = nullptr; p.xcol1 = nullptr; p.d0 = -1; p.d1 = -1;
        const int N = p.N, u0 = tid, u1 = tid + PF_THREADS;
        if (u0 < N * 8) {
            const int c = (u0 >> 1) % N, kb = (u0 & 1) + 2 * ((u0 >> 1) / N);
            p.d0 = kb * (N * 16) + c * 16;
            if (c < p.ncol) { const moexb_pair pr = a.pairs[p.it.start + c / a.parts]; p.xcol0 = a.xs + ((size_t)(DOWN ? pr.p : pr.t) * a.parts + c % a.parts) * KB + kb * 8; }
        }
        if (u1 < N * 8) {
            const int c = (u1 >> 1) % N, kb = (u1 & 1) + 2 * ((u1 >> 1) / N);
            p.d1 = kb * (N * 16) + c * 16;
            if (c < p.ncol) { const moexb_pair pr = a.pairs[p.it.start + c / a.parts]; p.xcol1 = a.xs + ((size_t)(DOWN ? pr.p : pr.t) * a.parts + c % a.parts) * KB + kb * 8; }
        }
        return p;
    };
    // request group G's raw bytes: the thread's unit as two 8-byte pieces, each to its row's 32 bytes of the ring slot
    // (so that the unpacking reads one row with one 16-byte load), and (one thread per row pair) the pair's two scales
    auto prefetch = [&](const Tile& p, int G) {
        const uint8_t* gb = p.it.slot + (size_t)(DOWN ? 256 + 16 * p.rt + cj : (16 * p.rt + cj) * 4 + (G >> 3)) * SB + (G & 7) * GB;
        uint8_t* slot = sR + (G % PF_RING) * PF_RAW;
        const uint8_t* src = gb + (4 * cg + ct) * 16;
        cp_async8(smem_u32(slot + (cj * 16 + cg) * 32 + ct * 8), src);
        cp_async8(smem_u32(slot + (cj * 16 + cg + 8) * 32 + ct * 8), src + 8);
        if (ct == 0) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(slot + 8192 + (cj * 8 + cg) * 4)), "l"(gb + 512 + 4 * cg) : "memory");
    };
    // request group G's activation rows into B stage G % 3
    auto fill_b = [&](const Tile& p, int G) {
        uint8_t* bb = sB + (G % 3) * PF_B_STAGE;
        if (p.d0 >= 0) { if (p.xcol0) cp_async16(smem_u32(bb + p.d0), p.xcol0 + G * 64); else *reinterpret_cast<uint4*>(bb + p.d0) = make_uint4(0, 0, 0, 0); }
        if (p.d1 >= 0) { if (p.xcol1) cp_async16(smem_u32(bb + p.d1), p.xcol1 + G * 64); else *reinterpret_cast<uint4*>(bb + p.d1) = make_uint4(0, 0, 0, 0); }
    };
    // the first copies of a tile: raw groups 0..AHEAD and the activation rows of groups 0 and 1
    auto prime = [&](const Tile& p) {
        for (int G = 0; G <= PF_AHEAD && G < NG; G++) prefetch(p, G);
        fill_b(p, 0); fill_b(p, 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    Tile cur;
    bool primed = false;   // the copies of `cur` have been requested already (during the epilogue of the tile before)
    for (int tile = blockIdx.x; tile < ntiles && !*s_fail; tile += gridDim.x) {
        if (!primed) cur = setup(tile);
        const moexb_pair_item it = cur.it;
        const int rt = cur.rt, N = cur.N;
        const uint32_t idesc = umma_idesc_f16(128, N);

        // unpack 32 weights of this thread's row of group G (the raw bytes have landed and are visible) into A stage G & 1 in
        // tensor memory: nh = -fp16(q*s) (the MMA negates it back) and lo = q*s + nh, two fp16 per column
        auto unpack = [&](int G) {
            const uint8_t* slot = sR + (G % PF_RING) * PF_RAW;
            const uint4 q = *reinterpret_cast<const uint4*>(slot + (uj * 16 + um) * 32 + ukh * 16);
            const uint32_t s1 = *reinterpret_cast<const uint16_t*>(slot + 8192 + (uj * 8 + (um & 7)) * 4 + 2 * (um >> 3));
            const uint32_t s2 = s1 | (s1 << 16), ns2 = s2 ^ 0x80008000u;
            uint32_t nh[16], lo[16];
            auto put = [&](uint32_t word, int at) {
                uint32_t P[4];
                dq_word_h(word, P);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(nh[at + i]) : "r"(P[i]), "r"(ns2));
                    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(lo[at + i]) : "r"(P[i]), "r"(s2), "r"(nh[at + i]));
                }
            };
            put(q.x, 0); put(q.y, 4); put(q.z, 8); put(q.w, 12);
            const uint32_t col = (uint32_t)(PF_TMEM_A + (G & 1) * 128 + uh * 64 + ukh * 16);
            tmem_st16(tmem + lane_base + col, nh);
            tmem_st16(tmem + lane_base + col + 32, lo);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        };
        // issue the 8 MMAs of weight half h of group G (one thread per half - issuing an MMA costs its thread about 90 cycles
        // whatever N is, so the two halves are issued from two warps): D[h] += (-A_nh + A_lo)[h] * B over the four K steps
        auto issue = [&](int G, int h) {
            const uint32_t aT = tmem + (uint32_t)(PF_TMEM_A + (G & 1) * 128), bB = smem_u32(sB + (G % 3) * PF_B_STAGE);
#pragma unroll
            for (int hl = 0; hl < 2; hl++)
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    umma_f16_ts(tmem + (uint32_t)(h * PF_NMAX), aT + (uint32_t)(h * 64 + hl * 32 + ks * 8),
                                umma_desc(bB + ks * 2 * (N * 16), N * 16, 128), hl ? idesc : (idesc | UMMA_NEGATE_A), G > 0 || hl > 0 || ks > 0);
            umma_commit(smem_u32(bars + (G & 1)));
        };
        auto wait_mma = [&](int G) {  // MMAs of group G (and all before) done (bounded)
            uint32_t& ph = (G & 1) ? ph1 : ph0;
            if (!mbar_wait(smem_u32(bars + (G & 1)), ph, a.err, 3)) *s_fail = 1;
            ph ^= 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        };

        __syncthreads();  // the previous tile's readers are done with the B stages, the ring and TMEM
        // prologue: raw groups 0..AHEAD and activations of groups 0, 1 on their way; group 0 unpacked and issued
        if (!primed) prime(cur);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();  // every thread's copies have landed: the rows are read by other threads than copied them
        unpack(0);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if ((tid & ~32) == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue(0, tid >> 5); }
#pragma unroll 8
        for (int G = 0; G < NG; G++) {
            // group G is on the tensor core. Meanwhile: unpack group G+1 (visible since the previous barrier), request what
            // comes later, and make sure that everything requested before this iteration has landed before the next barrier.
            if (G >= 1) wait_mma(G - 1);   // frees A stage (G+1)&1 and B stage (G+2)%3
            if (G + 2 < NG) fill_b(cur, G + 2);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (G + 1 + PF_AHEAD < NG) prefetch(cur, G + 1 + PF_AHEAD);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (G + 1 < NG) unpack(G + 1);
            asm volatile("cp.async.wait_group 2;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (*s_fail) break;
            if (G + 1 < NG && (tid & ~32) == 0) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); issue(G + 1, tid >> 5); }
        }
        if (*s_fail) break;
        wait_mma(NG - 1);
        // every MMA of this tile is done and every raw group unpacked: the ring and the activation stages are free, and the
        // next tile's first copies travel while this tile's sums are read out and stored
        primed = false;
        Tile nxt = cur;
        if (!*s_fail && tile + (int)gridDim.x < ntiles) { nxt = setup(tile + gridDim.x); prime(nxt); primed = true; }

        // epilogue. The thread reads row ui of both halves, columns ecq*N/4 .. +N/4-1, 8 at a time.
        const int cbase = ecq * (N >> 2);
        const uint32_t t0 = tmem + lane_base + (uint32_t)cbase;
        const bool two = a.parts == 2;
#pragma unroll
        for (int cb = 0; cb < 4; cb++) {
            if (cb * 8 < (N >> 2)) {
                float v0[8], v1[8];
                tmem_ld8(t0 + cb * 8, v0);
                tmem_ld8(t0 + PF_NMAX + cb * 8, v1);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int col = cbase + cb * 8 + i;
                    const int j = (DOWN || two) ? col >> 1 : col;
                    if (j >= it.count || ((DOWN || two) && (i & 1))) continue;
                    float x0 = v0[i], x1 = v1[i];
                    if (DOWN || two) { x0 += v0[i | 1]; x1 += v1[i | 1]; }   // columns (2j, 2j+1) = (hi, lo) of pair j
                    const moexb_pair pr = a.pairs[it.start + j];
                    if (DOWN) {
                        const int d = 256 * rt + ui;
                        a.ypair[(size_t)pr.p * EH + d] = pr.w * x0;
                        a.ypair[(size_t)pr.p * EH + d + 128] = pr.w * x1;
                    } else {
                        const int row = 128 * rt + ui;
                        const float val = x0 / (1.f + expf(-x0)) * x1;
                        if (a.act32) a.act32[(size_t)pr.p * EI + row] = val;
                        uint16_t hi, lo;
                        split_hi_lo<true>(val, hi, lo);
                        uint16_t* dst = a.act_out + (size_t)pr.p * 2 * EI + perm8_pos(row);
                        dst[0] = hi; dst[EI] = lo;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        cur = nxt;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // none of this thread's copies is in flight when the CTA leaves
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(PF_TMEM_COLS) : "memory");
}

template <int FMT, bool DOWN>
constexpr int pf_smem_bytes() { return 3 * PF_B_STAGE + PF_RING * PF_RAW + 64 + 1024; }
static_assert(pf_smem_bytes<FMT_SYM_F16, false>() > 114 * 1024, "more than half of an SM's shared memory, so that two CTAs (2 x 512 TMEM columns) never share an SM");

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
