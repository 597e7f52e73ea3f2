// Streaming expert kernels for 1..64 tokens: the bandwidth-bound skinny GEMM of the decode-size path.
//
// One kernel template serves both projections (gate/up with the SwiGLU epilogue, down with the routing-weight epilogue).
// A persistent CTA has one producer warp and NW consumer warps. The producer pulls tiles from a global queue and streams
// packed int4 rows through a ring of shared-memory stages with cp.async.bulk (the TMA bulk-copy engine), one 256-byte
// row piece (512 weights = 8 scale groups) per copy, 64 pieces per stage, completion counted on an mbarrier; the scale
// bytes of the same pieces follow with 16-byte cp.async copies on the same barrier. Consumer warps read 16 nibbles per
// lane and row with 8-byte shared loads (the piece stride of 288 bytes keeps them conflict-free), turn them into exact
// bf16 integers in registers (one lop3 + one bf16x2 subtract per two weights) and feed mma.sync.m16n8k16 with the
// activations as the 8-wide operand. Activations arrive as bf16 hi + lo halves (16 significand bits) in adjacent
// columns, so a lane adds its two accumulator columns to get one token's value; the fp32 scale of each 64-weight group
// is applied to the group's partial sum on the accumulators, so weights stay exact. Sub-items hold at most 4
// (token, expert) pairs = 8 columns = one n8 tile; experts with more tokens are split and re-stream their weights
// from L2. The 8 activation columns of the current sub-item sit in shared memory (the consumer warps copy them in when
// the sub-item changes); every CTA works on a contiguous range of tiles, so that happens once or twice per launch.
//
// k-slot permutation: within a 64-weight group lane t of a quad owns nibbles 16t..16t+15 (two 32-bit words w = 0, 1);
// the bf16x2 register P[i] of word w holds nibbles (8w+i, 8w+i+4). MMA (w, h) uses P[2h] for k-slots (2t, 2t+1) and
// P[2h+1] for k-slots (2t+8, 2t+9). The activation rows are stored in the matching order: position
// G*64 + w*32 + t*8 + e' holds input k = G*64 + 16t + 8w + e with e' = ((e & 3) << 1) | (e >> 2), so the four k-values
// of both MMAs of a word are one 16-byte load per lane (see split_pos).
#pragma once
#include "common.cuh"

namespace moexb {

constexpr int ST_PIECE = 256;    // bytes of one row piece: 512 int4 weights
constexpr int ST_STRIDE = 288;   // piece stride in shared memory (rows g..g+3 of a half-warp land on distinct banks)
constexpr int ST_SC_PER_PIECE = 48;  // zero point: 16 x [sc, mn] + 2 x (d, dm) = 40 scale bytes per piece, kept 16-byte aligned
constexpr int ST_MAXP = 4;       // pairs per sub-item: 4 x (hi, lo) = the 8 columns of one MMA tile
constexpr int ST_WAIT_LIMIT = 1 << 22;

enum : int { ST_ERR_NONE = 0, ST_ERR_FULL_WAIT = 1, ST_ERR_EMPTY_WAIT = 2 };

template <int FMT> constexpr int st_scale_bytes() { return FMT == FMT_SYM_F16 ? 16 : FMT == FMT_SYM_F32 ? 32 : ST_SC_PER_PIECE; }
template <int NW> constexpr int st_pieces() { return 16 * NW; }
template <int FMT, int NW> constexpr int st_slot_bytes() { return st_pieces<NW>() * (ST_STRIDE + st_scale_bytes<FMT>()); }
// activation columns in shared memory: 8 columns of K bf16, column stride K*2 + 64 bytes (conflict-free 16-byte reads)
template <bool DOWN> constexpr int st_bcol_bytes() { return (DOWN ? EI : EH) * 2 + 64; }
template <int FMT, bool DOWN, int NW, int STAGES> constexpr int st_smem_bytes() { return STAGES * st_slot_bytes<FMT, NW>() + 8 * st_bcol_bytes<DOWN>() + 256 + 8; }

// Position of input k inside a permuted activation row (see the header comment).
__host__ __device__ constexpr int split_pos(int k) {
    const int G = k >> 6, kl = k & 63, t = kl >> 4, w = (kl >> 3) & 1, e = kl & 7;
    return G * 64 + w * 32 + t * 8 + (((e & 3) << 1) | (e >> 2));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls, records why, and lets the caller leave the kernel.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code, int limit = ST_WAIT_LIMIT) {
    for (int i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Eight nibbles of q -> four bf16x2 registers P[i] = (nibble i, nibble i+4) as exact integers: (x & 0x000F000F) ^ C
// puts each nibble into the mantissa of 128.0 (C also flips bit 3 of two's-complement nibbles, turning v into v + 8),
// and subtracting 128 (or 136) leaves the integer.
template <bool SIGNED>
__device__ __forceinline__ void dq_word(uint32_t q, uint32_t (&P)[4]) {
    constexpr uint32_t C = SIGNED ? 0x43084308u : 0x43004300u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t r;
        asm("lop3.b32 %0, %1, 0x000F000F, %2, 0x6A;" : "=r"(r) : "r"(q >> (4 * i)), "r"(C));
        asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(P[i]) : "r"(r), "r"(C));
    }
}

// The same for fp16 operands, with one shift per word instead of three: fp16 has a 10-bit mantissa, so a nibble can also
// be picked up at bit 4 of its half-word ((x & 0x00F000F0) ^ C' = 1024 + 16 * (v + 8)) and one fused multiply-add
// (* 1/16, - 72) turns that into v exactly. Only two's-complement nibbles (the symmetric formats).
__device__ __forceinline__ void dq_word_h(uint32_t q, uint32_t (&P)[4]) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const uint32_t x = q >> (8 * j);
        uint32_t r0, r1;
        asm("lop3.b32 %0, %1, 0x000F000F, 0x64086408, 0x6A;" : "=r"(r0) : "r"(x));
        asm("lop3.b32 %0, %1, 0x00F000F0, 0x64806480, 0x6A;" : "=r"(r1) : "r"(x));
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(P[2 * j]) : "r"(r0), "r"(0x64086408u));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(P[2 * j + 1]) : "r"(r1), "r"(0x2C002C00u), "r"(0xD480D480u));
    }
}

// hi + lo halves of v as 16-bit patterns: fp16 (22 significand bits together) or bf16 (16 bits, full fp32 range)
template <bool F16>
__device__ __forceinline__ void split_hi_lo(float v, uint16_t& hi, uint16_t& lo) {
    if constexpr (F16) {
        const __half h = __float2half_rn(v), l = __float2half_rn(v - __half2float(h));
        hi = __half_as_ushort(h); lo = __half_as_ushort(l);
    } else {
        const __nv_bfloat16 h = __float2bfloat16_rn(v), l = __float2bfloat16_rn(v - __bfloat162float(h));
        hi = __bfloat16_as_ushort(h); lo = __bfloat16_as_ushort(l);
    }
}

// d = a * b (no accumulator input: the zero operand is an immediate, so nothing has to be cleared first)
__device__ __forceinline__ void mma_bf16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool F16>
__device__ __forceinline__ void mma_16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, bool first) {
    if constexpr (F16) {
        if (first) asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
        else asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                          : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        if (first) mma_bf16_first(d, a0, a1, a2, a3, b0, b1); else mma_bf16(d, a0, a1, a2, a3, b0, b1);
    }
}

struct StreamArgs {
    const moexb_pair_item* subs;  // sub-items: at most ST_MAXP pairs each
    const int* nsub;              // device count of sub-items
    const moexb_pair* pairs;
    const __nv_bfloat16* xs;      // gate/up: activations [token][2][H] (hi, lo), permuted; down: act [pair p][2][I]
    float* act32;                 // gate/up: optional fp32 copy of act [p][I]
    __nv_bfloat16* act_split;     // gate/up output [p][2][I], permuted
    float* ypair;                 // down output [p][H]
    int* err;                     // error word: first failed wait
};

struct StageInfo { int sub, tin, ks, first; };

// DOWN = false: tile = 8*NW gate rows + the same up rows, 4 stages (K slices of 512); act = silu(gate) * up.
// DOWN = true : tile = 16*NW down rows, 1 stage (K = 512); ypair = w * (down . act).
// CTA c of G works on tiles [c*U/G, (c+1)*U/G) of the U = nsub * TILES tiles, in order.
template <int FMT, bool DOWN, int NW, int STAGES>
__global__ void __launch_bounds__((NW + 1) * 32) stream_k(const StreamArgs a) {
    constexpr int PIECES = st_pieces<NW>();
    constexpr int SCB = st_scale_bytes<FMT>();
    constexpr int SLOT = st_slot_bytes<FMT, NW>();
    constexpr int KS = DOWN ? 1 : 4;                                  // stages per tile
    constexpr int TILES = DOWN ? EH / (16 * NW) : EI / (8 * NW);      // tiles per sub-item
    constexpr int KB = DOWN ? EI : EH;                                // inputs per activation row
    constexpr int BCOL = st_bcol_bytes<DOWN>();
    constexpr bool Z = FMT == FMT_ZP;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* bsm = smem + STAGES * SLOT;                                     // 8 activation columns
    uint64_t* bars = reinterpret_cast<uint64_t*>(bsm + 8 * BCOL);            // full[STAGES], empty[STAGES], consumer barrier
    StageInfo* info = reinterpret_cast<StageInfo*>(bars + 2 * STAGES + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_u32(bars + s), 33); mbar_init(smem_u32(bars + STAGES + s), NW); }
        mbar_init(smem_u32(bars + 2 * STAGES), NW);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long U = (long long)*a.nsub * TILES;
    const int tile0 = (int)(U * blockIdx.x / gridDim.x), tile1 = (int)(U * (blockIdx.x + 1) / gridDim.x);

    if (warp == NW) {
        // ---- producer: one warp streams the tiles' row pieces and scale bytes into the ring ----
        int s = 0; uint32_t ph = 0;
        uint32_t armed = 0, armed_ph = 0;   // per stage: a fill was requested, and the parity its full barrier completes with
        // a wait ran out: wait (bounded) for the fills already requested, so that no copy is in flight into this CTA's
        // shared memory when the producer leaves; the consumers run out of polls on their side
        auto give_up = [&]() {
            for (int i = 0; i < STAGES; i++)
                if (armed >> i & 1) mbar_wait(smem_u32(bars + i), armed_ph >> i & 1, a.err, ST_ERR_EMPTY_WAIT);
        };
        for (int tile = tile0; tile <= tile1; tile++) {
            const bool done = tile == tile1;  // one empty stage after the last tile tells the consumers to stop
            const int sub = done ? -1 : tile / TILES, tin = done ? 0 : tile % TILES;
            const uint8_t* slot = done ? nullptr : a.subs[sub].slot;
            for (int ks = 0; ks < (done ? 1 : KS); ks++) {
                const uint32_t full = smem_u32(bars + s), empty = smem_u32(bars + STAGES + s);
                if (!mbar_wait(empty, ph ^ 1, a.err, ST_ERR_EMPTY_WAIT)) { give_up(); return; }
                armed |= 1u << s; armed_ph = (armed_ph & ~(1u << s)) | (ph << s);
                if (lane == 0) {
                    info[s] = {sub, tin, ks, ks == 0};
                    mbar_arrive_expect_tx(full, done ? 0 : PIECES * ST_PIECE);
                }
                __syncwarp();
                if (!done) {
                    const uint32_t base = smem_u32(smem + s * SLOT);
#pragma unroll
                    for (int i = 0; i < PIECES / 32; i++) {
                        const int pi = lane + 32 * i;
                        size_t c0;  // first 32-weight chunk of the piece inside the blob
                        const uint8_t* src;
                        if (DOWN) {
                            const int d = tin * (16 * NW) + pi;
                            src = slot + DOWN_Q_OFF + (size_t)d * (EI / 2);
                            c0 = DOWN_C_OFF + (size_t)d * (EI / 32);
                        } else {
                            const int wq = pi >> 4, m = pi & 15;
                            const size_t row = (size_t)(m < 8 ? 0 : EI) + tin * (8 * NW) + wq * 8 + (m & 7);  // row in [gate | up]
                            src = slot + row * (EH / 2) + ks * ST_PIECE;
                            c0 = row * (EH / 32) + ks * 16;
                        }
                        bulk_g2s(base + pi * ST_STRIDE, src, ST_PIECE, full);
                        const uint32_t sdst = base + PIECES * ST_STRIDE + pi * SCB;
                        const uint8_t* sp = slot + Q_BYTES;
                        if constexpr (FMT == FMT_SYM_F16) cp_async16(sdst, sp + (c0 / 2) * 2);
                        else if constexpr (FMT == FMT_SYM_F32) { cp_async16(sdst, sp + (c0 / 2) * 4); cp_async16(sdst + 16, sp + (c0 / 2) * 4 + 16); }
                        else { cp_async16(sdst, sp + c0 * 2); cp_async16(sdst + 16, sp + c0 * 2 + 16); cp_async8(sdst + 32, sp + CHUNKS * 2 + (c0 / 8) * 4); }
                    }
                }
                cp_async_arrive_noinc(full);
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        // drain: every slot released, so no copy is in flight when the CTA exits
        for (int i = 0; i < STAGES; i++) {
            if (!mbar_wait(smem_u32(bars + STAGES + s), ph ^ 1, a.err, ST_ERR_EMPTY_WAIT)) { give_up(); return; }
            if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        return;
    }

    // ---- consumers ----
    const int g = lane >> 2, t = lane & 3, wq = warp;
    const int ctid = threadIdx.x;  // 0 .. NW*32-1
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int cur_sub = -1, n = 0, start = 0;
    int s = 0; uint32_t ph = 0, cph = 0;
    const uint8_t* bcol = bsm + g * BCOL + t * 16;  // the lane's activation column (pair slot g >> 1, part g & 1)
    // barrier over the consumer warps as an mbarrier with a bounded wait: a warp that gave up on a stage never arrives,
    // and the others then run out of polls here instead of waiting for it for ever
    auto consumer_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bars + 2 * STAGES));
        const bool ok = mbar_wait(smem_u32(bars + 2 * STAGES), cph, a.err, ST_ERR_FULL_WAIT);
        cph ^= 1;
        return ok;
    };
    while (true) {
        const uint32_t full = smem_u32(bars + s), empty = smem_u32(bars + STAGES + s);
        if (!mbar_wait(full, ph, a.err, ST_ERR_FULL_WAIT)) return;
        const StageInfo inf = info[s];
        if (inf.sub < 0) { __syncwarp(); if (lane == 0) mbar_arrive(empty); break; }
        if (inf.sub != cur_sub) {
            // new sub-item: all consumer warps swap the activation columns (the weights keep streaming meanwhile)
            cur_sub = inf.sub;
            const moexb_pair_item it = a.subs[cur_sub];
            n = it.count; start = it.start;
            if (!consumer_sync()) return;  // everyone is done with the old columns
            constexpr int CHUNKS16 = KB * 2 / 16;                        // 16-byte chunks per column
            for (int i = ctid; i < 2 * n * CHUNKS16; i += NW * 32) {
                const int col = i / CHUNKS16, ch = i % CHUNKS16;
                const moexb_pair pr = a.pairs[start + (col >> 1)];
                const size_t r = DOWN ? (size_t)pr.p : (size_t)pr.t;
                cp_async16(smem_u32(bsm + col * BCOL + ch * 16), a.xs + (r * 2 + (col & 1)) * KB + ch * 8);
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
            if (!consumer_sync()) return;
        }
        if (inf.first) acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        const uint8_t* st = smem + s * SLOT;
        const int pa = wq * 16 + g, pb = pa + 8;  // the lane's two row pieces: A rows g and g + 8
        const uint8_t *sca = st + PIECES * ST_STRIDE + pa * SCB, *scb = st + PIECES * ST_STRIDE + pb * SCB;
        const uint8_t *qpa = st + pa * ST_STRIDE + t * 8, *qpb = st + pb * ST_STRIDE + t * 8;
        const uint8_t* bp = bcol + inf.ks * 1024;  // 8 groups of 128 bytes per stage
#pragma unroll 4
        for (int G = 0; G < 8; G++) {
            const uint2 qa = *reinterpret_cast<const uint2*>(qpa + G * 32);
            const uint2 qb = *reinterpret_cast<const uint2*>(qpb + G * 32);
            const uint4 B0 = *reinterpret_cast<const uint4*>(bp + G * 128), B1 = *reinterpret_cast<const uint4*>(bp + G * 128 + 64);
            uint32_t Pa[2][4], Pb[2][4];
            dq_word<!Z>(qa.x, Pa[0]); dq_word<!Z>(qa.y, Pa[1]);
            dq_word<!Z>(qb.x, Pb[0]); dq_word<!Z>(qb.y, Pb[1]);
            if constexpr (!Z) {
                float sa, sb;
                if constexpr (FMT == FMT_SYM_F16) { sa = __half2float(reinterpret_cast<const __half*>(sca)[G]); sb = __half2float(reinterpret_cast<const __half*>(scb)[G]); }
                else { sa = reinterpret_cast<const float*>(sca)[G]; sb = reinterpret_cast<const float*>(scb)[G]; }
                float c[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};  // two chains, so consecutive MMAs do not wait on each other
                mma_bf16(c, Pa[0][0], Pb[0][0], Pa[0][1], Pb[0][1], B0.x, B0.y);
                mma_bf16(e, Pa[0][2], Pb[0][2], Pa[0][3], Pb[0][3], B0.z, B0.w);
                mma_bf16(c, Pa[1][0], Pb[1][0], Pa[1][1], Pb[1][1], B1.x, B1.y);
                mma_bf16(e, Pa[1][2], Pb[1][2], Pa[1][3], Pb[1][3], B1.z, B1.w);
                acc[0] = fmaf(c[0] + e[0], sa, acc[0]); acc[1] = fmaf(c[1] + e[1], sa, acc[1]);
                acc[2] = fmaf(c[2] + e[2], sb, acc[2]); acc[3] = fmaf(c[3] + e[3], sb, acc[3]);
            } else {
                // zero point: each 32-weight chunk has its own (s, m), w = s*u + m, so a group is two partial sums
                // s_c * sum(u x) + m_c * sum(x). Lanes t = 0,1 hold chunk 2G, lanes t = 2,3 chunk 2G+1, and an MMA mixes
                // the quad's k-slots, so the chunks are separated by zeroing the other half's nibbles; sum(x) comes
                // from an all-ones A fragment.
                const float2 dda = __half22float2(*reinterpret_cast<const __half2*>(sca + 32 + (G >> 2) * 4));
                const float2 ddb = __half22float2(*reinterpret_cast<const __half2*>(scb + 32 + (G >> 2) * 4));
#pragma unroll
                for (int hc = 0; hc < 2; hc++) {
                    const bool mine = (t >> 1) == hc;
                    float c[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t one = mine ? 0x3F803F80u : 0u;
                    mma_bf16(c, mine ? Pa[0][0] : 0u, mine ? Pb[0][0] : 0u, mine ? Pa[0][1] : 0u, mine ? Pb[0][1] : 0u, B0.x, B0.y);
                    mma_bf16(c, mine ? Pa[0][2] : 0u, mine ? Pb[0][2] : 0u, mine ? Pa[0][3] : 0u, mine ? Pb[0][3] : 0u, B0.z, B0.w);
                    mma_bf16(c, mine ? Pa[1][0] : 0u, mine ? Pb[1][0] : 0u, mine ? Pa[1][1] : 0u, mine ? Pb[1][1] : 0u, B1.x, B1.y);
                    mma_bf16(c, mine ? Pa[1][2] : 0u, mine ? Pb[1][2] : 0u, mine ? Pa[1][3] : 0u, mine ? Pb[1][3] : 0u, B1.z, B1.w);
                    mma_bf16(c1, one, one, one, one, B0.x, B0.y); mma_bf16(c1, one, one, one, one, B0.z, B0.w);
                    mma_bf16(c1, one, one, one, one, B1.x, B1.y); mma_bf16(c1, one, one, one, one, B1.z, B1.w);
                    const int ch = 2 * G + hc;
                    const float s_a = dda.x * (float)sca[2 * ch], m_a = dda.y * (float)(int8_t)sca[2 * ch + 1];
                    const float s_b = ddb.x * (float)scb[2 * ch], m_b = ddb.y * (float)(int8_t)scb[2 * ch + 1];
                    acc[0] += fmaf(s_a, c[0], m_a * c1[0]); acc[1] += fmaf(s_a, c[1], m_a * c1[1]);
                    acc[2] += fmaf(s_b, c[2], m_b * c1[2]); acc[3] += fmaf(s_b, c[3], m_b * c1[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty);
        if (inf.ks == KS - 1 && t < n) {
            // epilogue: the lane's columns 2t (hi) and 2t+1 (lo) belong to pair slot t
            const moexb_pair pr = a.pairs[start + t];
            const float va = acc[0] + acc[1], vb = acc[2] + acc[3];
            if (DOWN) {
                const int d = inf.tin * (16 * NW) + wq * 16 + g;
                a.ypair[(size_t)pr.p * EH + d] = pr.w * va;
                a.ypair[(size_t)pr.p * EH + d + 8] = pr.w * vb;
            } else {
                const int r = inf.tin * (8 * NW) + wq * 8 + g;
                const float v = va / (1.f + expf(-va)) * vb;
                if (a.act32) a.act32[(size_t)pr.p * EI + r] = v;
                const __nv_bfloat16 hi = __float2bfloat16_rn(v), lo = __float2bfloat16_rn(v - __bfloat162float(hi));
                __nv_bfloat16* dst = a.act_split + (size_t)pr.p * 2 * EI + split_pos(r);
                dst[0] = hi; dst[EI] = lo;
            }
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
    }
}

// x [rows][K] fp32 -> xs [rows][2][K] 16-bit: hi and lo halves (see split_hi_lo), both in the permuted order of split_pos.
template <bool F16>
__global__ void split_rows_k(const float* __restrict__ x, uint16_t* __restrict__ xs, int K, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t r = i / K; const int k = (int)(i % K);
    uint16_t hi, lo;
    split_hi_lo<F16>(x[i], hi, lo);
    uint16_t* dst = xs + r * 2 * K + split_pos(k);
    dst[0] = hi; dst[K] = lo;
}

// One row of D = 2048 floats held 8 per thread (thread i: elements 4i..4i+3 and 1024+4i..1024+4i+3): the sum of squares
// in the pinned order of rmsnorm_rows_k, then the normalised row as fp32 (for the router) and as bf16 hi + lo in the
// permuted order (for the streaming kernels).
// lo_off: distance (elements) from the hi row to the lo row of the split.
// 1 / sqrt(mean(v^2) + eps) of the row, the sum of squares in the pinned order (all 256 threads of the block call it).
__device__ __forceinline__ float row_rms_scale(const float (&v)[8], float eps) {
    __shared__ float part[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    return 1.f / sqrtf(tot / (float)EH + eps);
}
// The row times r as fp32 into xn and, when xs is given, as 16-bit hi + lo in the permuted order into xs (hi) and xs + lo_off (lo).
template <bool F16>
__device__ __forceinline__ void scaled_split_row(const float (&v)[8], float r, float* __restrict__ xn, uint16_t* __restrict__ xs, int lo_off = EH) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int k0 = 1024 * h + 4 * threadIdx.x;
        float4 o = make_float4(v[4 * h] * r, v[4 * h + 1] * r, v[4 * h + 2] * r, v[4 * h + 3] * r);
        *reinterpret_cast<float4*>(xn + k0) = o;
        if (!xs) continue;
        const float f[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint16_t hi, lo;
            split_hi_lo<F16>(f[i], hi, lo);
            const int pos = split_pos(k0 + i);
            xs[pos] = hi; xs[lo_off + pos] = lo;
        }
    }
}
template <bool F16>
__device__ __forceinline__ void norm_split_row(const float (&v)[8], float* __restrict__ xn, uint16_t* __restrict__ xs, float eps, int lo_off = EH) {
    scaled_split_row<F16>(v, row_rms_scale(v, eps), xn, xs, lo_off);
}

// xn[t] = rmsnorm(x[t]) and its bf16 split, one block of 256 per row (H = 2048).
template <bool F16>
__global__ void __launch_bounds__(256) rmsnorm_split_k(const float* __restrict__ x, float* __restrict__ xn, uint16_t* __restrict__ xs, float eps) {
    const size_t t = blockIdx.x;
    float v[8];
    const float4 a = *reinterpret_cast<const float4*>(x + t * EH + 4 * threadIdx.x), b = *reinterpret_cast<const float4*>(x + t * EH + 1024 + 4 * threadIdx.x);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    norm_split_row<F16>(v, xn + t * EH, xs + t * 2 * EH, eps);
}

// The end of a layer in one pass over the token's row: moe[t] = sum_{r<K} ypair[t*K+r] in rank order (+ extra[t]: the
// shared expert's row), out[t] = x[t] + moe[t] when x is given (the residual block) else moe[t]; and, when xn_next is
// given, the next layer's normalised input and its bf16 split straight from the registers. One block of 256 per token.
template <bool F16>
__global__ void __launch_bounds__(256) reduce_residual_norm_k(const float* __restrict__ ypair, const float* __restrict__ extra, const float* __restrict__ x,
                                                              float* __restrict__ out, int K, float* __restrict__ xn_next,
                                                              uint16_t* __restrict__ xs_next, float eps, int ex0, int ex1,
                                                              const int* __restrict__ idx, int e_lo, int e_hi) {
    pdl_wait();
    pdl_trigger();
    const size_t t = blockIdx.x;
    if ((int)t < ex0 || (int)t >= ex1) extra = nullptr;  // extra rows exist only for tokens [ex0, ex1)
    // idx given: only the ranks whose expert lies in [e_lo, e_hi) were computed here (expert parallelism); skip the others
    unsigned have = 0xffffffffu;
    if (idx) {
        have = 0;
        for (int r = 0; r < K; r++) { const int e = idx[t * K + r]; if (e >= e_lo && e < e_hi) have |= 1u << r; }
    }
    float v[8];
    // both halves of the row in one round trip: the shared expert's row, the residual row and the first eight pair rows of
    // either half are requested before the first addition
    float4 ye[2], yx[2], y0[2][8];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int k0 = 1024 * h + 4 * threadIdx.x;
        ye[h] = yx[h] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (extra) ye[h] = *reinterpret_cast<const float4*>(extra + t * EH + k0);
        if (x) yx[h] = *reinterpret_cast<const float4*>(x + t * EH + k0);
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (u < K && (have >> u & 1)) y0[h][u] = *reinterpret_cast<const float4*>(ypair + (t * K + u) * EH + k0);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int k0 = 1024 * h + 4 * threadIdx.x;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (u < K && (have >> u & 1)) { acc.x += y0[h][u].x; acc.y += y0[h][u].y; acc.z += y0[h][u].z; acc.w += y0[h][u].w; }
        for (int rb = 8; rb < K; rb += 8) {  // more than eight ranks: eight rows in flight at a time, added in rank order
            float4 y[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (rb + u < K && (have >> (rb + u) & 1)) y[u] = *reinterpret_cast<const float4*>(ypair + (t * K + rb + u) * EH + k0);
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (rb + u < K && (have >> (rb + u) & 1)) { acc.x += y[u].x; acc.y += y[u].y; acc.z += y[u].z; acc.w += y[u].w; }
        }
        if (extra) { acc.x += ye[h].x; acc.y += ye[h].y; acc.z += ye[h].z; acc.w += ye[h].w; }
        if (x) { acc.x = yx[h].x + acc.x; acc.y = yx[h].y + acc.y; acc.z = yx[h].z + acc.z; acc.w = yx[h].w + acc.w; }
        *reinterpret_cast<float4*>(out + t * EH + k0) = acc;
        v[4 * h] = acc.x; v[4 * h + 1] = acc.y; v[4 * h + 2] = acc.z; v[4 * h + 3] = acc.w;
    }
    if (xn_next) norm_split_row<F16>(v, xn_next + t * EH, xs_next + t * 2 * EH, eps);
}

// Exclusive prefix sum over the 1024 threads of a block; every thread also gets the total.
__device__ __forceinline__ int block_scan_1024(int v, int& total) {
    __shared__ int wsum[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += u; }
    __syncthreads();  // wsum may still be read by a previous scan
    if (lane == 31) wsum[w] = inc;
    __syncthreads();
    int ws = wsum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, ws, o); if (lane >= o) ws += u; }
    total = __shfl_sync(0xffffffffu, ws, 31);
    const int before = __shfl_sync(0xffffffffu, ws, (w + 31) & 31);
    return inc - v + (w ? before : 0);
}

// Grouping and planning of a batch in one block of 1024 threads (one expert per thread; E <= 1024): the (token, rank) pairs
// bucketed by expert (the host loop of moex.cu:1466-1486), the sub-items of at most maxp pairs that the streaming kernels
// walk, and optionally a second sub-item list with another width (the tensor-core kernels take 128 / parts pairs per tile
// for gate/up and 64 for down). Histogram of the T*K pairs in shared memory, block scans, then
// every pair takes the next free place of its expert (an atomic cursor: the order of an expert's pairs is not the token
// order and may change from run to run - every pair's result is independent of its place). List 1 keeps sub-items of more
// than maxp / 2 pairs first (nsub[1] = their number); list 2 is in expert order. The shared expert (slot_table[E], when
// gate_logits is given) gets the tokens [sh0, sh1) with weight sigmoid(gate logit), as the last item.
// EP: the ids and weights of the tokens outside [sh0, sh1) were stored by other GPUs (ep.cuh): the block first waits (bounded)
// until every such token's dispatch flag ep_flags[t] has reached *ep_step * EP_PHASES + ep_phase, and the lists are then read
// past L1.
template <bool EP>
__global__ void __launch_bounds__(1024) group_plan1_k(const int* __restrict__ idx, const float* __restrict__ w, int T, int K, int E,
                                                      const uint8_t* const* __restrict__ slot_table, moexb_pair_item* __restrict__ items,
                                                      moexb_pair* __restrict__ pairs, int* __restrict__ nitems,
                                                      moexb_pair_item* __restrict__ subs, int* __restrict__ nsub, int maxp,
                                                      moexb_pair_item* __restrict__ subs2, int* __restrict__ nsub2, int maxp2,
                                                      const float* __restrict__ gate_logits, int gl_stride, int sh0, int sh1,
                                                      int stage_pairs, const unsigned* ep_flags = nullptr, const unsigned* ep_step = nullptr,
                                                      unsigned ep_phase = 0, int ep_world = 0, int ep_rank = 0, int* err = nullptr) {
    __shared__ int cnt[1024], cur[1024], start[1024];
    extern __shared__ int stage[];   // stage_pairs pairs of 3 words, when the launch gave the room
    const int n = T * K, e = threadIdx.x;
    cnt[e] = 0; cur[e] = 0;
    // what does not come from the kernel before: the blob pointers
    const uint8_t* slot = e < E ? slot_table[e] : nullptr;
    const uint8_t* sslot = slot_table[E];
    const bool with_shared = gate_logits && sslot && sh1 > sh0;
    const int Ts = with_shared ? sh1 - sh0 : 0;
    __syncthreads();
    pdl_wait();
    pdl_trigger();
    if constexpr (EP) {
        const unsigned target = *ep_step * EP_PHASES + ep_phase;
        for (int t = e; t < T; t += 1024)
            if (t < sh0 || t >= sh1) ep_wait_flag(ep_flags + t, target, err, EP_ERR_DISPATCH_WAIT);
        __syncthreads();   // the polling threads' acquire loads, then the barrier: the peers' lists are visible to the whole block
    }
    auto ld_idx = [&](int p) { return EP ? __ldcg(idx + p) : __ldg(idx + p); };
    auto ld_w = [&](int p) { return EP ? __ldcg(w + p) : __ldg(w + p); };
    // Every global load of the first 8192 pairs and of the first 1024 gate logits is issued here, in one round trip; the
    // values stay in registers for the histogram and for the scatter.
    constexpr int B = 8;   // pairs per thread in flight
    int ex0[B]; float wp0[B];
#pragma unroll
    for (int u = 0; u < B; u++) {
        const int p = e + 1024 * u;
        ex0[u] = p < n ? ld_idx(p) : -1; wp0[u] = p < n ? ld_w(p) : 0.f;
    }
    const float gl0 = e < Ts ? gate_logits[(size_t)(sh0 + e) * gl_stride] : 0.f;
#pragma unroll
    for (int u = 0; u < B; u++) if (ex0[u] >= 0) atomicAdd(&cnt[ex0[u]], 1);
    for (int p0 = e + 1024 * B; p0 < n; p0 += 1024 * B) {
        int ex[B];
#pragma unroll
        for (int u = 0; u < B; u++) ex[u] = p0 + 1024 * u < n ? ld_idx(p0 + 1024 * u) : -1;
#pragma unroll
        for (int u = 0; u < B; u++) if (ex[u] >= 0) atomicAdd(&cnt[ex[u]], 1);
    }
    __syncthreads();
    const int c = slot ? cnt[e] : 0;   // pairs of experts that are not held here are dropped
    auto wide = [](int c, int mp) { return c / mp + (c % mp > mp / 2); };
    auto narrow = [](int c, int mp) { return (int)(c % mp > 0 && c % mp <= mp / 2); };
    int np, ni, nw, nn, n2 = 0;
    const int at = block_scan_1024(c, np), item = block_scan_1024(c != 0, ni);
    const int wat = block_scan_1024(wide(c, maxp), nw), nat = block_scan_1024(narrow(c, maxp), nn);
    const int at2 = subs2 ? block_scan_1024((c + maxp2 - 1) / maxp2, n2) : 0;
    start[e] = slot ? at : -1;
    const bool staged = stage_pairs >= n;
    const int all_wide = nw + wide(Ts, maxp);   // the routed experts' wide sub-items, then the shared expert's
    if (c) {
        items[item] = {slot, at, c};
        const int cw = wide(c, maxp);
        for (int j = 0; j * maxp < c; j++) subs[j < cw ? wat + j : all_wide + nat] = {slot, at + j * maxp, min(maxp, c - j * maxp)};
        if (subs2) for (int j = 0; j * maxp2 < c; j++) subs2[at2 + j] = {slot, at + j * maxp2, min(maxp2, c - j * maxp2)};
    }
    __syncthreads();
    auto place = [&](int p, int ex, float wp) {
        const int s0 = ex >= 0 ? start[ex] : -1;
        if (s0 < 0) return;
        const int at_p = s0 + atomicAdd(&cur[ex], 1);
        if (staged) { stage[3 * at_p] = p / K; stage[3 * at_p + 1] = p; stage[3 * at_p + 2] = __float_as_int(wp); }
        else pairs[at_p] = {p / K, p, wp};
    };
#pragma unroll
    for (int u = 0; u < B; u++) place(e + 1024 * u, ex0[u], wp0[u]);
    for (int p0 = e + 1024 * B; p0 < n; p0 += 1024 * B) {
        int ex[B]; float wp[B];
#pragma unroll
        for (int u = 0; u < B; u++) { const int p = p0 + 1024 * u; ex[u] = p < n ? ld_idx(p) : -1; wp[u] = p < n ? ld_w(p) : 0.f; }
#pragma unroll
        for (int u = 0; u < B; u++) place(p0 + 1024 * u, ex[u], wp[u]);
    }
    if (staged) {
        // scattered 12-byte stores from one SM cost a sector each; from shared memory the list leaves as full lines
        __syncthreads();
        int* out = reinterpret_cast<int*>(pairs);
        for (int i = e; i < 3 * np; i += 1024) out[i] = stage[i];
    }
    if (with_shared) {
        const int cw = wide(Ts, maxp), ns = all_wide + nn;   // ns: where the shared expert's narrow sub-item goes
        for (int t = e; t < Ts; t += 1024) {
            const float gl = t == e ? gl0 : gate_logits[(size_t)(sh0 + t) * gl_stride];
            pairs[np + t] = {sh0 + t, n + sh0 + t, 1.f / (1.f + expf(-gl))};
        }
        for (int j = e; j * maxp < Ts; j += 1024) subs[j < cw ? nw + j : ns] = {sslot, np + j * maxp, min(maxp, Ts - j * maxp)};
        if (subs2) for (int j = e; j * maxp2 < Ts; j += 1024) subs2[n2 + j] = {sslot, np + j * maxp2, min(maxp2, Ts - j * maxp2)};
        if (e == 0) {
            items[ni] = {sslot, np, Ts}; *nitems = ni + 1;
            nsub[0] = ns + narrow(Ts, maxp); nsub[1] = all_wide;
            if (subs2) *nsub2 = n2 + (Ts + maxp2 - 1) / maxp2;
        }
    } else if (e == 0) {
        *nitems = ni; nsub[0] = all_wide + nn; nsub[1] = all_wide;
        if (subs2) *nsub2 = n2;
    }
}

// Sub-items of at most maxp pairs from the items of a work list. One block of 1024 threads, one item per thread
// and pass.
__global__ void __launch_bounds__(1024) plan_subitems_k(const moexb_pair_item* __restrict__ items, const int* __restrict__ nitems_dev, int nitems_host,
                                                        moexb_pair_item* __restrict__ subs, int* __restrict__ nsub, int maxp) {
    const int ni = nitems_dev ? *nitems_dev : nitems_host;
    int done = 0;
    for (int base = 0; base < ni; base += 1024) {
        const int i = base + threadIdx.x;
        moexb_pair_item it = {nullptr, 0, 0};
        if (i < ni) it = items[i];
        const int mine = (it.count + maxp - 1) / maxp;
        int total;
        const int at = done + block_scan_1024(mine, total);
        for (int j = 0; j < mine; j++) subs[at + j] = {it.slot, it.start + j * maxp, min(maxp, it.count - j * maxp)};
        done += total;
    }
    if (threadIdx.x == 0) *nsub = done;
}

// One token: the K (or *nh) decode experts as sub-items of one pair each, pair k = (token 0, row k, weight w[k]).
__global__ void plan_decode_k(const uint8_t* const* __restrict__ slots, const float* __restrict__ w, int K, const int* __restrict__ nh,
                              moexb_pair_item* __restrict__ subs, moexb_pair* __restrict__ pairs, int* __restrict__ nsub) {
    const int k = threadIdx.x, n = nh ? min(max(*nh, 0), K) : K;
    if (k < n) { subs[k] = {slots[k], k, 1}; pairs[k] = {0, k, w[k]}; }
    if (k == 0) *nsub = n;
}

// Self-test of the bounded waits (moexb_ctx_selftest_timeout): one warp waits on an mbarrier that expects 16 bytes which
// nobody ever sends. Nothing is in flight, nothing faults: the wait runs out of polls, records `code` and the kernel returns.
__global__ void selftest_mbar_timeout_k(int* err, int code, int limit, int* polls_done) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_arrive_expect_tx(smem_u32(&bar), 16);
    }
    __syncthreads();
    const bool ok = mbar_wait(smem_u32(&bar), 0, err, code, limit);
    if (threadIdx.x == 0) *polls_done = ok ? 0 : limit;
}

}  // namespace moexb
