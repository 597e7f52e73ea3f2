// Expert formats: full dequantisation (for the bit-exact weight check), GGUF Q4_K super-blocks (dequantise, and the
// bit-preserving conversion into the zero-point blob), and the seeded synthetic expert generator (host and device).
#pragma once
#include "common.cuh"
#include "synth.h"

namespace moexb {

// ---- GGUF Q4_K (144-byte super-block: f16 d, f16 dmin, 12 bytes of 6-bit scales/mins, 128 bytes of quants) ----------

// 6-bit scale and min of sub-block j (0..7) from the 12 packed bytes, as llama.cpp's get_scale_min_k4 (gguf.h:79-82).
__host__ __device__ inline void q4k_scale_min(int j, const uint8_t* sc, int& s, int& m) {
    if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
    else { s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}

// One super-block -> 128 nibble bytes in element order (element 2k low, 2k+1 high), [sc, mn] per 32 weights with
// mn = -min, and the untouched (d, dmin) halves: the same bits, re-ordered (gguf.h:261-270 and 330). Sub-block pair j
// keeps elements 64j..64j+31 in the low nibbles of quant bytes 32j..32j+31 and elements 64j+32..64j+63 in the high ones.
__host__ __device__ inline void q4k_block_to_zp(const uint8_t* blk, uint8_t* qb, uint8_t* cs, uint8_t* sup) {
    for (int i = 0; i < 4; i++) sup[i] = blk[i];
    const uint8_t *sc = blk + 4, *q = blk + 16;
    for (int j = 0; j < 8; j++) {
        int s, m;
        q4k_scale_min(j, sc, s, m);
        cs[2 * j] = (uint8_t)s; cs[2 * j + 1] = (uint8_t)(int8_t)-m;
    }
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 16; l++) {
            const uint8_t a = q[32 * j + 2 * l], b = q[32 * j + 2 * l + 1];
            qb[32 * j + l] = (uint8_t)((a & 0xF) | ((b & 0xF) << 4));       // elements 64j + 2l, 64j + 2l + 1
            qb[32 * j + 16 + l] = (uint8_t)((a >> 4) | ((b >> 4) << 4));    // elements 64j + 32 + 2l, + 1
        }
}

// Where super-block sb (0 .. 3*H*I/256-1, in blob order [gate | up | down]) lands inside a zero-point blob.
__host__ __device__ inline void zp_block_dst(uint8_t* blob, size_t sb, uint8_t*& qb, uint8_t*& cs, uint8_t*& sup) {
    qb = blob + sb * 128;
    cs = blob + Q_BYTES + sb * 16;
    sup = blob + Q_BYTES + CHUNKS * 2 + sb * 4;
}

// y = (d*s_j)*q - dmin*m_j for one thread per (super-block, sub-block pair) (gguf.h:98-110)
__global__ void q4k_dequant_k(const uint8_t* __restrict__ blocks, long long nblocks, float* __restrict__ y) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblocks * 4) return;
    const uint8_t* p = blocks + (i >> 2) * 144;
    const int j = (int)(i & 3);
    const float d = __half2float(*reinterpret_cast<const __half*>(p)), dmin = __half2float(*reinterpret_cast<const __half*>(p + 2));
    int s, m;
    q4k_scale_min(2 * j, p + 4, s, m); const float d1 = d * (float)s, m1 = dmin * (float)m;
    q4k_scale_min(2 * j + 1, p + 4, s, m); const float d2 = d * (float)s, m2 = dmin * (float)m;
    const uint8_t* q = p + 16 + 32 * j;
    float* o = y + (i >> 2) * 256 + 64 * j;
    for (int l = 0; l < 32; l++) { o[l] = d1 * (float)(q[l] & 0xF) - m1; o[32 + l] = d2 * (float)(q[l] >> 4) - m2; }
}

// Raw Q4_K tensors of one expert -> zero-point blob, one thread per super-block. gate/up rows hold 8 super-blocks,
// down rows 2; rows of the three tensors are consecutive in the blob, so super-block sb of the blob is block
// sb (gate), sb - 4096 (up), sb - 8192 (down) of its tensor (gguf.h:676-685).
__global__ void q4k_to_zp_k(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up, const uint8_t* __restrict__ down,
                            uint8_t* __restrict__ blob) {
    const size_t sb = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr size_t NB = (size_t)EH * EI / 256;
    if (sb >= 3 * NB) return;
    const uint8_t* src = sb < NB ? gate + sb * 144 : sb < 2 * NB ? up + (sb - NB) * 144 : down + (sb - 2 * NB) * 144;
    uint8_t blk[144], *qb, *cs, *sup;
    for (int i = 0; i < 144; i++) blk[i] = src[i];
    zp_block_dst(blob, sb, qb, cs, sup);
    q4k_block_to_zp(blk, qb, cs, sup);
}

// ---- full dequantisation of a blob ---------------------------------------------------------------------------------------

// out[i] for the 32 weights of chunk g32, one thread per chunk: q * scale, or (d*sc) * u + dm*mn.
template <int FMT>
__global__ void dequant_k(const uint8_t* __restrict__ blob, float* __restrict__ out) {
    const size_t g32 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g32 >= CHUNKS) return;
    const uint4 q = *reinterpret_cast<const uint4*>(blob + g32 * 16);
    const float2 sm = chunk_scale<FMT>(blob, g32);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    for (int j = 0; j < 4; j++)
        for (int n = 0; n < 8; n++) {
            const int v = (w[j] >> (4 * n)) & 0xF;
            out[g32 * 32 + 8 * j + n] = FMT == FMT_ZP ? fmaf(sm.x, (float)v, sm.y) : (float)(v >= 8 ? v - 16 : v) * sm.x;
        }
}

// ---- synthetic experts ----------------------------------------------------------------------------------------------------

// The 144 bytes of synthetic Q4_K super-block sb (blob order) of expert (layer, expert).
__host__ __device__ inline void synth_q4k_block(uint32_t seed, int layer, int expert, size_t sb, const uint16_t* table_d, uint8_t* blk) {
    for (uint32_t j = 0; j < 36; j++) {
        const uint32_t w = synth_q4k_word(seed, layer, expert, sb, j, table_d);
        blk[4 * j] = (uint8_t)w; blk[4 * j + 1] = (uint8_t)(w >> 8); blk[4 * j + 2] = (uint8_t)(w >> 16); blk[4 * j + 3] = (uint8_t)(w >> 24);
    }
}

// One 32-bit word (or one scale, or one super-block) of expert e0 + blockIdx.y per thread.
template <int FMT>
__global__ void synth_experts_k(uint32_t seed, int layer, int e0, uint8_t* __restrict__ dst, const uint16_t* __restrict__ table_s,
                                const uint16_t* __restrict__ table_d) {
    const int expert = e0 + blockIdx.y;
    uint8_t* blob = dst + (size_t)blockIdx.y * expert_bytes(FMT);
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if constexpr (FMT == FMT_ZP) {
        if (i >= CHUNKS / 8) return;
        uint8_t blk[144], *qb, *cs, *sup;
        synth_q4k_block(seed, layer, expert, i, table_d, blk);
        zp_block_dst(blob, i, qb, cs, sup);
        q4k_block_to_zp(blk, qb, cs, sup);
    } else {
        if (i < Q_BYTES / 4) reinterpret_cast<uint32_t*>(blob)[i] = synth_nibble_word(seed, layer, expert, i);
        if (i < CHUNKS / 2) {
            const uint16_t h = synth_scale_h(seed, layer, expert, i, table_s);
            if constexpr (FMT == FMT_SYM_F16) reinterpret_cast<uint16_t*>(blob + Q_BYTES)[i] = h;
            else reinterpret_cast<float*>(blob + Q_BYTES)[i] = __half2float(__ushort_as_half(h));
        }
    }
}

}  // namespace moexb
