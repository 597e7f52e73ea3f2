// Counter-based synthetic expert weights, identical bytes on host and device.
//
// Every 32-bit word of a synthetic tensor is a pure function of (seed, layer, expert, stream, word index), built from
// integer arithmetic only, so the CUDA fill kernel and the host fill routine produce the same bytes and a parity test can
// regenerate on the CPU exactly the experts it needs without downloading 17 GB from the GPU. Normally distributed
// quantities (the fp16 group scales |N(0, 0.02)| of the symmetric format, the fp16 d / dmin |N(0, 0.01)| of Q4_K
// super-blocks) come from a 4096-entry table of half-normal quantiles that the host computes once in double precision
// and uploads; the device only indexes it.
//
// Shapes follow the reference's expert blob (kernels.cuh:413-428): H = 2048, I = 512, group size 64.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SYNTH_HD __host__ __device__ __forceinline__
#else
#define SYNTH_HD static inline
#endif

#define SYNTH_TABLE_N 4096

enum {
    SYNTH_STREAM_NIBBLES = 0,  // packed int4 area of a symmetric blob
    SYNTH_STREAM_SCALES = 1,   // group scales of a symmetric blob
    SYNTH_STREAM_Q4K = 2,      // raw GGUF Q4_K super-blocks
    SYNTH_STREAM_Q4K_D = 3     // d / dmin of each super-block
};

SYNTH_HD uint64_t synth_key(uint32_t seed, uint32_t layer, uint32_t expert, uint32_t stream) {
    uint64_t k = ((uint64_t)seed << 32) ^ ((uint64_t)layer << 20) ^ ((uint64_t)expert << 4) ^ (uint64_t)stream;
    k = (k ^ (k >> 30)) * 0xBF58476D1CE4E5B9ull;
    k = (k ^ (k >> 27)) * 0x94D049BB133111EBull;
    return k ^ (k >> 31);
}

// splitmix64 finaliser over key + counter; the high half is returned
SYNTH_HD uint32_t synth_u32(uint64_t key, uint64_t word) {
    uint64_t z = key + (word + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (uint32_t)(z >> 32);
}

// Word w of the nibble area of expert (layer, expert): 8 int4 values uniform over [-8, 7], two per byte.
SYNTH_HD uint32_t synth_nibble_word(uint32_t seed, uint32_t layer, uint32_t expert, uint64_t w) {
    return synth_u32(synth_key(seed, layer, expert, SYNTH_STREAM_NIBBLES), w);
}

// Group scale g of expert (layer, expert) as fp16 bits; table = half-normal quantiles scaled by 0.02, as fp16 bits.
SYNTH_HD uint16_t synth_scale_h(uint32_t seed, uint32_t layer, uint32_t expert, uint64_t g, const uint16_t* table) {
    return table[synth_u32(synth_key(seed, layer, expert, SYNTH_STREAM_SCALES), g) & (SYNTH_TABLE_N - 1)];
}

// Word j (0..35) of Q4_K super-block b of expert (layer, expert). Word 0 holds d (low half) and dmin (high half), both
// from the 0.01-sigma table; words 1..3 the 12 packed 6-bit scale/min bytes; words 4..35 the 128 quant bytes.
SYNTH_HD uint32_t synth_q4k_word(uint32_t seed, uint32_t layer, uint32_t expert, uint64_t b, uint32_t j,
                                 const uint16_t* table_d) {
    if (j == 0) {
        const uint32_t h = synth_u32(synth_key(seed, layer, expert, SYNTH_STREAM_Q4K_D), b);
        return (uint32_t)table_d[h & (SYNTH_TABLE_N - 1)] | ((uint32_t)table_d[(h >> 12) & (SYNTH_TABLE_N - 1)] << 16);
    }
    return synth_u32(synth_key(seed, layer, expert, SYNTH_STREAM_Q4K), b * 36 + j);
}
