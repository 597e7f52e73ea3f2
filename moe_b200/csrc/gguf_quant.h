// GGUF expert tensors in other block formats than Q4_K, brought into the zero-point expert blob at load time (host code).
//
// Q4_K super-blocks map onto the zero-point blob bit for bit (formats.cuh). Every other ggml type has to be re-quantised to
// 4 bits: the reference's importer does it per 32 weights with a small least-squares fit (gguf.h:272-330, gg_zp_group and
// the non-Q4_K branch of gg_zp_row), and this file restates that procedure so that a GGUF whose expert tensors are Q5_K,
// Q6_K, Q8_0, IQ4_NL, IQ4_XS, Q4_0/1, Q5_0/1, F16, BF16 or F32 loads into a resident layer as the reference's own
// container would hold it:
//   1. the row is de-quantised to fp32 (gq_dequant: the published ggml block layouts, as gg_dequant gguf.h:85-255 reads them);
//   2. per 32 weights: u in [0, 15] and (s, m) with w ~ s * u + m - start on the min/max grid, then twice refit (s, m) by
//      least squares for the current rounding and round again, keeping the best;
//   3. per 256 weights: d = max s / 255 and dm = max |m| / 127 as fp16, sc = round(s / d) in [0, 255], mn = round(m / dm) in
//      [-127, 127], and the nibbles rounded once more on that final grid.
// Needs no GPU.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>
#include <algorithm>
#include <cmath>
#include <cstring>

namespace moexb {

enum : uint32_t { GQ_F32 = 0, GQ_F16 = 1, GQ_Q4_0 = 2, GQ_Q4_1 = 3, GQ_Q5_0 = 6, GQ_Q5_1 = 7, GQ_Q8_0 = 8, GQ_Q4_K = 12, GQ_Q5_K = 13,
                 GQ_Q6_K = 14, GQ_IQ4_NL = 20, GQ_IQ4_XS = 23, GQ_BF16 = 30 };

// Weights per block and bytes per block of a ggml type this file can read; false for the others.
inline bool gq_block(uint32_t type, int& n, int& bytes) {
    switch (type) {
        case GQ_F32: n = 1; bytes = 4; return true;
        case GQ_F16: case GQ_BF16: n = 1; bytes = 2; return true;
        case GQ_Q4_0: case GQ_IQ4_NL: n = 32; bytes = 18; return true;
        case GQ_Q4_1: n = 32; bytes = 20; return true;
        case GQ_Q5_0: n = 32; bytes = 22; return true;
        case GQ_Q5_1: n = 32; bytes = 24; return true;
        case GQ_Q8_0: n = 32; bytes = 34; return true;
        case GQ_Q4_K: n = 256; bytes = 144; return true;
        case GQ_Q5_K: n = 256; bytes = 176; return true;
        case GQ_Q6_K: n = 256; bytes = 210; return true;
        case GQ_IQ4_XS: n = 256; bytes = 136; return true;
    }
    return false;
}

inline float gq_h2f(const uint8_t* p) { __half h; memcpy(&h, p, 2); return __half2float(h); }
inline uint16_t gq_f2h(float f) { const __half h = __float2half_rn(f); uint16_t u; memcpy(&u, &h, 2); return u; }

// 6-bit (scale, min) number j of the 12 packed bytes of a K-quant super-block
inline void gq_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
    if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// the 16 levels of the non-linear 4-bit types (IQ4_NL, IQ4_XS)
static const int8_t GQ_IQ4_LEVELS[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// n values (a multiple of the block size) of `type` at p as fp32. False for a type gq_block does not know.
inline bool gq_dequant(uint32_t type, const uint8_t* p, int64_t n, float* y) {
    int bn, bb;
    if (!gq_block(type, bn, bb) || n % bn) return false;
    switch (type) {
        case GQ_F32: memcpy(y, p, (size_t)n * 4); return true;
        case GQ_F16: for (int64_t i = 0; i < n; i++) y[i] = gq_h2f(p + 2 * i); return true;
        case GQ_BF16:
            for (int64_t i = 0; i < n; i++) { uint16_t h; memcpy(&h, p + 2 * i, 2); const uint32_t u = (uint32_t)h << 16; memcpy(y + i, &u, 4); }
            return true;
        default: break;
    }
    for (int64_t b = 0; b < n / bn; b++, p += bb, y += bn) {
        switch (type) {
            case GQ_Q8_0: {
                const float d = gq_h2f(p);
                for (int i = 0; i < 32; i++) y[i] = d * (float)(int8_t)p[2 + i];
                break;
            }
            case GQ_Q4_0: case GQ_Q4_1: case GQ_Q5_0: case GQ_Q5_1: case GQ_IQ4_NL: {
                const float d = gq_h2f(p);
                const bool has_m = type == GQ_Q4_1 || type == GQ_Q5_1, five = type == GQ_Q5_0 || type == GQ_Q5_1;
                const float m = has_m ? gq_h2f(p + 2) : 0.f;
                const uint8_t* q = p + (has_m ? 4 : 2);
                uint32_t qh = 0;
                if (five) { memcpy(&qh, q, 4); q += 4; }
                for (int j = 0; j < 16; j++) {
                    int lo = q[j] & 0xF, hi = q[j] >> 4;
                    if (five) { lo |= ((qh >> j) << 4) & 0x10; hi |= (qh >> (j + 12)) & 0x10; }
                    if (type == GQ_IQ4_NL) { y[j] = d * (float)GQ_IQ4_LEVELS[lo]; y[j + 16] = d * (float)GQ_IQ4_LEVELS[hi]; }
                    else if (has_m) { y[j] = (float)lo * d + m; y[j + 16] = (float)hi * d + m; }
                    else { const int off = five ? 16 : 8; y[j] = (float)(lo - off) * d; y[j + 16] = (float)(hi - off) * d; }
                }
                break;
            }
            case GQ_Q4_K: case GQ_Q5_K: {
                const float d = gq_h2f(p), dmin = gq_h2f(p + 2);
                const uint8_t* sc = p + 4;
                const uint8_t* qh = p + 16;                       // Q5_K only: the fifth bits, 32 bytes
                const uint8_t* ql = p + (type == GQ_Q5_K ? 48 : 16);
                for (int j = 0; j < 4; j++, ql += 32) {           // 64 values: low nibbles, then high nibbles of 32 bytes
                    int s1, m1, s2, m2;
                    gq_scale_min(2 * j, sc, s1, m1); gq_scale_min(2 * j + 1, sc, s2, m2);
                    const float d1 = d * (float)s1, n1 = dmin * (float)m1, d2 = d * (float)s2, n2 = dmin * (float)m2;
                    for (int l = 0; l < 32; l++) {
                        int a = ql[l] & 0xF, b2 = ql[l] >> 4;
                        if (type == GQ_Q5_K) { a += (qh[l] >> (2 * j) & 1) << 4; b2 += (qh[l] >> (2 * j + 1) & 1) << 4; }
                        y[64 * j + l] = d1 * (float)a - n1;
                        y[64 * j + 32 + l] = d2 * (float)b2 - n2;
                    }
                }
                break;
            }
            case GQ_Q6_K: {
                const uint8_t *ql = p, *qh = p + 128;
                const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192);
                const float d = gq_h2f(p + 208);
                for (int half = 0; half < 2; half++, ql += 64, qh += 32, sc += 8)
                    for (int l = 0; l < 32; l++) {
                        const int is = l / 16;
                        const int q1 = (int)((ql[l] & 0xF) | ((qh[l] >> 0 & 3) << 4)) - 32, q2 = (int)((ql[l + 32] & 0xF) | ((qh[l] >> 2 & 3) << 4)) - 32;
                        const int q3 = (int)((ql[l] >> 4) | ((qh[l] >> 4 & 3) << 4)) - 32, q4 = (int)((ql[l + 32] >> 4) | ((qh[l] >> 6 & 3) << 4)) - 32;
                        float* o = y + 128 * half + l;
                        o[0] = d * (float)sc[is] * (float)q1; o[32] = d * (float)sc[is + 2] * (float)q2;
                        o[64] = d * (float)sc[is + 4] * (float)q3; o[96] = d * (float)sc[is + 6] * (float)q4;
                    }
                break;
            }
            case GQ_IQ4_XS: {
                const float d = gq_h2f(p);
                uint16_t sh; memcpy(&sh, p + 2, 2);
                const uint8_t *sl = p + 4, *q = p + 8;
                for (int ib = 0; ib < 8; ib++, q += 16) {
                    const int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
                    const float dl = d * (float)(ls - 32);
                    for (int j = 0; j < 16; j++) { y[32 * ib + j] = dl * (float)GQ_IQ4_LEVELS[q[j] & 0xF]; y[32 * ib + 16 + j] = dl * (float)GQ_IQ4_LEVELS[q[j] >> 4]; }
                }
                break;
            }
            default: return false;
        }
    }
    return true;
}

// 32 weights -> u in [0, 15] and (s, m) with x ~ s * u + m (gguf.h:272-300)
inline void zp_fit_group(const float* x, uint8_t* u, float& s, float& m) {
    float lo = x[0], hi = x[0];
    for (int i = 1; i < 32; i++) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
    s = (hi - lo) / 15; m = lo;
    if (s == 0) { memset(u, 0, 32); return; }
    auto sq_err = [&](float sc, float mn, const uint8_t* v) {
        float e = 0;
        for (int i = 0; i < 32; i++) { const float r = x[i] - sc * v[i] - mn; e += r * r; }
        return e;
    };
    auto round_on = [&](float sc, float mn, uint8_t* v) {
        for (int i = 0; i < 32; i++) v[i] = (uint8_t)std::clamp((int)std::nearbyint((x[i] - mn) / sc), 0, 15);
    };
    round_on(s, m, u);
    float best = sq_err(s, m, u);
    uint8_t v[32];
    for (int it = 0; it < 2; it++) {
        const uint8_t* cur = it ? v : u;
        double su = 0, suu = 0, sx = 0, sxu = 0;
        for (int i = 0; i < 32; i++) { su += cur[i]; suu += cur[i] * cur[i]; sx += x[i]; sxu += (double)x[i] * cur[i]; }
        const double det = 32 * suu - su * su;
        if (det <= 0) break;
        const float s1 = (float)((32 * sxu - su * sx) / det), m1 = (float)((sx - s1 * su) / 32);
        if (s1 <= 0) break;
        round_on(s1, m1, v);
        const float e = sq_err(s1, m1, v);
        if (e < best) { best = e; s = s1; m = m1; memcpy(u, v, 32); }
    }
}

// One row of `cols` fp32 weights (a multiple of 256) -> the zero-point form of a blob row: nibble bytes (element 2k in the low
// nibble), [sc, mn] per 32 weights, (d, dm) as fp16 bits per 256 weights (the non-Q4_K branch of gg_zp_row, gguf.h:310-327).
inline void zp_row_from_values(const float* w, int cols, uint8_t* qb, uint8_t* cs, uint16_t* sup) {
    uint8_t u[256];
    for (int b = 0; b < cols / 256; b++) {
        const float* x = w + 256 * b;
        uint8_t* c = cs + 16 * b;
        float s[8], m[8], smax = 0, mmax = 0;
        for (int g = 0; g < 8; g++) {
            zp_fit_group(x + 32 * g, u + 32 * g, s[g], m[g]);
            smax = std::max(smax, s[g]); mmax = std::max(mmax, std::fabs(m[g]));
        }
        sup[2 * b] = gq_f2h(smax / 255); sup[2 * b + 1] = gq_f2h(mmax / 127);
        const float d = gq_h2f(reinterpret_cast<const uint8_t*>(sup + 2 * b)), dm = gq_h2f(reinterpret_cast<const uint8_t*>(sup + 2 * b + 1));
        for (int g = 0; g < 8; g++) {
            const int sc = d > 0 ? std::clamp((int)std::nearbyint(s[g] / d), 0, 255) : 0;
            const int mn = dm > 0 ? std::clamp((int)std::nearbyint(m[g] / dm), -127, 127) : 0;
            c[2 * g] = (uint8_t)sc; c[2 * g + 1] = (uint8_t)(int8_t)mn;
            const float s1 = d * sc, m1 = dm * mn;
            for (int i = 0; i < 32; i++)
                u[32 * g + i] = s1 > 0 ? (uint8_t)std::clamp((int)std::nearbyint((x[32 * g + i] - m1) / s1), 0, 15) : 0;
        }
        for (int i = 0; i < 128; i++) qb[b * 128 + i] = (uint8_t)(u[2 * i] | u[2 * i + 1] << 4);
    }
}

}  // namespace moexb
