/* CPU oracle for the MoE expert-FFN path - TEST INFRASTRUCTURE, not part of the product.
 *
 * A plain-C restatement of the reference's algorithm for this path, used only as the checker by tests/, by
 * __graft_entry__.smoke() and by bench.py's CPU-baseline legs. Nothing in the moe_b200 package links or calls it.
 * Every function cites the reference file:line (paths inside the reference tree) whose arithmetic it follows.
 *
 * Parity pins (tests/test_oracle_pins.py):
 *   - orc_q4k_dequant against the reference's own fixture tests/gguf_blocks.bin (Q4_K record: 16 real super-blocks and
 *     the 4096 values gguf-py gives for them), committed as tests/golden/q4k_fixture.bin;
 *   - orc_q4k_to_zp_row / orc_zp_at against gg_zp_row / gg_zp_at of the compiled reference, bytes identical;
 *   - orc_run_pairs (symmetric) against CpuExperts::run_pairs of the compiled reference, bit for bit: the 8-lane
 *     accumulation order of the AVX code is reproduced with scalar fmaf; the zero-point variant to 1e-6 of the
 *     largest value (its final 4-term sum is left to the compiler's contraction in the reference);
 *   - golden outputs of the compiled reference for small seeded cases are committed under tests/golden/.
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off -mfma -fopenmp -shared)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <immintrin.h>
#include <omp.h>
#include "../moe_b200/csrc/synth.h"   /* the counter-based generator itself: integer arithmetic, no CUDA types */

#define EH 2048 /* kernels.cuh:422 */
#define EI 512
#define EGS 64
#define Q_BYTES ((size_t)3 * EH * EI / 2)      /* kernels.cuh:423 */
#define CHUNKS ((size_t)3 * EH * EI / 32)       /* kernels.cuh:425 */

enum { FMT_SYM_F32 = 0, FMT_SYM_F16 = 1, FMT_ZP = 2 };

size_t orc_expert_bytes(int fmt) {
    if (fmt == FMT_SYM_F32) return Q_BYTES + (size_t)3 * EI * (EH / EGS) * 4; /* kernels.cuh:424 */
    if (fmt == FMT_SYM_F16) return Q_BYTES + (size_t)3 * EI * (EH / EGS) * 2;
    if (fmt == FMT_ZP) return Q_BYTES + CHUNKS * 2 + CHUNKS / 8 * 4;          /* kernels.cuh:426 */
    return 0;
}

/* IEEE half -> float, all cases (gguf.h:64-70) */
float orc_half(uint16_t h) {
    const uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF;
    uint32_t u;
    float f;
    if (e == 0) { f = (float)m * (1.0f / 16777216.0f); memcpy(&u, &f, 4); u |= s; }
    else u = s | (e == 31 ? (0x7F800000u | (m << 13)) : (((e + 112) << 23) | (m << 13)));
    memcpy(&f, &u, 4);
    return f;
}

static inline float sym_scale(int fmt, const uint8_t* blob, size_t g) {
    if (fmt == FMT_SYM_F32) { float s; memcpy(&s, blob + Q_BYTES + 4 * g, 4); return s; }
    uint16_t h; memcpy(&h, blob + Q_BYTES + 2 * g, 2); return orc_half(h);
}

/* (s, m) of 32-weight chunk c of a zero-point blob: s = d*sc, m = dm*mn (kernels.cuh:468-474, cpu_expert.h:112-118) */
static inline void zp_chunk(const uint8_t* blob, size_t c, float* s, float* m) {
    const uint8_t* b = blob + Q_BYTES;
    uint16_t d, dm;
    memcpy(&d, b + CHUNKS * 2 + 4 * (c >> 3), 2);
    memcpy(&dm, b + CHUNKS * 2 + 4 * (c >> 3) + 2, 2);
    *s = orc_half(d) * (float)b[2 * c];
    *m = orc_half(dm) * (float)(int8_t)b[2 * c + 1];
}

/* Weight i of the blob (blob order [gate | up | down]) as fp32: q*scale (qwen36_ref.py:39-59) or
 * d*sc*u + dm*mn (gguf.h:332-335). */
void orc_dequant(int fmt, const uint8_t* blob, float* out) {
    const size_t n = (size_t)3 * EH * EI;
    for (size_t i = 0; i < n; i++) {
        const int v = (blob[i / 2] >> ((i & 1) * 4)) & 0xF;
        if (fmt == FMT_ZP) {
            float s, m;
            zp_chunk(blob, i / 32, &s, &m);
            out[i] = s * (float)v + m;
        } else {
            out[i] = (float)(v >= 8 ? v - 16 : v) * sym_scale(fmt, blob, i / 64);
        }
    }
}

/* ---- GGUF Q4_K ----------------------------------------------------------------------------------------------------- */

/* 6-bit scale and min of sub-block j from the 12 packed bytes (gguf.h:79-82) */
static inline void scale_min_k4(int j, const uint8_t* q, int* d, int* m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

/* n values of 144-byte super-blocks: y = (d*s)*q - dmin*m (gguf.h:98-110) */
void orc_q4k_dequant(const uint8_t* p, long long n, float* y) {
    for (long long b = 0; b < n / 256; b++, p += 144) {
        uint16_t hd, hm;
        memcpy(&hd, p, 2); memcpy(&hm, p + 2, 2);
        const float d = orc_half(hd), dmin = orc_half(hm);
        const uint8_t *sc = p + 4, *q = p + 16;
        for (int j = 0, is = 0; j < 256; j += 64, q += 32, is += 2) {
            int s, m;
            scale_min_k4(is, sc, &s, &m);
            const float d1 = d * (float)s, m1 = dmin * (float)m;
            scale_min_k4(is + 1, sc, &s, &m);
            const float d2 = d * (float)s, m2 = dmin * (float)m;
            for (int l = 0; l < 32; l++) *y++ = d1 * (float)(q[l] & 0xF) - m1;
            for (int l = 0; l < 32; l++) *y++ = d2 * (float)(q[l] >> 4) - m2;
        }
    }
}

/* One row of Q4_K super-blocks -> nibble bytes in element order, [sc, mn] per 32, (d, dmin) per 256
 * (gguf.h:261-270 for the block, gguf.h:302-330 for the row; Q4_K branch only) */
void orc_q4k_to_zp_row(const uint8_t* src, int cols, uint8_t* qb, uint8_t* cs, uint16_t* sup) {
    uint8_t u[256];
    for (int b = 0; b < cols / 256; b++) {
        const uint8_t* p = src + (size_t)b * 144;
        uint8_t* c = cs + 16 * b;
        memcpy(sup + 2 * b, p, 4);
        const uint8_t *sc = p + 4, *q = p + 16;
        for (int j = 0; j < 4; j++, q += 32) {
            int a, m;
            scale_min_k4(2 * j, sc, &a, &m); c[4 * j] = (uint8_t)a; c[4 * j + 1] = (uint8_t)(int8_t)-m;
            scale_min_k4(2 * j + 1, sc, &a, &m); c[4 * j + 2] = (uint8_t)a; c[4 * j + 3] = (uint8_t)(int8_t)-m;
            for (int l = 0; l < 32; l++) { u[64 * j + l] = q[l] & 0xF; u[64 * j + 32 + l] = q[l] >> 4; }
        }
        for (int i = 0; i < 128; i++) qb[b * 128 + i] = (uint8_t)(u[2 * i] | (u[2 * i + 1] << 4));
    }
}

/* Weight i of a converted row decoded back (gguf.h:332-335) */
float orc_zp_at(const uint8_t* qb, const uint8_t* cs, const uint16_t* sup, int i) {
    const int g = i / 32, b = i / 256;
    return orc_half(sup[2 * b]) * (float)cs[2 * g] * (float)((qb[i / 2] >> (i % 2 * 4)) & 0xF) +
           orc_half(sup[2 * b + 1]) * (float)(int8_t)cs[2 * g + 1];
}

/* One expert: raw Q4_K gate [I][H], up [I][H], down [H][I] -> zero-point blob (per-expert body of gg_experts,
 * gguf.h:676-685: merged row index, chunk offset c0, scale-part addresses) */
void orc_q4k_to_zp(const uint8_t* gate, const uint8_t* up, const uint8_t* down, uint8_t* blob) {
    uint8_t* se = blob + Q_BYTES;
    for (int part = 0; part < 3; part++) {
        const int rows = part < 2 ? EI : EH, cols = part < 2 ? EH : EI;
        const uint8_t* src = part == 0 ? gate : part == 1 ? up : down;
        const size_t row_bytes = (size_t)cols / 256 * 144;
        for (int r = 0; r < rows; r++) {
            const size_t row = (size_t)part * EI + r;
            uint8_t* qr = part < 2 ? blob + row * (EH / 2) : blob + (size_t)EI * EH + (size_t)r * (EI / 2);
            const size_t c0 = part < 2 ? row * (EH / 32) : (size_t)2 * EI * (EH / 32) + (size_t)r * (EI / 32);
            orc_q4k_to_zp_row(src + r * row_bytes, cols, qr, se + 2 * c0, (uint16_t*)(se + CHUNKS * 2) + 2 * (c0 / 8));
        }
    }
}

/* ---- router -------------------------------------------------------------------------------------------------------- */

/* y[r][o] = W[o] . x[r], fp32 (kernels.cuh:73-91 accumulates in fp32 with one warp per row; the order is pinned here:
 * partial j of 32 takes elements 128c+4j..4j+3 in ascending order with fused multiply-adds, then a xor-butterfly
 * 16,8,4,2,1 combines the partials). w16 != 0: W holds IEEE halves, as the reference uploads the router. */
void orc_router_logits(const void* W, int w16, const float* x, float* y, int In, int O, int rows) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int r = 0; r < rows; r++)
        for (int o = 0; o < O; o++) {
            float p[32];
            const float* xr = x + (size_t)r * In;
            for (int j = 0; j < 32; j++) {
                float acc = 0.f;
                for (int c = 0; c < In / 128; c++)
                    for (int i = 0; i < 4; i++) {
                        const size_t k = (size_t)128 * c + 4 * j + i;
                        const float wv = w16 ? orc_half(((const uint16_t*)W)[(size_t)o * In + k]) : ((const float*)W)[(size_t)o * In + k];
                        acc = fmaf(wv, xr[k], acc);
                    }
                p[j] = acc;
            }
            for (int s = 16; s; s >>= 1) {
                float n[32];
                for (int j = 0; j < 32; j++) n[j] = p[j] + p[j ^ s];
                memcpy(p, n, sizeof p);
            }
            y[(size_t)r * O + o] = p[0];
        }
}

/* Softmax over E, the K largest with ties to the lower index, weights renormalised over the selected K when norm
 * (kernels.cuh:373-406; qwen36_ref.py:203-209). Selection compares logits: softmax is monotone, and the rounded
 * probabilities the reference's GPU kernel compares cannot be reproduced on a CPU. */
void orc_router_topk(const float* logits, int E, int K, int norm, int* idx, float* w, int T, int ld) {
    for (int t = 0; t < T; t++) {
        const float* l = logits + (size_t)t * ld;
        float m = l[0];
        for (int e = 1; e < E; e++) m = fmaxf(m, l[e]);
        double sum = 0;
        for (int e = 0; e < E; e++) sum += (double)expf(l[e] - m);
        char* used = (char*)calloc(E, 1);
        double total = 0;
        for (int k = 0; k < K; k++) {
            int bi = -1;
            for (int e = 0; e < E; e++)
                if (!used[e] && (bi < 0 || l[e] > l[bi])) bi = e;
            used[bi] = 1;
            idx[t * K + k] = bi;
            const float p = (float)((double)expf(l[bi] - m) / sum);
            w[t * K + k] = p;
            total += p;
        }
        if (norm) for (int k = 0; k < K; k++) w[t * K + k] = (float)((double)w[t * K + k] / total);
        free(used);
    }
}

/* ---- routed experts, fp32 (the parity oracle: CpuExperts::run_pairs_f, cpu_expert.h:360-396) ----------------------- */

/* 8-lane horizontal sum in the order of hsum (cpu_expert.h:103-107) */
static inline float hsum8(const float* v) {
    const float s0 = v[0] + v[4], s1 = v[1] + v[5], s2 = v[2] + v[6], s3 = v[3] + v[7];
    return (s0 + s1) + (s2 + s3);
}

/* Row dot over n inputs in the accumulation order of row_dot / dot_group / dot_group_zp (cpu_expert.h:86-148):
 * q = the row's nibble bytes, c0 = the row's first 32-chunk, xe / xo = even / odd inputs. */
static float row_dot(int fmt, const uint8_t* blob, const uint8_t* q, size_t c0, const float* xe, const float* xo, int n) {
    if (fmt == FMT_ZP) {
        float acc = 0.f;
        for (int g = 0; g < n / 64; g++) {
            float v[4];
            zp_chunk(blob, c0 + 2 * g, &v[0], &v[1]);
            zp_chunk(blob, c0 + 2 * g + 1, &v[2], &v[3]);
            float gg[2][8] = {{0}}, sx[2][8] = {{0}};
            const uint8_t* b = q + 32 * g;
            const float *e = xe + 32 * g, *o = xo + 32 * g;
            for (int c = 0; c < 4; c++)
                for (int l = 0; l < 8; l++) {
                    gg[c / 2][l] = fmaf((float)(b[8 * c + l] & 0xF), e[8 * c + l], gg[c / 2][l]);
                    gg[c / 2][l] = fmaf((float)(b[8 * c + l] >> 4), o[8 * c + l], gg[c / 2][l]);
                    sx[c / 2][l] = sx[c / 2][l] + (e[8 * c + l] + o[8 * c + l]);
                }
            acc += v[0] * hsum8(gg[0]) + v[1] * hsum8(sx[0]) + v[2] * hsum8(gg[1]) + v[3] * hsum8(sx[1]);
        }
        return acc;
    }
    float acc[8] = {0};
    for (int g = 0; g < n / 64; g++) {
        float g8[8] = {0};
        const uint8_t* b = q + 32 * g;
        const float *e = xe + 32 * g, *o = xo + 32 * g;
        for (int c = 0; c < 4; c++)
            for (int l = 0; l < 8; l++) {
                const int lo = b[8 * c + l] & 0xF, hi = b[8 * c + l] >> 4;
                g8[l] = fmaf((float)(lo >= 8 ? lo - 16 : lo), e[8 * c + l], g8[l]);
                g8[l] = fmaf((float)(hi >= 8 ? hi - 16 : hi), o[8 * c + l], g8[l]);
            }
        const float s = sym_scale(fmt, blob, c0 / 2 + g);
        for (int l = 0; l < 8; l++) acc[l] = fmaf(g8[l], s, acc[l]);
    }
    return hsum8(acc);
}

static void deinterleave(const float* x, float* xe, float* xo, int n) { /* cpu_expert.h:150-152 */
    for (int i = 0; i < n / 2; i++) { xe[i] = x[2 * i]; xo[i] = x[2 * i + 1]; }
}

/* Jobs (one per expert) in flat form: job j uses blobs[j] and pairs job_start[j] .. job_start[j+1]-1 of
 * (toks, pids, ws). act[pid][I] = silu(g)*u with expf; ypair[pid][H] = w * (down . act) (cpu_expert.h:368-394).
 * act_out (optional) receives the activations. */
void orc_run_pairs(int fmt, int njobs, const uint8_t* const* blobs, const int* job_start, const int* toks,
                   const int* pids, const float* ws, const float* X, int T, int npairs, float* ypair, float* act_out) {
    float* xe = (float*)malloc((size_t)T * EH / 2 * 4);
    float* xo = (float*)malloc((size_t)T * EH / 2 * 4);
    float* act = (float*)malloc((size_t)npairs * EI * 4);
    float* ae = (float*)malloc((size_t)npairs * EI / 2 * 4);
    float* ao = (float*)malloc((size_t)npairs * EI / 2 * 4);
    for (int t = 0; t < T; t++) deinterleave(X + (size_t)t * EH, xe + (size_t)t * EH / 2, xo + (size_t)t * EH / 2, EH);
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
    for (int j = 0; j < njobs; j++)
        for (int r = 0; r < EI; r++) {
            const uint8_t* blob = blobs[j];
            for (int k = job_start[j]; k < job_start[j + 1]; k++) {
                const float *pe = xe + (size_t)toks[k] * EH / 2, *po = xo + (size_t)toks[k] * EH / 2;
                const float g = row_dot(fmt, blob, blob + (size_t)r * (EH / 2), (size_t)r * (EH / 32), pe, po, EH);
                const float u = row_dot(fmt, blob, blob + (size_t)(EI + r) * (EH / 2), (size_t)(EI + r) * (EH / 32), pe, po, EH);
                act[(size_t)pids[k] * EI + r] = g / (1.f + expf(-g)) * u;
            }
        }
    for (int j = 0; j < njobs; j++)
        for (int k = job_start[j]; k < job_start[j + 1]; k++) {
            const int p = pids[k];
            deinterleave(act + (size_t)p * EI, ae + (size_t)p * EI / 2, ao + (size_t)p * EI / 2, EI);
        }
#pragma omp parallel for collapse(2) schedule(dynamic, 32)
    for (int j = 0; j < njobs; j++)
        for (int d = 0; d < EH; d++) {
            const uint8_t* blob = blobs[j];
            for (int k = job_start[j]; k < job_start[j + 1]; k++) {
                const int p = pids[k];
                ypair[(size_t)p * EH + d] =
                    ws[k] * row_dot(fmt, blob, blob + (size_t)2 * EI * (EH / 2) + (size_t)d * (EI / 2),
                                    (size_t)2 * EI * (EH / 32) + (size_t)d * (EI / 32), ae + (size_t)p * EI / 2,
                                    ao + (size_t)p * EI / 2, EI);
            }
        }
    if (act_out) memcpy(act_out, act, (size_t)npairs * EI * 4);
    free(xe); free(xo); free(act); free(ae); free(ao);
}

/* moe[t][d] = sum over ranks of ypair[t*K+r][d], in rank order (kernels.cuh:744-753; moex.cu:1594-1599) */
void orc_pairs_reduce(const float* ypair, float* moe, int K, int D, int T) {
    for (int t = 0; t < T; t++)
        for (int d = 0; d < D; d++) {
            float acc = 0.f;
            for (int r = 0; r < K; r++) acc += ypair[((size_t)t * K + r) * D + d];
            moe[(size_t)t * D + d] = acc;
        }
}

/* Bucket the T*K (token, rank) pairs by expert: experts ascending, pairs in token order inside an expert, p = t*K+rank
 * (moex.cu:1466-1486; route_export_k, kernels.cuh:1030-1045). held (optional, E chars): experts with held[e] == 0 are
 * dropped. item_e / item_start / item_count: up to E entries. Returns the number of items. */
int orc_group_pairs(const int* idx, const float* w, int T, int K, int E, const char* held, int* item_e, int* item_start,
                    int* item_count, int* pair_t, int* pair_p, float* pair_w) {
    int* cnt = (int*)calloc(E, sizeof(int));
    for (int p = 0; p < T * K; p++) cnt[idx[p]]++;
    int ni = 0, np = 0;
    int* at = (int*)malloc(E * sizeof(int));
    for (int e = 0; e < E; e++) {
        at[e] = -1;
        if (!cnt[e] || (held && !held[e])) continue;
        item_e[ni] = e; item_start[ni] = np; item_count[ni] = cnt[e];
        at[e] = np; np += cnt[e]; ni++;
    }
    for (int p = 0; p < T * K; p++) {
        const int e = idx[p];
        if (at[e] < 0) continue;
        pair_t[at[e]] = p / K; pair_p[at[e]] = p; pair_w[at[e]] = w[p];
        at[e]++;
    }
    free(cnt); free(at);
    return ni;
}

/* y = x / sqrt(mean(x^2) + eps) with unit weight (kernels.cuh:48-64 with w = 0). The sum of squares follows a pinned
 * order so that a GPU kernel can reproduce it bit for bit: 256 partials, partial i takes elements 4i..4i+3, 1024+4i..
 * with fused multiply-adds; each group of 32 partials is combined by a xor-butterfly; the 8 group sums are added in
 * order. */
void orc_rmsnorm(const float* x, float* y, int D, int rows, float eps) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * D;
        float p[256];
        for (int i = 0; i < 256; i++) {
            float ss = 0.f;
            for (int b = 4 * i; b < D; b += 1024)
                for (int k = 0; k < 4; k++) ss = fmaf(xr[b + k], xr[b + k], ss);
            p[i] = ss;
        }
        float tot = 0.f;
        for (int wv = 0; wv < 8; wv++) {
            float* q = p + 32 * wv;
            for (int s = 16; s; s >>= 1) {
                float n[32];
                for (int j = 0; j < 32; j++) n[j] = q[j] + q[j ^ s];
                memcpy(q, n, sizeof n);
            }
            tot += q[0];
        }
        const float sc = 1.f / sqrtf(tot / (float)D + eps);
        for (int i = 0; i < D; i++) y[(size_t)r * D + i] = xr[i] * sc;
    }
}

/* One MoE layer for T tokens (qwen36_ref.py:201-220; moex.cu:1093-1107 and 1414-1617): router logits (row E of W =
 * the shared expert's gate vector) -> top-K, renormalised -> fp32 expert pairs -> rank-order sum -> + shared expert
 * scaled by sigmoid(gate logit), applied as sh / (1 + exp(-gl)) (kernels.cuh:973-977).
 * blobs: E+1 pointers (blob E = shared expert; null routed entries are skipped: expert-parallel partial result).
 * flags bit 0: no shared expert. */
void orc_layer_forward(int fmt, const uint8_t* const* blobs, const void* W, int w16, const float* X, int T, int E, int K,
                       float* out, int* idx, float* w, float* logits_out, int flags) {
    const int ld = E + 1;
    float* logits = (float*)malloc((size_t)T * ld * 4);
    orc_router_logits(W, w16, X, logits, EH, ld, T);
    orc_router_topk(logits, E, K, 1, idx, w, T, ld);
    int *ie = (int*)malloc(E * 4), *is = (int*)malloc((E + 1) * 4), *ic = (int*)malloc(E * 4);
    int *pt = (int*)malloc((size_t)T * K * 4), *pp = (int*)malloc((size_t)T * K * 4);
    float* pw = (float*)malloc((size_t)T * K * 4);
    char* held = (char*)malloc(E);
    for (int e = 0; e < E; e++) held[e] = blobs[e] != NULL;
    const int ni = orc_group_pairs(idx, w, T, K, E, held, ie, is, ic, pt, pp, pw);
    const uint8_t** jb = (const uint8_t**)malloc((ni + 1) * sizeof(void*));
    for (int i = 0; i < ni; i++) jb[i] = blobs[ie[i]];
    is[ni] = ni ? is[ni - 1] + ic[ni - 1] : 0;
    float* ypair = (float*)calloc((size_t)T * K * EH, 4);
    if (ni) orc_run_pairs(fmt, ni, jb, is, pt, pp, pw, X, T, T * K, ypair, NULL);
    orc_pairs_reduce(ypair, out, K, EH, T);
    if (!(flags & 1) && blobs[E]) {
        int* st = (int*)malloc(T * 4);
        float* one = (float*)malloc(T * 4);
        float* sh = (float*)malloc((size_t)T * EH * 4);
        for (int t = 0; t < T; t++) { st[t] = t; one[t] = 1.f; }
        const int js[2] = {0, T};
        const uint8_t* sb = blobs[E];
        orc_run_pairs(fmt, 1, &sb, js, st, st, one, X, T, T, sh, NULL);
        for (int t = 0; t < T; t++) {
            const float gl = logits[(size_t)t * ld + E];
            for (int d = 0; d < EH; d++) out[(size_t)t * EH + d] += sh[(size_t)t * EH + d] / (1.f + expf(-gl));
        }
        free(st); free(one); free(sh);
    }
    if (logits_out) memcpy(logits_out, logits, (size_t)T * ld * 4);
    free(logits); free(ie); free(is); free(ic); free(pt); free(pp); free(pw); free(held); free(jb); free(ypair);
}

/* ---- seeded synthetic experts on the host --------------------------------------------------------------------------------
 * The benchmark's CPU arm needs the same expert bytes as the GPU without loading the product library. The word generator is
 * shared source (synth.h, plain C); the half-normal quantile tables and the blob assembly are restated here and pinned
 * bit for bit against the product's host generator in tests/test_oracle_pins.py. */

void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

static uint16_t g_table_s[SYNTH_TABLE_N], g_table_d[SYNTH_TABLE_N];
static int g_tables_ready = 0;

/* table[i] = fp16 bits of sigma * q_i, q_i the (i + 0.5) / N quantile of |N(0, 1)| by bisection on erf */
static void synth_table(double sigma, uint16_t* table) {
    for (int i = 0; i < SYNTH_TABLE_N; i++) {
        const double p = (i + 0.5) / SYNTH_TABLE_N;
        double lo = 0, hi = 10;
        for (int it = 0; it < 80; it++) {
            const double mid = 0.5 * (lo + hi);
            if (erf(mid / sqrt(2.0)) < p) lo = mid; else hi = mid;
        }
        table[i] = _cvtss_sh((float)(sigma * 0.5 * (lo + hi)), _MM_FROUND_TO_NEAREST_INT);
    }
}

static void synth_tables(void) {
#pragma omp critical(orc_synth_tables)
    if (!g_tables_ready) { synth_table(0.02, g_table_s); synth_table(0.01, g_table_d); g_tables_ready = 1; }
}

/* Raw Q4_K tensors of synthetic expert (layer, expert): gate, up [I][H], down [H][I] as 144-byte super-blocks in blob order */
void orc_synth_q4k(unsigned seed, int layer, int expert, uint8_t* gate, uint8_t* up, uint8_t* down) {
    synth_tables();
    const size_t NB = (size_t)EH * EI / 256;
    for (size_t sb = 0; sb < 3 * NB; sb++) {
        uint8_t* d = sb < NB ? gate + sb * 144 : sb < 2 * NB ? up + (sb - NB) * 144 : down + (sb - 2 * NB) * 144;
        for (uint32_t j = 0; j < 36; j++) {
            const uint32_t w = synth_q4k_word(seed, layer, expert, sb, j, g_table_d);
            memcpy(d + 4 * j, &w, 4);
        }
    }
}

/* The synthetic expert (layer, expert) as a blob of format fmt */
int orc_synth_expert(int fmt, unsigned seed, int layer, int expert, uint8_t* dst) {
    synth_tables();
    if (fmt == FMT_ZP) {
        const size_t part = (size_t)EH * EI / 256 * 144;
        uint8_t* raw = (uint8_t*)malloc(3 * part);
        if (!raw) return -1;
        orc_synth_q4k(seed, layer, expert, raw, raw + part, raw + 2 * part);
        orc_q4k_to_zp(raw, raw + part, raw + 2 * part, dst);
        free(raw);
        return 0;
    }
    if (fmt != FMT_SYM_F32 && fmt != FMT_SYM_F16) return -1;
    for (size_t i = 0; i < Q_BYTES / 4; i++) {
        const uint32_t w = synth_nibble_word(seed, layer, expert, i);
        memcpy(dst + 4 * i, &w, 4);
    }
    for (size_t g = 0; g < CHUNKS / 2; g++) {
        const uint16_t h = synth_scale_h(seed, layer, expert, g, g_table_s);
        if (fmt == FMT_SYM_F16) memcpy(dst + Q_BYTES + 2 * g, &h, 2);
        else { const float f = orc_half(h); memcpy(dst + Q_BYTES + 4 * g, &f, 4); }
    }
    return 0;
}
