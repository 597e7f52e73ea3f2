/* moexb.h - C ABI of the B200 (sm_100a) MoE expert-FFN path.
 *
 * The reference engine ("moex") has no plugin or FFI boundary: its expert layer is a set of inline C++ launch wrappers
 * in src/kernels.cuh that Engine (src/moex.cu) calls on one CUDA stream, plus the CPU expert class in
 * src/cpu_expert.h and the GGUF block code in src/gguf.h. Each entry point below stands behind one of those functions,
 * with the same argument order, buffer shapes and ownership rules, and names the function it replaces (file:line in
 * the reference tree). Differences that a C ABI forces:
 *   - every function returns an int status (MOEXB_OK = 0, negative = error) instead of exiting; the text of the last
 *     error on the calling thread is moexb_last_error();
 *   - the reference's global "zero-point experts" switch g_zp (kernels.cuh:427) is an explicit `fmt` argument;
 *   - cudaStream_t is passed as void*.
 * As in the reference, the pointer-level entry points allocate nothing, never synchronise and never read device memory
 * on the host, so they can be captured in a CUDA graph; all buffers are device pointers owned by the caller unless a
 * parameter says "host". Geometry is fixed like the reference's constexprs (kernels.cuh:422): hidden H = 2048, expert
 * intermediate I = 512, quantisation group 64, so one expert holds 3*H*I = 3,145,728 int4 weights.
 */
#ifndef MOEXB_H
#define MOEXB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOEXB_H_DIM 2048
#define MOEXB_I_DIM 512
#define MOEXB_GROUP 64
#define MOEXB_Q_BYTES 1572864u /* packed nibbles of one expert, kernels.cuh:423 */

enum {
    MOEXB_OK = 0,
    MOEXB_ERR_ARG = -1,         /* bad argument (null pointer, size out of range, unknown format) */
    MOEXB_ERR_CUDA = -2,        /* a CUDA runtime call failed; see moexb_last_error() */
    MOEXB_ERR_UNSUPPORTED = -3, /* valid request that this build does not implement */
    MOEXB_ERR_NOMEM = -4
};

/* Expert blob formats. A blob is [gate I x H | up I x H | down H x I] packed int4 (byte k = element 2k in the low
 * nibble, 2k+1 in the high nibble, rows contiguous along the input dimension), followed by its scale part. */
enum {
    MOEXB_FMT_SYM_F32 = 0, /* two's-complement nibbles in [-8,7], one f32 scale per 64: the reference container layout
                              (kernels.cuh:413-415, EXPERT_BYTES_SYM = 1,769,472) */
    MOEXB_FMT_SYM_F16 = 1, /* same nibbles, one fp16 scale per 64 (1,671,168 bytes) */
    MOEXB_FMT_ZP = 2       /* unsigned nibbles, w = d*sc*u + dm*mn with [sc u8, mn i8] per 32 and half2 (d, dm) per 256:
                              the reference zero-point layout that holds GGUF Q4_K exactly (kernels.cuh:416-421,
                              EXPERT_BYTES_ZP = 1,818,624) */
};

/* How a resident layer keeps its expert blobs. TILED is the streaming layout of the B200 kernels: the same bytes as the
 * reference blob, re-ordered into contiguous 4-5 KB slices in tensor-core lane order (see moe_b200/csrc/tiled.cuh), so a
 * slice is one bulk copy; only the layer-level calls read it. REFERENCE keeps the reference blob as it is, which the
 * pointer-level entry points (moexb_experts_forward, moexb_pairs_forward, moexb_pairs_forward_tc) require. */
enum { MOEXB_LAYOUT_TILED = 0, MOEXB_LAYOUT_REFERENCE = 1 };

/* Activation element types accepted by the layer-level calls. */
enum { MOEXB_F32 = 0, MOEXB_BF16 = 1 };

typedef struct moexb_ctx moexb_ctx;     /* one per device (or more): stream-ordered workspace, synthetic tables */
typedef struct moexb_layer moexb_layer; /* one MoE layer resident in HBM: E routed experts + 1 shared + router */

/* Work list of the multi-token path, identical to kernels.cuh:688-689. */
typedef struct { const uint8_t* slot; int start, count; } moexb_pair_item; /* pairs[start, start+count) use this expert */
typedef struct { int t, p; float w; } moexb_pair;                          /* token row, output row of ypair, routing weight */

const char* moexb_last_error(void);
int moexb_version(void);
size_t moexb_expert_bytes(int fmt); /* 0 for an unknown format */

/* ---- router ------------------------------------------------------------------------------------------------------ */

/* y[r][o] = sum_i W[o][i] * x[r][i], fp32 accumulation in a fixed order (lane j of 32 takes elements 128c+4j..4j+3 for
 * c = 0,1,..; the 32 partial sums are combined by a xor-butterfly 16,8,4,2,1), so that the CPU oracle reproduces the
 * logits bit for bit and the selected experts cannot differ. Replaces gemv_f16 (kernels.cuh:73-96; call sites
 * moex.cu:1093, 1414). I must be a multiple of 128. W is F16 as the reference uploads the router (moex.cu:752-758). */
int moexb_gemv_f16(const void* W, const float* x, float* y, int I, int O, void* stream, int rows);
/* The same with fp32 weights. */
int moexb_gemv_f32(const float* W, const float* x, float* y, int I, int O, void* stream, int rows);

/* Softmax over E logits per token, then the K largest (ties -> lower index), in descending order; w = probability,
 * divided by the sum over the selected K when norm != 0. logits [T][ld] with ld >= E (ld lets the shared-expert gate
 * logit ride along as column E, as the reference appends it as router row E, moex.cu:876). Replaces router_topk
 * (kernels.cuh:373-411). E multiple of 32, E <= 1024, K <= 31. */
int moexb_router_topk(const float* logits, int E, int K, int norm, int* idx, float* w, void* stream, int T, int ld);

/* ---- routed experts, one token (decode) ---------------------------------------------------------------------------- */

/* act[k][I] = silu(gate_k x) * (up_k x); out[H] = sum_k w[k] * (down_k act_k), k in rank order. slots: device array of
 * K blob pointers; nh: optional device count of valid entries (0 gives zeros; a count above K is treated as K).
 * Replaces experts_forward (kernels.cuh:597-673). K <= 16. */
int moexb_experts_forward(int fmt, const uint8_t* const* slots, const float* w, int K, const float* x, float* act,
                          float* out, void* stream, const int* nh);
/* Which kernels moexb_experts_forward runs. Its reference signature carries no workspace, and the B200 streaming kernels
 * (cp.async.bulk rings, tensor-core MMA, exact hi + lo activations) need one for the 16-bit activation columns and the
 * per-expert rows; so an engine that wants them creates a context at start-up and names it here as the workspace of the
 * pointer-level one-token entry point on that device (null takes it away again; moexb_ctx_destroy does that by itself).
 * Without one - or with moexb_ctx_set_path(ctx, 1) - moexb_experts_forward runs the fp32 SIMT restatement of the
 * reference's own two kernels, which is kept as the on-device cross-check. Calls that share a context must not overlap
 * on the GPU. The multi-token counterpart with a workspace is moexb_pairs_forward_tc. */
int moexb_set_default_ctx(moexb_ctx* ctx, int device);

/* The same computation for callers that cannot allocate device memory (an engine that gave all free memory to its
 * expert cache at load time, or a decode thread that must never block in cudaMalloc). It has no counterpart in the
 * reference, which always receives `act` from its caller. The intermediate activations live in a fixed 32 KB array
 * inside the library image, which every GPU that loads the library keeps until the process exits, so there is no
 * `act` argument and K is limited to 16 experts per call (larger K is rejected with MOEXB_ERR_ARG). The function calls
 * no allocator. The first call on each device looks up the array's device address, and - with CUDA's default lazy module
 * loading - is also when the driver loads this library's kernels onto that device, which itself needs some device
 * memory: make one warm-up call per device and expert format at start-up, before the process commits the rest of the
 * memory and outside any stream capture. nh as in moexb_experts_forward (a count above K is treated as K).
 * All calls on a device share the array, which keeps the previous call's values: nothing in it needs
 * clearing between calls, but two calls whose kernels overlap on the GPU (different streams) race on it - keep them
 * on one stream or order them with events. */
int moexb_experts_forward_static(int fmt, const uint8_t* const* slots, const float* w, int K, const float* x, float* out,
                                 void* stream, const int* nh);

/* ---- routed experts, T tokens grouped by expert -------------------------------------------------------------------- */

/* For every pair of every item: act[p][I] = silu(gate x_t) * (up x_t), ypair[p][H] = w * (down act[p]).
 * Replaces pairs_forward / pairs_forward_dev (kernels.cuh:686-778): fp32 SIMT math, any token count per item.
 * In the _dev form the item count is read on the device (*nitems <= max_items), so a captured graph needs no host value. */
int moexb_pairs_forward(int fmt, const moexb_pair_item* items, int n_items, const moexb_pair* pairs, const float* X,
                        float* act, float* ypair, void* stream);
int moexb_pairs_forward_dev(int fmt, const moexb_pair_item* items, const int* nitems, int max_items,
                            const moexb_pair* pairs, const float* X, float* act, float* ypair, void* stream);

/* The same work list on the tensor-core streaming kernels (bf16 mma.sync, weights exact, activations as bf16 hi + lo,
 * fp32 accumulation and group scales). Stands behind pairs_forward_tc (kernels.cuh:780-965). Needs the context's
 * workspace: T <= max_tokens rows in X, npairs <= max_tokens * (top_k + 1); act (fp32 [npairs][I]) may be null. */
int moexb_pairs_forward_tc(moexb_ctx* ctx, int fmt, const moexb_pair_item* items, int n_items, const moexb_pair* pairs,
                           const float* X, int T, int npairs, float* act, float* ypair, void* stream);

/* moe[t][d] = sum_{r<K} ypair[t*K+r][d] (rank order) + (ycpu ? ycpu[t][d] : 0). Replaces pairs_reduce_k
 * (kernels.cuh:744-753). use_cpu: optional device flag, ycpu is added only if *use_cpu != 0. */
int moexb_pairs_reduce(const float* ypair, const float* ycpu, float* moe, int K, int D, int T, const int* use_cpu,
                       void* stream);
/* out[t][d] += sh[t][d] * sigmoid(gl[t*gl_stride]). Replaces gated_add_k / gated_add_rows_k (kernels.cuh:973-977,
 * 1101-1106). */
int moexb_gated_add_rows(float* out, const float* sh, const float* gl, int gl_stride, int D, int T, void* stream);

/* Shared expert held as one int4 blob of the routed experts' shape: out[t] += sigmoid(gl[t*gl_stride]) *
 * down(silu(gate x_t) * up x_t) for t < T. scratch: >= T*(I + H + 3) + 4 floats, 16-byte aligned. Stands behind shared_expert_add
 * (kernels.cuh:2018-2028) and shared_rows (moex.cu:1674-1682), whose dense int8/int6 weight matrices are replaced by
 * an expert blob. */
int moexb_shared_expert_add(int fmt, const uint8_t* blob, const float* gl, int gl_stride, const float* X, int T,
                            float* out, float* scratch, void* stream);

/* Bucket the T*K (token, rank) pairs by expert id: items in ascending expert id, pairs in token order inside an
 * expert, p = t*K + rank, as the host loop at moex.cu:1466-1486 and route_export_k (kernels.cuh:1020-1054) do.
 * slot_table: E blob pointers (null = expert not held here: its pairs are dropped, which is how an expert-parallel
 * rank sees only its own experts). items: E entries; pairs: T*K entries; nitems: 1 int; counts: E ints of scratch. */
int moexb_group_pairs(const int* idx, const float* w, int T, int K, int E, const uint8_t* const* slot_table,
                      moexb_pair_item* items, moexb_pair* pairs, int* nitems, int* counts, void* stream);

/* ---- formats -------------------------------------------------------------------------------------------------------- */

/* Every weight of a blob as fp32, in blob order [gate | up | down] (3*H*I floats): q*scale for the symmetric formats
 * (ref/qwen36_ref.py:45-59), (d*sc)*u + dm*mn for zero point (gguf.h:332-335). For the bit-exact weight check. */
int moexb_dequant(int fmt, const uint8_t* blob, float* out, void* stream);
/* n values (a multiple of 256) of raw GGUF Q4_K super-blocks (144 bytes each) as fp32: y = (d*s_j)*q - dmin*m_j.
 * Replaces gg_dequant(GG_Q4_K, ...) (gguf.h:98-110). */
int moexb_q4k_dequant(const uint8_t* blocks, long long n, float* y, void* stream);
/* One expert from raw Q4_K tensors (gate [I][H], up [I][H], down [H][I], rows of cols/256 super-blocks) to a
 * MOEXB_FMT_ZP blob, bit-preserving. Replaces gg_q4k_zp / gg_zp_row / the per-expert body of gg_experts
 * (gguf.h:261-270, 302-330, 666-694). */
int moexb_q4k_to_zp(const uint8_t* gate, const uint8_t* up, const uint8_t* down, uint8_t* blob, void* stream);

/* ---- synthetic experts (seeded, identical bytes on host and device) ----------------------------------------------- */

/* Fill dst (device) with n consecutive experts e0..e0+n-1 of `layer` in format fmt (blob stride =
 * moexb_expert_bytes(fmt)); MOEXB_FMT_ZP experts are synthetic Q4_K super-blocks converted as moexb_q4k_to_zp does. */
int moexb_synth_experts(moexb_ctx* ctx, int fmt, unsigned seed, int layer, int e0, int n, uint8_t* dst, void* stream);
/* The same bytes for one expert, written to host memory; needs no GPU. */
int moexb_synth_expert_host(int fmt, unsigned seed, int layer, int expert, uint8_t* dst_host);
/* Raw Q4_K tensors of one synthetic expert on the host: gate, up (I*H/256*144 bytes each), down (H*I/256*144). */
int moexb_synth_q4k_host(unsigned seed, int layer, int expert, uint8_t* gate, uint8_t* up, uint8_t* down);

/* ---- resident layers -------------------------------------------------------------------------------------------------- */

/* max_tokens, max_experts (routed experts per layer, a multiple of 32 up to 1024) and top_k (<= 15) bound the
 * layer-level calls; their workspace (about max_tokens * (top_k + 1) * 10 KB) is allocated here, once. */
int moexb_ctx_create(int device, int max_tokens, int max_experts, int top_k, moexb_ctx** out);
int moexb_ctx_destroy(moexb_ctx* ctx);
/* Which expert kernels the layer-level calls use on a REFERENCE-layout layer: 0 = the streaming tensor-core kernels on
 * 256-byte row pieces (default), 1 = the fp32 SIMT kernels (the restatement of the reference's pairs_forward /
 * experts_forward, kept for cross-checks). TILED layers always use the tiled streaming kernels. */
int moexb_ctx_set_path(moexb_ctx* ctx, int path);
/* Batches of at least this many tokens run the experts on the tcgen05 grouped GEMM (TILED layers, symmetric formats);
 * smaller ones on the streaming kernels. Default 256. */
int moexb_ctx_set_prefill_min_tokens(moexb_ctx* ctx, int tokens);
/* Pairs of one expert that a pass of the tiled streaming kernels takes (batches of 8 to prefill_min_tokens - 1 tokens,
 * symmetric formats): 8 (default; an expert with 5-8 pairs is unpacked once) or 4. Smaller batches and zero-point blobs
 * always take 4. */
int moexb_ctx_set_pairs_per_pass(moexb_ctx* ctx, int pairs);
/* A stack of residual blocks for ONE token (TILED layers, every expert held here) runs as a single
 * cooperative launch that walks all layers with grid barriers inside (default on); 0 = the graph of per-layer kernels.
 * Read when a stack is created. */
int moexb_ctx_set_fused_decode(moexb_ctx* ctx, int on);
/* Waits for the device and reads the error word of the kernels: 0 = none; 1 / 2 = a consumer warp / the producer warp of a
 * streaming kernel gave up waiting on a pipeline barrier, 3 = the same in the tensor-core grouped GEMM, 5 / 6 = the one-token
 * stack kernel gave up at a grid barrier / on a weight copy, 7 / 8 = an expert-parallel rank gave up waiting for a peer's
 * dispatch / combine flag (every device-side wait is bounded). The word is cleared. */
int moexb_ctx_status(moexb_ctx* ctx, int* status);
/* Exercises the time-out path of the bounded waits without touching any data: which = 0 launches one warp that waits on a
 * pipeline barrier whose bytes never arrive, which = 1 a one-CTA grid at a grid barrier that expects two arrivals; both
 * give up after `polls` polls (1..2^20) instead of the production limit; which = 2 the same for the expert-parallel
 * kernels' wait on a flag that a peer GPU raises. *status receives what moexb_ctx_status then reports (1, 5 and 8) and the
 * word is cleared. The counterpart of the reference's wait_add_k giving up after timeout_ns and
 * raising its abort word (kernels.cuh:1055-1089). */
int moexb_ctx_selftest_timeout(moexb_ctx* ctx, int which, int polls, int* status);

/* Allocates the image of one layer: n_routed experts (ids 0..n_routed-1) and the shared expert (id n_routed), each a
 * blob of format fmt, plus the router [n_routed+1][H] (row n_routed = the shared expert's gate vector).
 * first_local/n_local select the routed experts this process holds (expert parallelism); the others take no memory and
 * their pairs are dropped by moexb_group_pairs. router_dtype: MOEXB_F32, or 2 for F16 as the reference stores it. */
int moexb_layer_create(moexb_ctx* ctx, int fmt, int n_routed, int first_local, int n_local, int router_dtype, int layout,
                       moexb_layer** out);
int moexb_layer_destroy(moexb_layer* layer);
/* Device pointer of expert e's blob in the layer's layout (e == n_routed: shared expert); null if not held. */
uint8_t* moexb_layer_blob(moexb_layer* layer, int e);
/* Device array of n_routed+1 blob pointers (null = not held), usable as `slot_table`. */
const uint8_t* const* moexb_layer_slot_table(moexb_layer* layer);
/* Copies one expert blob (format of the layer, moexb_expert_bytes(fmt) bytes, host memory) into expert e's place; the
 * role of the reference's slot admission copy (moex.cu:257) with every expert resident. The blob is given in the
 * reference layout and converted on the device when the layer is TILED. Synchronous. */
int moexb_layer_upload_expert(moexb_layer* layer, int e, const uint8_t* blob_host);
/* The inverse: expert e's blob back in the reference layout, to host memory. Synchronous. */
int moexb_layer_export_expert(moexb_layer* layer, int e, uint8_t* blob_host);
/* Copies router weights from the host: W [n_routed+1][H] in the layer's router dtype. */
int moexb_layer_set_router(moexb_layer* layer, const void* W_host);
void* moexb_layer_router(moexb_layer* layer);
/* Fills all held experts with synthetic weights (moexb_synth_experts with this layer's format). */
int moexb_layer_fill_synth(moexb_layer* layer, unsigned seed, int layer_index, void* stream);

/* ---- GGUF ingest ------------------------------------------------------------------------------------------------------ */

/* A GGUF model file (versions 2 and 3), mapped read-only with its tensor directory parsed; needs no GPU. Stands where
 * the reference's importer opens the file (gguf.h:345-462, struct Gguf: magic, version, metadata, general.alignment,
 * tensor directory, every length checked against the file size). A file that is truncated, corrupt or not GGUF gives
 * MOEXB_ERR_ARG with the reason in moexb_last_error(). */
typedef struct moexb_gguf moexb_gguf;
int moexb_gguf_open(const char* path, moexb_gguf** out);
int moexb_gguf_close(moexb_gguf* g);
int moexb_gguf_tensor_count(const moexb_gguf* g);
const char* moexb_gguf_tensor_name(const moexb_gguf* g, int i); /* null when i is out of range */
/* One tensor by name (Gguf::at, gguf.h:373-377): ggml type, dimensions ne[0..3] (ne[0] = row length, unused ones 1),
 * a pointer into the mapping and the tensor's size in bytes (null / 0 for a ggml type whose block size is not known
 * here). Any out pointer may be null. */
int moexb_gguf_tensor(const moexb_gguf* g, const char* name, int* type, int* n_dims, long long* ne, const void** data,
                      long long* nbytes);
/* The block formats other than Q4_K, on the host (no GPU): moexb_gguf_dequant_host stands behind gg_dequant (gguf.h:85-255)
 * for ggml types F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q4_K, Q5_K, Q6_K, IQ4_NL and IQ4_XS (n a multiple of the
 * block size); moexb_gguf_row_to_zp behind gg_zp_row (gguf.h:302-330): one row of `cols` weights (a multiple of 256) into
 * the zero-point form - qb[cols / 2] nibble bytes, cs[cols / 32 * 2] = [sc, mn] per 32, sup[cols / 256 * 2] = (d, dm) as
 * fp16 bits per 256 - bit for bit for Q4_K, by the reference's least-squares refit per 32 weights (gguf.h:272-300) for the
 * others. Other ggml types give MOEXB_ERR_UNSUPPORTED. */
int moexb_gguf_dequant_host(int ggml_type, const uint8_t* src_host, long long n, float* y_host);
int moexb_gguf_row_to_zp(int ggml_type, const uint8_t* src_host, int cols, uint8_t* qb, uint8_t* cs, uint16_t* sup);
/* Fills a MOEXB_FMT_ZP layer from block `block` of the file: blk.N.ffn_{gate,up,down}_exps.weight (Q4_K, shapes
 * [H, I, E], [H, I, E], [I, H, E] with E = the layer's n_routed) for the routed experts the layer holds, re-packed on
 * the device exactly as moexb_q4k_to_zp does; the role of gg_experts (gguf.h:666-694) without the pass through a
 * container on disk. Also, when present: the shared expert from blk.N.ffn_{gate,up,down}_shexp.weight if all three
 * are Q4_K, the router rows from blk.N.ffn_gate_inp.weight and the shared expert's gate vector from
 * blk.N.ffn_gate_inp_shexp.weight (F32, F16 or BF16, converted to the layer's router dtype). *loaded (may be null)
 * receives a bit set: 1 routed experts, 2 shared expert, 4 router rows, 8 shared gate vector; what a bit does not
 * name is left as it was. Expert tensors in one of the other types moexb_gguf_row_to_zp reads are re-quantised to 4 bits on
 * the host (all host threads) as the reference's importer does (gg_experts, gguf.h:666-694); any other ggml type gives
 * MOEXB_ERR_UNSUPPORTED. Synchronous. */
int moexb_layer_load_gguf(moexb_layer* layer, const moexb_gguf* g, int block, int* loaded);

/* ---- safetensors container ingest ---------------------------------------------------------------------------------- */

/* One safetensors file of the reference engine's model container (one per layer), mapped read-only with its JSON
 * directory parsed; needs no GPU. Stands where the reference indexes and maps the files (st.h:19-111, struct
 * Container: index(), at(), map()). A malformed header or offsets outside the file give MOEXB_ERR_ARG with the reason
 * in moexb_last_error() (the reference prints and exits). */
typedef struct moexb_st moexb_st;
int moexb_st_open(const char* path, moexb_st** out);
int moexb_st_close(moexb_st* s);
int moexb_st_tensor_count(const moexb_st* s);
const char* moexb_st_tensor_name(const moexb_st* s, int i); /* null when i is out of range */
/* One tensor by name (Container::at / map, st.h:30-35, 64-84): dtype string (buffer of 8 chars), number of dimensions,
 * shape (the first 8 dimensions at most, and n_dims counts only those), a pointer into the mapping and the size in
 * bytes. Any out pointer may be null. */
int moexb_st_tensor(const moexb_st* s, const char* name, char* dtype, int* n_dims, long long* shape, const void** data,
                    long long* nbytes);
/* Fills a layer from a container file: for every routed expert e the layer holds, `<prefix>mlp.experts.<e>.merged_weight`
 * (the packed nibbles) and `<prefix>mlp.experts.<e>.qs` (the scale part) as the engine reads them (moex.cu:933-939), with
 * prefix = "model.layers.<l>." or "mtp.layers.0."; F32 `qs` for the symmetric formats, U8 `qs` for MOEXB_FMT_ZP
 * (moex.cu:221-225). A MOEXB_FMT_SYM_F16 layer takes F32 scales only if each of them is an fp16 value (nothing is
 * rounded on the way in); otherwise, and for a `qs` of the other format, MOEXB_ERR_UNSUPPORTED. Also, when present,
 * the router rows `<prefix>mlp.gate.weight` [E][H] and the shared expert's gate vector
 * `<prefix>mlp.shared_expert_gate.weight` [1][H] (F32, F16 or BF16), converted to the layer's router dtype. The
 * container holds the shared expert as dense matrices (moex.cu:768), not as an expert blob: it is left as it was.
 * *loaded (may be null): bit 1 routed experts, 4 router rows, 8 shared gate vector. Synchronous. */
int moexb_layer_load_st(moexb_layer* layer, const moexb_st* s, const char* prefix, int* loaded);

/* One MoE layer for T tokens: router logits -> top-K softmax (renormalised) -> routed experts -> rank-order combine ->
 * + sigmoid(gate) * shared expert. X [T][H] of x_dtype; out [T][H] f32. The sequence the reference runs at
 * moex.cu:1093-1107 (decode) and moex.cu:1414-1415, 1466-1617 (chunk). Optional outputs (may be null): idx_out [T][K],
 * w_out [T][K]. flags bit 0: skip the shared expert; bit 1: X is the layer input before RMSNorm, so normalise it first
 * (unit weight, eps 1e-6) and write out = X + moe(norm(X)) - the residual block the 40-layer stack chains. */
int moexb_layer_forward(moexb_ctx* ctx, moexb_layer* layer, const void* X, int x_dtype, int T, int K, float* out,
                        int* idx_out, float* w_out, int flags, void* stream);

/* The expert-parallel share of one residual block. Every rank of R holds the router, the shared expert and a slice of
 * the routed experts (first_local / n_local of moexb_layer_create) and sees all T tokens: it normalises X, routes every
 * token (the logits are bit-identical on all ranks), runs the pairs of the experts it holds, and the shared expert for
 * the tokens [shared_t0, shared_t1) only. out [T][H] = that partial sum, without the residual; the ranks' outputs are
 * then added (one all-reduce, the path's only exchange) and x_next = X + sum. pre_normed != 0: the context already holds
 * the normalised X (left by moexb_ep_residual_norm of the previous layer). The reference has no multi-GPU path. */
int moexb_layer_forward_ep(moexb_ctx* ctx, moexb_layer* layer, const void* X, int x_dtype, int T, int K, float* out,
                           int* idx_out, float* w_out, int shared_t0, int shared_t1, int pre_normed, void* stream);
/* After the all-reduce: out = x + total (out may be x), and, when `next` is given, the normalised out and its 16-bit
 * split are left in the context for next's moexb_layer_forward_ep(pre_normed = 1). */
int moexb_ep_residual_norm(moexb_ctx* ctx, moexb_layer* next, const float* x, const float* total, float* out, int T,
                           void* stream);

/* ---- expert parallelism with the token all-to-all over peer memory ------------------------------------------------------ */

/* The path the batched configurations use on 2, 4 or 8 GPUs of one NVLink node, one process per GPU. Rank r of `world` holds
 * the routed experts [r * E / world, (r + 1) * E / world) of every layer (moexb_layer_create's first_local / n_local; router
 * and shared expert on every rank) and OWNS the tokens [r * T / world, (r + 1) * T / world) (remainders to the first ranks):
 * it keeps their residual rows, normalises and routes them, runs the shared expert for them and returns their outputs. Per
 * layer the kernels exchange, by plain stores into the peers' mapped "exchange buffers": each token's ids and weights to
 * every rank and its normalised activation row to the ranks that hold one of its selected experts (dispatch); and one
 * partial output row per (token, rank that ran one of its experts) back to the token's owner (combine), who adds the
 * partial rows in rank order, the shared expert and the residual. Flags in the same buffers order the steps; every wait on
 * a peer is bounded (moexb_ctx_status reports 7 / 8 when a dispatch / combine flag never came). No NCCL call is made. The
 * reference has no multi-GPU path; the grouping that is sharded is the host loop at moex.cu:1466-1506, and the bounded
 * device-side wait follows wait_add_k (kernels.cuh:1055-1089).
 *
 * Exchange buffers: every rank allocates one (moexb_ep_buffer_alloc, which also returns a 64-byte handle), passes the handle
 * to the other processes by any means (the tests and the benchmark use torch.distributed), and maps the others'
 * (moexb_ep_buffer_open: cudaIpcOpenMemHandle, peer access enabled on demand). In one process (several contexts on one GPU:
 * how the single-GPU tests drive this path) the pointers are used as they are. */
typedef struct moexb_ep moexb_ep;
size_t moexb_ep_buffer_bytes(int max_tokens, int top_k, int world); /* 0 for bad arguments; world <= 8 */
int moexb_ep_buffer_alloc(size_t bytes, void** ptr, unsigned char* handle64 /* may be null */);
int moexb_ep_buffer_open(const unsigned char* handle64, void** ptr);
int moexb_ep_buffer_close(void* ptr); /* a pointer from moexb_ep_buffer_open */
int moexb_ep_buffer_free(void* ptr);  /* a pointer from moexb_ep_buffer_alloc */
/* bufs[world]: the exchange buffer of every rank as a device pointer valid in this process (bufs[rank] = the local one), each
 * of moexb_ep_buffer_bytes(T, K, world) bytes. T tokens per step (world <= T <= the context's max_tokens), K experts per
 * token, n_routed routed experts per layer. While the object exists the context's activation, id and weight workspace lives
 * in the local exchange buffer: use the context for this path only. */
int moexb_ep_create(moexb_ctx* ctx, int rank, int world, int T, int K, int n_routed, void* const* bufs, moexb_ep** out);
int moexb_ep_destroy(moexb_ep* ep);
int moexb_ep_own_tokens(const moexb_ep* ep, int* first, int* count);
/* Optional outputs (either may be null): the selected experts and routing weights [T][K] of ALL tokens as this rank holds
 * them after moexb_ep_experts of a layer (its own tokens' from its router, the others' as the peers sent them). */
int moexb_ep_read_routing(moexb_ep* ep, int* idx_out, float* w_out, void* stream);
/* A step = begin_step, then for each layer l = 0.. dispatch(l) and experts(l), then finish. Every rank makes the same calls
 * in the same order; all are enqueued on `stream` without synchronising and can be captured in a CUDA graph.
 *   begin_step  advances the step number the flags carry.
 *   dispatch    l == 0: takes the own rows of X [T][H] (x_dtype; every rank passes the whole batch); l > 0: adds up layer
 *               l - 1 for the own tokens (waits for the peers' partial rows). Then normalises (residual != 0: the blocks
 *               x_{l+1} = x_l + moe_l(rmsnorm(x_l)); residual == 0: the plain layer moe(X), single layer only), routes the
 *               own tokens and sends ids, weights and activation rows.
 *   experts     waits for all ranks' dispatch of layer l, runs the pairs of the experts held here (and the shared expert for
 *               the own tokens) and sends the partial rows to the token owners.
 *   finish      adds up the last layer: out_own [own tokens][H] f32. */
int moexb_ep_begin_step(moexb_ep* ep, void* stream);
int moexb_ep_dispatch(moexb_ep* ep, moexb_layer* layer, int l, const void* X, int x_dtype, int residual, void* stream);
int moexb_ep_experts(moexb_ep* ep, moexb_layer* layer, int l, void* stream);
int moexb_ep_finish(moexb_ep* ep, int n_layers, int residual, float* out_own, void* stream);
/* The whole step in one call. */
int moexb_ep_step(moexb_ep* ep, moexb_layer* const* layers, int n_layers, const void* X, int x_dtype, int residual,
                  float* out_own, void* stream);

/* ---- a stack of layers as one replayable unit ---------------------------------------------------------------------- */

typedef struct moexb_stack moexb_stack;

/* Chains n_layers residual blocks x_{l+1} = x_l + moe_l(rmsnorm(x_l)) (unit norm weight, eps 1e-6; the structure of
 * the reference's decoder block around its MoE, moex.cu:1082, 1092) for a fixed token count T and captures the whole
 * sequence of launches in one CUDA graph, as the reference captures its per-step graph (moex.cu:1165-1181).
 * Input [T][H] of x_dtype, output x_{n_layers} [T][H] f32. residual = 0 chains the plain layers instead,
 * x_{l+1} = moe_l(x_l) (one layer: exactly moexb_layer_forward). The layers must outlive the stack.
 * A residual stack for T = 1 is not a graph but one cooperative kernel over all layers (moexb_ctx_set_fused_decode):
 * moexb_stack_run then issues a cudaMemsetAsync and a cooperative launch, which takes every SM of the device - launch it
 * outside stream capture, and do not expect other kernels to run beside it. A context's stacks and layers share its
 * workspace: their calls must not overlap on the GPU. */
int moexb_stack_create(moexb_ctx* ctx, moexb_layer* const* layers, int n_layers, int T, int K, int x_dtype, int residual,
                       moexb_stack** out);
int moexb_stack_destroy(moexb_stack* stack);
/* Device buffers: copies X in, replays the graph (or launches the one-token kernel), copies the result to out; all on
 * `stream`, no synchronisation. */
int moexb_stack_run(moexb_stack* stack, const void* X, float* out, void* stream);
/* Host buffers (pinned memory recommended): host->device copy of X, the graph, device->host copy of the result, then
 * waits for the stream. This is the call an engine that keeps activations on the host makes once per step. */
int moexb_stack_run_host(moexb_stack* stack, const void* X_host, float* out_host, void* stream);
/* The expert-parallel step (moexb_ep_step) captured as one CUDA graph: moexb_stack_run / _run_host then take the whole batch
 * X [T][H] and return this rank's own rows [own tokens][H]. Every rank replays its graph once per step. */
int moexb_ep_stack_create(moexb_ep* ep, moexb_layer* const* layers, int n_layers, int x_dtype, int residual, struct moexb_stack** out);
/* Kernel launches of one replay. */
int moexb_stack_kernel_count(moexb_stack* stack);

/* ---- instrumentation ------------------------------------------------------------------------------------------------ */

/* Kernels launched by this library in this process so far (graph replays count their kernel nodes). */
long long moexb_launch_count(void);

enum { MOEXB_PROF_ROUTER = 0, MOEXB_PROF_TOPK = 1, MOEXB_PROF_GROUP = 2, MOEXB_PROF_GATE_UP = 3, MOEXB_PROF_DOWN = 4,
       MOEXB_PROF_COMBINE = 5, MOEXB_PROF_OTHER = 6, MOEXB_PROF_TAGS = 7 };
/* While on, moexb_layer_forward brackets each of its kernels with CUDA events on the launching stream (not valid during
 * graph capture). moexb_ctx_profile_read waits for the device, then returns per tag the summed kernel time in ms and
 * the number of launches since the last read (arrays of MOEXB_PROF_TAGS), and clears the records. */
int moexb_ctx_profile(moexb_ctx* ctx, int on);
int moexb_ctx_profile_read(moexb_ctx* ctx, float* ms, int* launches);

#ifdef __cplusplus
}
#endif
#endif
