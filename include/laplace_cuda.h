/*
 * laplace_cuda.h - C ABI of the B200 (sm_100a) back-end for Laplace's
 * block-quantized weight matmul.
 *
 * The library replaces the box that Laplace calls its "SIMD back-end": the
 * three function pointers of src/kernels.h:92-119 and the weight-registration
 * hook of src/matmul.h:26. Every entry point below names the reference
 * interface it stands in for. Signatures carry plain pointers and sizes only.
 *
 * Conventions (all taken from the reference, src/matmul_simd.cpp:432-544):
 *   - a weight matrix is N contiguous rows of K elements in GGUF block format;
 *     one row is rb = K / elems_per_block * bytes_per_block bytes;
 *   - stacked experts are contiguous, N * rb bytes apart;
 *   - x is fp32 row-major, y is fp32 row-major and is OVERWRITTEN;
 *   - activations are quantized per 32 values to int8 with an fp32 scale
 *     (amax / 127) before the dot products; block sums are exact integers.
 *
 * Return values: 0 = done; 1 = this weight type is not handled here (the
 * reference's contract for "return false, caller falls back", kernels.h:94-96);
 * negative = error (see enum). No entry point ever computes on the CPU.
 *
 * Threading: one caller at a time per process, like the reference
 * (src/threadpool.h:236-257 has a single dispatch slot). Host-pointer entry
 * points are synchronous. *_dev entry points only enqueue work on the given
 * stream.
 */
#ifndef LAPLACE_CUDA_H
#define LAPLACE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids, src/tensor.h:11-34 */
#define LAPLACE_TYPE_Q4_0 2u
#define LAPLACE_TYPE_Q5_0 6u
#define LAPLACE_TYPE_Q8_0 8u
#define LAPLACE_TYPE_Q4_K 12u
#define LAPLACE_TYPE_Q6_K 14u

enum {
    LAPLACE_OK            = 0,
    LAPLACE_UNSUPPORTED   = 1,   /* type not handled: caller may fall back */
    LAPLACE_ERR_ARG       = -1,  /* null pointer, bad size, K not a block multiple */
    LAPLACE_ERR_CUDA      = -2,  /* a CUDA call failed; text in laplace_cuda_last_error() */
    LAPLACE_ERR_STATE     = -3,  /* not initialised / no CUDA device */
    LAPLACE_ERR_TIMEOUT   = -4,  /* a bounded device-side wait gave up */
    LAPLACE_ERR_LIMIT     = -5   /* request exceeds a documented size limit */
};

/* ---- lifetime ---------------------------------------------------------- */

/* Binds the calling process to one GPU and creates the library's stream and
 * scratch. Safe to call again with the same device. No reference counterpart
 * (the reference has no device); called from the shim's static initialiser. */
int  laplace_cuda_init(int device);
void laplace_cuda_shutdown(void);
/* Drains the library's own stream, then reads and clears the device status word (time-outs of bounded waits,
 * bad expert indices). Work enqueued by *_dev calls on a CALLER's stream is not waited for here: synchronise that
 * stream first, or use laplace_cuda_sync_stream, otherwise a status raised by such work can be missed or be
 * attributed to a later call. */
int  laplace_cuda_sync(void);
/* The same after waiting for `stream` (a cudaStream_t) as well. */
int  laplace_cuda_sync_stream(void* stream);
const char* laplace_cuda_last_error(void);
int  laplace_cuda_sm_count(void);

/* ---- weights ----------------------------------------------------------- */

/* Replaces matmul_register_weights(base, size) (src/matmul.h:26, called once
 * per model at src/main.cpp:705; Metal version src/metal.mm:552-584). Copies
 * the whole mapped file region into HBM. Later calls that pass a weight
 * pointer inside [base, base+size) resolve it by offset, as
 * src/metal.mm:590-599 does. Weight pointers outside every registered region
 * are uploaded for that call only. */
int laplace_cuda_register_weights(const void* base, size_t size);
int laplace_cuda_unregister_weights(const void* base);

/* Row range [row_begin, row_end) of an N-row matrix as seen by rank `rank`
 * of `world` when the matrix is split along N (no reference counterpart; the
 * reference is single-device). */
void laplace_cuda_nsplit(int N, int rank, int world, int* row_begin, int* row_end);

/* Scratch memory and CUDA graphs. laplace_cuda_gemm_dev (more than 8 activation rows), laplace_cuda_moe_grouped_dev,
 * laplace_cuda_moe_ffn_dev and laplace_cuda_gemm_peers_dev keep their quantized operands in scratch buffers that grow to
 * the largest call seen. A buffer that was handed to a launch is never freed before laplace_cuda_shutdown (a captured
 * graph may hold its address), but growing calls the allocator, which is illegal while the call's stream is being
 * captured: such a call returns LAPLACE_ERR_STATE and leaves the capture valid. Make every call shape once before
 * capturing it. Calls that share a scratch buffer must not overlap on the GPU (one stream, or the caller's own
 * ordering). laplace_cuda_gemm_dev with 3 to 8 rows of Q4_K uses a fixed array inside the library in the same way. */

/* ---- the three back-end entry points (host pointers) -------------------- */

/* Replaces kernels::gemm_fn (src/kernels.h:97), implemented in the reference
 * by gemm_simd (src/matmul_simd.cpp:480-496): y[m*N+j] = dot(x[m], row j).
 * Q4_0, Q5_0, Q8_0, Q4_K and Q6_K are computed as that back-end computes them (activations quantized to Q8 per 32
 * values, integer block sums, fp32 scales); the three MoE entry points below take the same five types. More than 8
 * rows run on the tensor cores for Q4_0 / Q8_0 / Q4_K / Q6_K when K % 256 == 0, otherwise (and for Q5_0) in passes
 * of 8 rows through the streaming kernel. */
int laplace_cuda_gemm(const float* x, const uint8_t* w, uint32_t type,
                      float* y, int M, int K, int N);

/* Replaces kernels::moe_gemv_fn (src/kernels.h:103; src/matmul_simd.cpp:506-522):
 * y[k*N+j] = dot(x, row j of expert expert_idx[k]); one shared x of length K. */
int laplace_cuda_moe_gemv(const float* x, const uint8_t* w, uint32_t type,
                          const int* expert_idx, int n_experts,
                          float* y, int K, int N);

/* Replaces kernels::moe_gemv_multi_fn (src/kernels.h:110;
 * src/matmul_simd.cpp:527-544): as above with x[k*K..] per selected expert. */
int laplace_cuda_moe_gemv_multi(const float* x, const uint8_t* w, uint32_t type,
                                const int* expert_idx, int n_experts,
                                float* y, int K, int N);

/* ---- device-pointer twins (all pointers are device memory) -------------- */

/* `stream` is a cudaStream_t passed as void* (NULL = the library's stream). */
int laplace_cuda_gemm_dev(const float* x, const uint8_t* w, uint32_t type,
                          float* y, int M, int K, int N, void* stream);
int laplace_cuda_moe_gemv_dev(const float* x, const uint8_t* w, uint32_t type,
                              const int* expert_idx, int n_experts,
                              float* y, int K, int N, int per_expert_x, void* stream);

/* Several weight matrices of one type and one K against the SAME activation rows in one launch, with an optional
 * RMSNorm in front: what the reference does as  ops::rmsnorm(x, w_norm, x_norm)  followed by one matmul_rows call per
 * matrix on x_norm (src/ops.cpp:34-74; src/arch_llama.cpp:475-501: q, k, v after the attention norm, gate and up
 * after the FFN norm - it quantizes x_norm again for every matrix). Here x is normalised (norm_weight != NULL:
 * x_norm = x * 1/sqrt(mean(x^2) + norm_eps) * norm_weight, fp32) and quantized ONCE inside the kernel's prologue and
 * every matrix streams past it: y_i[m*N_i + j] = dot(quantize(x_norm[m]), row j of matrix i). x_norm_out (optional)
 * receives the normalised rows [M][K]. 1..8 matrices. Device pointers. With M <= 8 (decode) everything is one launch;
 * with more rows (prefill; K a multiple of 256) one quantizer launch normalises and quantizes the rows once and every
 * matrix then runs as a tensor-core GEMM on that shared operand. */
typedef struct { const uint8_t* w; float* y; int N; } laplace_cuda_matrix;
int laplace_cuda_gemm_multi_dev(const float* x, const float* norm_weight, float norm_eps, float* x_norm_out,
                                const laplace_cuda_matrix* mats, int n_mats, uint32_t type, int M, int K, void* stream);

/* Expert-grouped matmul for a batch of tokens. The reference runs a mixture-of-experts layer
 * token by token: one fused_moe_gemm_idx call per token for gate/up (src/matmul.h:36-44,
 * src/arch_gemma4.cpp:604) and one fused_moe_gemm_multi call for down (src/matmul.h:46-54,
 * src/arch_gemma4.cpp:626). This entry point computes what T such calls compute, in one pass over
 * the expert weights: for every pair p < n_pairs
 *     y[p*N + j] = dot(x[pair_row[p]*K ...], row j of expert pair_expert[p]).
 * pair_row = NULL means pair p reads x row p (the "multi" form: one input per selected expert);
 * for the shared-input form pass pair_row[p] = token of pair p. Pairs may come in any order; they
 * are grouped by expert on the device. Q4_0, Q8_0, Q4_K and Q6_K with K % 256 == 0; anything else
 * returns LAPLACE_UNSUPPORTED and the caller loops laplace_cuda_moe_gemv_dev per token.
 * A negative expert index marks a pair that is not computed here (its y row is left untouched):
 * with experts placed on several GPUs every GPU passes the whole pair list with the experts of
 * the other GPUs set to -1. An index >= n_experts_total also skips the pair and makes the next
 * laplace_cuda_sync() return LAPLACE_ERR_ARG. x must be 16-byte aligned, Q4_K weights too (other types: 2 bytes).
 * All pointers are device memory. */
int laplace_cuda_moe_grouped_dev(const float* x, const uint8_t* w, uint32_t type,
                                 const int* pair_expert, const int* pair_row,
                                 int n_pairs, int n_experts_total,
                                 float* y, int K, int N, void* stream);

/* The expert FFN of a mixture-of-experts layer for a batch of tokens, fused: what the reference
 * does per token in src/arch_gemma4.cpp:600-638 - fused_moe_gemm_idx over the token's experts
 * (gate and up rows stacked, N = 2*inter), ops::swiglu / ops::geglu (src/ops.cpp:128-176),
 * fused_moe_gemm_multi (down), out = sum_k top_w[k] * expert_out[k] - with one device-side
 * grouping shared by both matmuls and the intermediate results kept in grouped order.
 *   x [n_tokens][hidden]; w_gate_up: experts x (2*inter rows of K = hidden), gate rows first;
 *   w_down: experts x (hidden rows of K = inter); top_idx / top_w [n_tokens][top_k];
 *   activation 0 = SwiGLU (silu(gate) * up), 1 = GeGLU (tanh-GELU(gate) * up);
 *   down_scale (optional, may be NULL): per-expert output scale, indexed like top_idx (by the ids this call
 *   sees, i.e. local ids on an expert-parallel GPU); the weight of a pair is top_w * down_scale[expert], as in
 *   src/arch_gemma4.cpp:634-638;
 *   out [n_tokens][hidden] is OVERWRITTEN with the weighted sum over the experts computed here.
 * Negative entries of top_idx are experts that live on another GPU: they contribute nothing, so
 * the per-GPU outputs of an expert-parallel layer add up to the layer's output. h_out (optional,
 * may be NULL) receives the activation result per pair, [n_tokens*top_k][inter] (rows of skipped
 * pairs untouched). Types as for laplace_cuda_moe_grouped_dev, else LAPLACE_UNSUPPORTED. */
int laplace_cuda_moe_ffn_dev(const float* x, const uint8_t* w_gate_up, const uint8_t* w_down,
                             uint32_t type_gate_up, uint32_t type_down,
                             const int* top_idx, const float* top_w, const float* down_scale,
                             int n_tokens, int top_k, int n_experts_total, int hidden, int inter, int activation,
                             float* out, float* h_out, void* stream);

/* The reference's expert selection (src/arch_gemma4.cpp:547-565) for a batch of tokens, on the device, operation
 * for operation: softmax over logits [n_tokens][n_experts] (maximum, exponentials summed in index order, division),
 * top_k times the largest remaining probability (the lowest index wins among equal values), the selected
 * probabilities divided by their sum. Writes top_idx / top_w [n_tokens][top_k] in selection order - the form
 * laplace_cuda_moe_ffn_dev takes. The router's own matmul (logits = W_router . x) is an ordinary
 * laplace_cuda_gemm_dev call for quantized router weights. Device pointers. */
int laplace_cuda_moe_route_dev(const float* logits, int n_tokens, int n_experts, int top_k,
                               int* top_idx, float* top_w, void* stream);

/* Exchange helpers of an expert-parallel MoE layer (no reference counterpart): one all-gather moves
 * [x (hidden floats) | expert ids (top_k ints, bit pattern) | weights (top_k floats)] per token.
 * pack builds this GPU's rows, [n_tokens][hidden + 2*top_k]; unpack splits gathered rows into
 * x [n_tokens][hidden], top_w [n_tokens][top_k] and idx_local [n_tokens][top_k], where a global
 * expert id e becomes e - expert_first if it lies in [expert_first, expert_first + expert_count)
 * and -1 otherwise (the form laplace_cuda_moe_ffn_dev takes). Device pointers. */
int laplace_cuda_moe_pack_dev(const float* x, const int* top_idx, const float* top_w,
                              int n_tokens, int hidden, int top_k, float* packed, void* stream);
int laplace_cuda_moe_unpack_dev(const float* packed, int n_tokens, int hidden, int top_k,
                                int expert_first, int expert_count,
                                float* x, int* idx_local, float* top_w, void* stream);

/* Prefill GEMM (M > 8, K % 256 == 0; Q4_0, Q8_0, Q4_K, Q6_K) that allocates nothing. It has no counterpart in
 * the reference: it exists for hosts that must not touch the CUDA allocator on the request
 * path - serving processes whose own pools (KV cache, activations) already hold all HBM, so
 * that cudaMalloc would fail or fragment them, and latency-bound loops that cannot take the
 * allocator's locks or the implicit device synchronisation of cudaFree. Same arguments as
 * laplace_cuda_gemm_dev and the same result (bit-identical whenever the call fits the array with the same
 * K-split that entry point would choose, else equal to fp32 rounding); the quantized activations go to a
 * 10 MiB array built into the library (held by every GPU that loads it) instead of a cudaMalloc'd buffer.
 *   - LAPLACE_ERR_LIMIT when the call needs more scratch than the array holds: about
 *     4.13 * pad128(M) * K bytes (M = 512, K = 4096: 8.3 MiB), plus the partial sums of a K-split when they fit;
 *     LAPLACE_ERR_ARG for shapes that are not the prefill case (decode calls use no scratch).
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress); make
 *     that call before any stream capture begins.
 *   - All calls share the one array and it keeps the last call's contents (what must start
 *     from zero is cleared by each call): two calls that overlap on the GPU - different
 *     streams, or the same stream with programmatic overlap - race. Serialise them. */
int laplace_cuda_gemm_noalloc_dev(const float* x, const uint8_t* w, uint32_t type,
                                  float* y, int M, int K, int N, void* stream);

/* ---- weight types without an int8 kernel, dequantize(), LM head ---------------------------
 * laplace_cuda_gemm and laplace_cuda_gemm_dev also take F32 (0), F16 (1), BF16 (30), Q2_K (10), Q3_K (11) and
 * Q5_K (13) weights. For those the reference has no int8 kernel and computes
 * y[m][j] = dot_row_<type>(x[m], row j) with fp32 activations (gemm_fallback, src/matmul.cpp:336-352); so does the
 * library (activations are NOT quantized for these types). K must be a multiple of the type's block (16 for the
 * plain types).
 *
 * laplace_cuda_dequantize_dev replaces dequantize(const Tensor&, float* dst, int n) (src/matmul.cpp:504-675) for
 * every type above plus Q4_0 / Q5_0 / Q8_0 / Q4_K / Q6_K, bit for bit (the reference's expressions, separate roundings);
 * n = number of values, a multiple of the block size. laplace_cuda_embed_rows_dev is the token-embedding lookup of
 * src/model.cpp:366-378: dst[m] = dequantize(row tokens[m]) * scale (scale = the model's embedding scale, 1 for most);
 * a token id outside [0, vocab) is reported through laplace_cuda_sync like a bad expert index.
 * laplace_cuda_lm_head_dev replaces matmul_lm_head (src/matmul.cpp:439-444) followed by the optional logit
 * soft-cap of src/model.cpp:399-406 (softcap > 0: y = tanh(y / softcap) * softcap). */
int laplace_cuda_dequantize_dev(const uint8_t* w, uint32_t type, float* dst, long long n, void* stream);
int laplace_cuda_embed_rows_dev(const uint8_t* w, uint32_t type, const int* tokens, int M, int H, long long vocab, float scale,
                                float* dst, void* stream);
int laplace_cuda_lm_head_dev(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, float softcap,
                             void* stream);

/* ---- row-split prefill: the GEMM stores into every GPU's buffer --------------------------
 * laplace_cuda_gemm_peers_dev is laplace_cuda_gemm_dev for M > 8 over a weight matrix split along N: this GPU's
 * n_local columns of y go, from the kernel's own drain, to every GPU's row-major [M][n_total] buffer at column
 * row_begin (plain stores to peer-mapped memory allocated with laplace_cuda_peer_alloc; no collective, no copy
 * afterwards). LAPLACE_UNSUPPORTED for shapes the tensor-core kernels do not take (M <= 8, K not a multiple of 256).
 * The stores are complete when the call's kernels are; laplace_cuda_allgather_step_wait_dev, enqueued next, advances
 * this GPU's step counter, announces the step to every GPU and waits (bounded) until every GPU has announced it:
 * after it, all slices are in this GPU's buffer. Every gemm_peers call must be followed by that call before its
 * buffers are read or written again on any GPU. */
int laplace_cuda_gemm_peers_dev(const float* x, const uint8_t* w, uint32_t type, float* const* peer_y, int world,
                                int row_begin, int n_total, int M, int K, int n_local, void* stream);
int laplace_cuda_allgather_step_wait_dev(int* const* peer_flags, int* step_counter, int rank, int world, void* stream);

/* ---- GGUF file -> HBM ------------------------------------------------------------------
 * Replaces, for a GPU box, what GGUFContext::open (src/gguf.cpp:217-335) plus matmul_register_weights
 * (src/matmul.h:26, src/main.cpp:705) do on the host: the file is mapped and its header, metadata and tensor
 * table are parsed (GGUF v2 / v3); laplace_cuda_gguf_upload then copies, straight from the mapping, the part of
 * every tensor that rank `rank` of `world` GPUs works on:
 *   kind 2  stacked expert tensors (3 dims and more, dims = [K, rows, experts]): whole experts,
 *           expert e on GPU e / ceil(experts / world)
 *   kind 1  matrices (2 dims, at least 256 rows): the rows of laplace_cuda_nsplit(rows, rank, world)
 *   kind 0  everything else, and every tensor named in `replicate` (e.g. the token embedding, which is read
 *           by row index): the whole tensor
 * Blocks keep the on-disk format, which is the matmul kernels' wire format (src/tensor.h:130-163). Opening and
 * the tensor / metadata queries need no GPU; the upload needs laplace_cuda_init. The handle owns the mapping
 * and one device allocation; `dev` pointers stay valid until laplace_cuda_gguf_close. */
typedef struct laplace_cuda_gguf laplace_cuda_gguf;
typedef struct {
    const char*        name;
    uint32_t           type;             /* ggml type id */
    uint32_t           n_dims;
    unsigned long long dims[4];          /* innermost first, as in the file; unused dims are 1 */
    int                kind;             /* 0 whole tensor, 1 rows [row_begin, row_end), 2 experts [expert_begin, expert_end) */
    unsigned long long row_begin, row_end;
    unsigned long long expert_begin, expert_end;
    unsigned long long file_offset;      /* of this rank's part */
    unsigned long long bytes;            /* of this rank's part */
    const void*        host;             /* the part inside the mapping */
    void*              dev;              /* the part in HBM; NULL before laplace_cuda_gguf_upload */
} laplace_cuda_gguf_tensor_info;
int  laplace_cuda_gguf_open(const char* path, int rank, int world, const char* const* replicate, int n_replicate,
                            laplace_cuda_gguf** out);
int  laplace_cuda_gguf_upload(laplace_cuda_gguf* g);
int  laplace_cuda_gguf_tensor_count(const laplace_cuda_gguf* g);
/* By name when `name` is not NULL (LAPLACE_UNSUPPORTED = 1 when the file has no such tensor), else by index. */
int  laplace_cuda_gguf_tensor(const laplace_cuda_gguf* g, int index, const char* name, laplace_cuda_gguf_tensor_info* info);
/* Scalar metadata (general.alignment, llama.block_count, ...): 1 when the key is absent or of another kind. */
int  laplace_cuda_gguf_meta_u64(const laplace_cuda_gguf* g, const char* key, unsigned long long* value);
int  laplace_cuda_gguf_meta_f64(const laplace_cuda_gguf* g, const char* key, double* value);
const char* laplace_cuda_gguf_meta_str(const laplace_cuda_gguf* g, const char* key);
void laplace_cuda_gguf_close(laplace_cuda_gguf* g);

/* ---- fused all-gather for the row-split (tensor-parallel) decode matmul ---------------
 * No reference counterpart (the reference is single-device). With a weight matrix split
 * along N over `world` GPUs, every GPU's GEMV stores its slice of y straight into EVERY
 * GPU's full-width result buffer through peer-mapped pointers (coalesced NVLink stores from the
 * kernel's own epilogue, no fence on the kernel's critical path). A step's slices are announced
 * (flag [rank] of every GPU raised to the step number) by the NEXT gemm_allgather kernel's
 * prologue, or by laplace_cuda_allgather_wait_dev, which closes a chain of steps: it announces the
 * current step and waits (bounded) until all `world` flags of this GPU have reached it; the full y
 * of step s is then in slot (s & 3) of this GPU's buffer; consumers of y run after that call. A kernel
 * stores step s (over the slices of step s - 4) only after it has seen every GPU's flag at s - 3 or more: a
 * GPU raises its flag to s' - 1 when its step-s' kernel starts, i.e. when everything it enqueued before that
 * kernel - the readers of steps up to s' - 2 - has finished. Four slots keep that check off a step's critical
 * path. Replaces "GEMV + ncclAllGather" for decode, where the
 * collective's latency is 2-3x the kernel.
 *
 * Memory: each GPU allocates one buffer with laplace_cuda_peer_alloc (zeroed; returns a 64-byte
 * IPC handle to pass to the other processes by any host channel) and opens the others' with
 * laplace_cuda_peer_open. Layout is up to the caller; the calls take pointers:
 *   peer_y[r]     GPU r's result area, float [4][M][n_total]
 *   peer_flags[r] GPU r's flag array, int [world]
 *   step_counter  this GPU's int, done_counter this GPU's unsigned (both start at 0)
 * Steps are counted on the device, so the calls can be replayed from a CUDA graph. Every GPU must
 * issue the same sequence of steps. A wait that gives up (a peer never arrived) surfaces as
 * LAPLACE_ERR_TIMEOUT from laplace_cuda_sync(); nothing spins forever. M <= 8. */
int laplace_cuda_peer_alloc(size_t bytes, void** dev_ptr, unsigned char* handle64);
int laplace_cuda_peer_open(const unsigned char* handle64, void** dev_ptr);
int laplace_cuda_peer_close(void* dev_ptr);
int laplace_cuda_peer_free(void* dev_ptr);
int laplace_cuda_gemm_allgather_dev(const float* x, const uint8_t* w, uint32_t type,
                                    float* const* peer_y, int* const* peer_flags,
                                    int* step_counter, unsigned* done_counter,
                                    int rank, int world, int row_begin, int n_total,
                                    int M, int K, int n_local, void* stream);
int laplace_cuda_allgather_wait_dev(int* const* peer_flags, int* step_counter, int rank, int world, void* stream);

/* The activation quantizer on its own (src/matmul_simd.cpp:348-427).
 * Outputs, all device memory, M rows: q int8 [M][K]; d fp32 [M][K/32];
 * sum fp32 [M][K/32] (= d * (sum_lo + sum_hi)); isum int16 [M][K/32][2]
 * (sum_lo, sum_hi). Any output pointer may be NULL. */
int laplace_cuda_quantize_act_dev(const float* x, int M, int K,
                                  int8_t* q, float* d, float* sum, int16_t* isum,
                                  void* stream);

/* Exact integer block sums, for parity tests on small shapes:
 * out[(m*N+j)*per_row + b], per_row = K/32 (Q8_0, Q4_0, Q5_0, Q4_K) or K/16 (Q6_K);
 * same definition as the per-block accumulations of
 * src/matmul_simd.cpp:143-342. Device pointers. */
int laplace_cuda_debug_blocksums_dev(const float* x, const uint8_t* w, uint32_t type,
                                     int32_t* out, int M, int K, int N, void* stream);

/* Dense tensor-core rate of the bound GPU, measured with a bare tcgen05.mma loop on every SM (M = 128, N = 128
 * instructions from two issuing threads): kind 0 = fp16 operands / fp32 accumulate, 1 = int8 / int32. Result in
 * Tera-operations per second, 2 per multiply-add. For the benchmark's roofline; no reference counterpart.
 * Synchronous (a few milliseconds). */
int laplace_cuda_debug_tensor_peak(int kind, double* tops);

/* Which kernel family the last *_dev gemm call used: 1 = streaming dp4a GEMV,
 * 2 = tensor-core GEMM, 3 = expert-grouped tensor-core GEMM, 4 = fused expert FFN. For tests and the benchmark's launch count. */
int laplace_cuda_last_path(void);
/* Kernel launches issued by this library since the counter was last reset. */
long long laplace_cuda_launch_count(int reset);

#ifdef __cplusplus
}
#endif
#endif
