// lp_common.cuh - shared declarations of the sm_100a back-end.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "laplace_cuda.h"

namespace lp {

// ---- block geometry (Laplace src/kernels.h:21-54, src/tensor.h:41-100) ------
constexpr int Q4_0_BYTES = 18;
constexpr int Q5_0_BYTES = 22;
constexpr int Q8_0_BYTES = 34;
constexpr int Q4_K_BYTES = 144;
constexpr int Q6_K_BYTES = 210;

__host__ __device__ inline int block_elems(uint32_t type) {
    switch (type) {
        case LAPLACE_TYPE_Q4_0: case LAPLACE_TYPE_Q5_0: case LAPLACE_TYPE_Q8_0: return 32;
        case LAPLACE_TYPE_Q4_K: case LAPLACE_TYPE_Q6_K: return 256;
        default: return 0;
    }
}
__host__ __device__ inline int block_bytes(uint32_t type) {
    switch (type) {
        case LAPLACE_TYPE_Q4_0: return Q4_0_BYTES;
        case LAPLACE_TYPE_Q5_0: return Q5_0_BYTES;
        case LAPLACE_TYPE_Q8_0: return Q8_0_BYTES;
        case LAPLACE_TYPE_Q4_K: return Q4_K_BYTES;
        case LAPLACE_TYPE_Q6_K: return Q6_K_BYTES;
        default: return 0;
    }
}
inline size_t row_bytes(uint32_t type, int K) {
    return static_cast<size_t>(K / block_elems(type)) * block_bytes(type);
}

// ---- host-side state shared by the translation units -----------------------
struct Context {
    bool         ready = false;
    int          device = -1;
    int          sm_count = 0;
    size_t       smem_optin = 0;       // largest dynamic shared memory one CTA may ask for
    size_t       smem_per_sm = 0;      // shared memory of one SM
    cudaStream_t stream = nullptr;
    int*         d_err = nullptr;      // device view of the status word, 0 = fine
    int*         h_err = nullptr;      // host view of the same word (mapped pinned memory)
    int          last_path = 0;
    long long    launches = 0;
};
Context& ctx();
int  fail(int code, const char* fmt, ...);   // records the message, returns code
int  cuda_check(cudaError_t e, const char* what);

// Device status codes written to Context::d_err by bounded waits.
enum : int { DEV_OK = 0, DEV_TIMEOUT_FULL = 1, DEV_TIMEOUT_EMPTY = 2, DEV_TIMEOUT_DRAIN = 3,
             DEV_TIMEOUT_MMA = 4, DEV_TIMEOUT_TMEM = 5, DEV_BAD_INDEX = 6, DEV_TIMEOUT_PEER = 7 };

// ---- kernel launchers (one per .cu) ----------------------------------------
struct GemvArgs {
    const float*   x;            // fp32 activations, device
    const uint8_t* w;            // weights, device
    float*         y;            // output, device
    const int*     expert_idx;   // device, or nullptr for a plain matrix
    uint32_t       type;
    int            M;            // activation rows applied to every weight row (1..8)
    int            K, N;
    int            n_seg;        // 1, or the number of selected experts
    int            per_seg_x;    // 0: all segments read rows [0,M); 1: segment s reads row s (M == 1)
    const struct PeerOut* peers; // nullptr, or: results go to every GPU's buffer instead of y (fused all-gather)
    // several matrices of the same type and K that share x (w, y, N above are then unused)
    int            n_mats;
    const uint8_t* const* mat_w;
    float* const*  mat_y;
    const int*     mat_n;
    // optional RMSNorm of x in front of the quantizer: x_norm = x * inv_rms * norm_w
    const float*   norm_w;
    float          norm_eps;
    float*         x_norm_out;
};
// Fused all-gather of a row-split matmul: every GPU stores its slice of the result straight into
// every GPU's full-width buffer through peer-mapped pointers, then raises a per-source step flag.
constexpr int MAX_PEERS = 8;
struct PeerOut {
    float*    y[MAX_PEERS];      // every GPU's result buffer: [4 slots][M][ld], slot = step & 3
    int*      flags[MAX_PEERS];  // every GPU's flag array [world]; GPU r writes entry r of each
    int*      step_ctr;          // this GPU's step counter; nullptr = no step protocol at all: the results are only
                                 // staged and written, coalesced, to y[0] (used for output in host-mapped memory)
    unsigned* done_ctr;          // this GPU's "CTAs that have read the step counter" count (zero between launches)
    int       world, rank;
    int       ld;                // columns of the full result (N of the whole matrix)
    int       col0;              // first column of this GPU's slice
};
int launch_gemv_stream(const GemvArgs& a, cudaStream_t st);
int launch_gemv_mma_q4k(const float* x, const uint8_t* w, float* y, int M, int K, int N, cudaStream_t st);
// weight types served with fp32 activations (the reference's scalar path), dequantize() and friends (lp_types.cu)
bool   f32act_type(uint32_t type);
bool   dequant_type(uint32_t type);
size_t any_row_bytes(uint32_t type, long long K);
int    any_block_elems(uint32_t type);
int launch_gemm_f32act(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, cudaStream_t st);
int launch_dequantize(const uint8_t* w, uint32_t type, float* dst, long long n, float scale, cudaStream_t st);
int launch_embed_rows(const uint8_t* w, uint32_t type, const int* tokens, int M, int H, long long vocab, float scale, float* dst,
                      cudaStream_t st);
int launch_softcap(float* y, long long n, float cap, cudaStream_t st);
int launch_allgather_wait(const PeerOut& po, cudaStream_t st, bool advance = false);
int launch_gemm_sa_multi(const float* x, const float* norm_w, float eps, float* x_norm_out, const uint8_t* const* ws, float* const* ys,
                         const int* ns, int n_mats, uint32_t type, int M, int K, cudaStream_t st);
int launch_gemm_sa_peers(const float* x, const uint8_t* w, uint32_t type, const PeerOut& po, int M, int K, int N, cudaStream_t st);

// Tensor-core prefill GEMM with the activation scales folded into the operand (lp_gemm_sa.cu): Q4_0, Q8_0, Q4_K, Q6_K
// with M > 8 and K % 256 == 0. Uses library-owned scratch for the quantized activations, or the caller's.
bool gemm_sa_supports(uint32_t type, int M, int K, int N);
int  launch_gemm_sa(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, cudaStream_t st);
int  launch_gemm_sa_prealloc(uint8_t* scratch, size_t cap, const float* x, const uint8_t* w, uint32_t type, float* y,
                             int M, int K, int N, cudaStream_t st);
void release_gemm_sa_scratch();
// Expert-grouped matmul over (token, expert) pairs and the fused expert FFN (gate/up matmul, gated activation, down
// matmul, weighted sum) for a batch of tokens, on the same kernels.
bool moe_sa_supports(uint32_t type, int K, int N);
int  launch_moe_grouped_sa(const float* x, const uint8_t* w, uint32_t type, const int* pair_expert, const int* pair_row,
                           int P, int E, float* y, int K, int N, cudaStream_t st);
int  launch_moe_ffn_sa(const float* x, const uint8_t* w_gate_up, const uint8_t* w_down, uint32_t type_gu, uint32_t type_dn,
                       const int* top_idx, const float* top_w, const float* down_scale, int T, int top_k, int E, int H, int I,
                       int activation, float* out, float* h_out, cudaStream_t st);
int  launch_moe_route(const float* logits, int T, int E, int top_k, int* top_idx, float* top_w, cudaStream_t st);
void release_moe_sa_scratch();
int  launch_moe_pack(const float* x, const int* idx, const float* wts, int T, int H, int k, float* packed, cudaStream_t st);
int  launch_moe_unpack(const float* packed, int T, int H, int k, int first, int count, float* x, int* idx_local, float* wts,
                       cudaStream_t st);

int launch_quantize_act(const float* x, int M, int K, int8_t* q, float* d, float* sum,
                        int16_t* isum, cudaStream_t st);
int launch_blocksums_q(const int8_t* q, const uint8_t* w, uint32_t type, int32_t* out,
                       int M, int K, int N, cudaStream_t st);

// ---- device helpers ---------------------------------------------------------
#ifdef __CUDACC__

// Records a device-side failure in the status word (host-mapped memory).
__device__ __forceinline__ void report_status(int* err, int code) {
    *reinterpret_cast<volatile int*>(err) = code;
    __threadfence_system();
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// unsigned bytes (weights) x signed bytes (activations)
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int r;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// NaN-propagating maximum, like the FMAX the reference's quantizer uses.
__device__ __forceinline__ float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xffffu)));
}

// Quantizes four consecutive activations that belong to one 32-value block
// whose scale inverse is `id`: separate multiply, round to nearest even,
// clamp to int8 (Laplace src/matmul_simd.cpp:374-407). Returns the packed
// bytes and adds the unclamped integers to `isum`.
__device__ __forceinline__ uint32_t quantize4(float4 v, float id, int& isum) {
    int q0 = __float2int_rn(__fmul_rn(v.x, id));
    int q1 = __float2int_rn(__fmul_rn(v.y, id));
    int q2 = __float2int_rn(__fmul_rn(v.z, id));
    int q3 = __float2int_rn(__fmul_rn(v.w, id));
    isum += q0 + q1 + q2 + q3;
    q0 = max(-128, min(127, q0));
    q1 = max(-128, min(127, q1));
    q2 = max(-128, min(127, q2));
    q3 = max(-128, min(127, q3));
    return (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | (static_cast<uint32_t>(q3 & 0xff) << 24);
}

// One 32-value activation block handled by 8 adjacent lanes (lane t holds
// values 4t..4t+3). Every lane returns the block's scale d; `packed` gets the
// lane's four int8; lanes 0 and 4 of the group get the two 16-value integer
// sums in `half_sum` (the other lanes hold partial values).
__device__ __forceinline__ float quantize_block_8lanes(float4 v, uint32_t& packed, int& half_sum) {
    float amax = max_nan(max_nan(fabsf(v.x), fabsf(v.y)), max_nan(fabsf(v.z), fabsf(v.w)));
    amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d  = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int s = 0;
    packed = quantize4(v, id, s);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    half_sum = s;
    return d;
}

// ---- mbarrier / bulk-copy wrappers (all waits are bounded) ------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(200u) /* suspend-time hint, ns */ : "memory");
    return ok != 0;
}
// Same without a suspend-time hint: for hand-offs on a critical path, where the wake-up
// must follow the phase completion at once.
__device__ __forceinline__ bool mbar_try_wait_nohint(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Returns false when the wait gave up (a second or so of polling). After the
// first miss the warp backs off between polls so that it does not take issue
// slots from warps that have data.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        __nanosleep(40);
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Plain (non-tensor, single-CTA) bulk copy global -> this CTA's shared memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int lds_s8(uint32_t addr) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// 16 bytes from a shared address that is only 2-byte aligned: five aligned
// words, funnel-shifted. Reads up to 4 bytes past the 16 (callers keep slack).
__device__ __forceinline__ void lds16B_align2(uint32_t addr, uint32_t (&out)[4]) {
    const uint32_t base = addr & ~3u;
    const uint32_t sh   = (addr & 3u) * 8u;
    uint32_t w0 = lds32(base), w1 = lds32(base + 4), w2 = lds32(base + 8), w3 = lds32(base + 12),
             w4 = lds32(base + 16);
    out[0] = __funnelshift_r(w0, w1, sh);
    out[1] = __funnelshift_r(w1, w2, sh);
    out[2] = __funnelshift_r(w2, w3, sh);
    out[3] = __funnelshift_r(w3, w4, sh);
}

#endif  // __CUDACC__

}  // namespace lp
