// lp_quantize.cu - the activation Q8 quantizer as a kernel of its own, and the
// integer block-sum kernel used by parity tests.
//
// quantize_act_kernel follows Laplace src/matmul_simd.cpp:348-427: per 32
// values, d = amax/127 (fp32), id = d > 0 ? 1/d : 0, q = rne(x * id) with a
// separate multiply, clamped to int8; sum_lo / sum_hi are the integer sums of
// the first / last 16 values before clamping; sum = d * (sum_lo + sum_hi).
// The output is structure-of-arrays (the reference's 44-byte ActQ8 is an
// array of structures): q [M][K], d [M][K/32], sum [M][K/32], isum [M][K/32][2].
#include "lp_common.cuh"

namespace lp {

namespace {

__global__ void __launch_bounds__(256) quantize_act_kernel(const float* __restrict__ x, long long n_blocks,
                                                           int8_t* __restrict__ q, float* __restrict__ d,
                                                           float* __restrict__ sum, int16_t* __restrict__ isum) {
    const int t8 = threadIdx.x & 7;
    const long long groups = static_cast<long long>(gridDim.x) * (blockDim.x >> 3);
    const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x >> 3) + (threadIdx.x >> 3);
    // all lanes of a warp run the same number of iterations (shuffles inside)
    const long long iters = (n_blocks + groups - 1) / groups;
    for (long long it = 0; it < iters; ++it) {
        const long long b = first + it * groups;
        const bool live = b < n_blocks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = __ldg(reinterpret_cast<const float4*>(x + b * 32) + t8);
        uint32_t packed; int hs;
        const float dv = quantize_block_8lanes(v, packed, hs);
        const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
        if (!live) continue;
        if (q) reinterpret_cast<uint32_t*>(q + b * 32)[t8] = packed;
        if (t8 == 0) {
            const short lo = static_cast<short>(hs), hi = static_cast<short>(hs_hi);
            if (d) d[b] = dv;
            if (sum) sum[b] = dv * static_cast<float>(static_cast<int>(lo) + static_cast<int>(hi));
            if (isum) { isum[2 * b] = lo; isum[2 * b + 1] = hi; }
        }
    }
}

// Integer weight value of element k of a row, written straight from the block
// layouts (Laplace src/kernels.h:21-54, src/matmul.cpp:84-198) without any of
// the word-level unpacking the fast kernels use. Q4_0 / Q4_K give the unsigned
// nibble, Q8_0 the signed byte, Q5_0 the 5-bit value minus 16, Q6_K the 6-bit
// value minus 32.
__device__ int weight_value(uint32_t type, const uint8_t* row, int k) {
    switch (type) {
        case LAPLACE_TYPE_Q4_0: {
            const uint8_t* blk = row + (k >> 5) * Q4_0_BYTES;
            const int l = k & 31;
            const int byte = blk[2 + (l & 15)];
            return l < 16 ? (byte & 15) : (byte >> 4);
        }
        case LAPLACE_TYPE_Q5_0: {
            const uint8_t* blk = row + (k >> 5) * Q5_0_BYTES;
            const int l = k & 31;
            const int byte = blk[6 + (l & 15)];
            const int bit = (blk[2 + (l >> 3)] >> (l & 7)) & 1;           // qh is little-endian: bit l of the 32
            return ((l < 16 ? (byte & 15) : (byte >> 4)) | (bit << 4)) - 16;
        }
        case LAPLACE_TYPE_Q8_0: {
            const uint8_t* blk = row + (k >> 5) * Q8_0_BYTES;
            return static_cast<int8_t>(blk[2 + (k & 31)]);
        }
        case LAPLACE_TYPE_Q4_K: {
            const uint8_t* blk = row + (k >> 8) * Q4_K_BYTES;
            const int e = k & 255, c = e >> 6, r = e & 63;
            const int byte = blk[16 + 32 * c + (r & 31)];
            return r < 32 ? (byte & 15) : (byte >> 4);
        }
        default: {  // Q6_K
            const uint8_t* blk = row + (k >> 8) * Q6_K_BYTES;
            const int e = k & 255, half = e >> 7, r = e & 127, g = r >> 5, l = r & 31;
            const int ql = blk[64 * half + 32 * (g & 1) + l];
            const int nib = g >= 2 ? (ql >> 4) : (ql & 15);
            const int top = (blk[128 + 32 * half + l] >> (2 * g)) & 3;
            return (nib | (top << 4)) - 32;
        }
    }
}

// One thread per (m, j, 32-value block).
__global__ void blocksum_kernel(const int8_t* __restrict__ q, const uint8_t* __restrict__ w, uint32_t type,
                                int32_t* __restrict__ out, int M, int K, int N, size_t rb) {
    const int bpr = K >> 5;
    const long long total = static_cast<long long>(M) * N * bpr;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int b = static_cast<int>(idx % bpr);
    const long long mj = idx / bpr;
    const int j = static_cast<int>(mj % N), m = static_cast<int>(mj / N);
    const uint8_t* row = w + static_cast<size_t>(j) * rb;
    const int8_t* xq = q + static_cast<size_t>(m) * K + b * 32;
    int s0 = 0, s1 = 0;
    for (int l = 0; l < 16; ++l) s0 += weight_value(type, row, b * 32 + l) * xq[l];
    for (int l = 16; l < 32; ++l) s1 += weight_value(type, row, b * 32 + l) * xq[l];
    if (type == LAPLACE_TYPE_Q6_K) {
        out[mj * (2 * bpr) + 2 * b] = s0;
        out[mj * (2 * bpr) + 2 * b + 1] = s1;
    } else {
        out[mj * bpr + b] = s0 + s1;
    }
}

}  // namespace

int launch_quantize_act(const float* x, int M, int K, int8_t* q, float* d, float* sum, int16_t* isum,
                        cudaStream_t st) {
    Context& c = ctx();
    if (M <= 0 || K <= 0 || (K & 31)) return fail(LAPLACE_ERR_ARG, "quantize: M=%d K=%d (K must be a multiple of 32)", M, K);
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(LAPLACE_ERR_ARG, "quantize: x not 16-byte aligned");
    const long long n_blocks = static_cast<long long>(M) * (K / 32);
    long long want = (n_blocks + 31) / 32;                       // 32 blocks per 256-thread CTA per pass
    const long long cap = static_cast<long long>(c.sm_count) * 8;
    const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
    quantize_act_kernel<<<grid, 256, 0, st>>>(x, n_blocks, q, d, sum, isum);
    c.launches++;
    return cuda_check(cudaGetLastError(), "quantize_act launch");
}

// Needs a scratch int8 buffer for the quantized activations; the caller passes it.
int launch_blocksums_q(const int8_t* q, const uint8_t* w, uint32_t type, int32_t* out, int M, int K, int N,
                       cudaStream_t st) {
    Context& c = ctx();
    const long long total = static_cast<long long>(M) * N * (K / 32);
    const long long grid = (total + 255) / 256;
    if (grid > 0x7fffffffLL) return fail(LAPLACE_ERR_LIMIT, "blocksums: problem too large for the debug kernel");
    blocksum_kernel<<<static_cast<int>(grid), 256, 0, st>>>(q, w, type, out, M, K, N, row_bytes(type, K));
    c.launches++;
    return cuda_check(cudaGetLastError(), "blocksum launch");
}

}  // namespace lp
