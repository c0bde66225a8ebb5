// lp_types.cu - the weight types that have no int8 kernel in the reference, and dequantize() on the device.
//
// Laplace serves Q4_0 / Q5_0 / Q8_0 / Q4_K / Q6_K matmuls through its int8 back-end and everything else -
// F32, F16, BF16, Q2_K, Q3_K, Q5_K - through the scalar path with fp32 activations
// (gemm_fallback, src/matmul.cpp:336-352: y[m][j] = dot_row_<type>(x[m], row j)). dequantize() (src/matmul.cpp:504-675)
// turns blocks into floats for token-embedding lookups (src/model.cpp:366-378). Here:
//   dequantize_kernel        every type, 16 values per thread, the reference's expressions with separate roundings
//                            (d * sc * q - dmin * m and the like), so the result is bit-identical to dequantize()
//   embed_rows_kernel        rows tokens[m] of the embedding table, times the model's embedding scale
//   gemv_f32act_kernel       fp32 activations against on-the-fly dequantized rows: one warp per weight row; plain
//                            rows stream at 5 TB/s and more (an F16 LM head of 32,000 rows: 48 us), K-quant rows at
//                            0.7-1.2 TB/s (bound by instruction issue) - these types carry embeddings, LM
//                            heads and the odd tensor of a mixed-precision file, not the bulk of the weights
//   softcap_kernel           logits = tanh(logits / cap) * cap (src/model.cpp:399-406)
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "lp_common.cuh"

namespace lp {
namespace {

constexpr uint32_t T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q5_0 = 6, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12,
                   T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30;

struct Geo { int elems, bytes; };       // per block; plain types are handled as "blocks" of 16 values
__host__ __device__ constexpr Geo geo_of(uint32_t t) {
    switch (t) {
        case T_F32: return {16, 64};
        case T_F16: case T_BF16: return {16, 32};
        case T_Q4_0: return {32, 18};
        case T_Q5_0: return {32, 22};
        case T_Q8_0: return {32, 34};
        case T_Q2_K: return {256, 84};
        case T_Q3_K: return {256, 110};
        case T_Q4_K: return {256, 144};
        case T_Q5_K: return {256, 176};
        case T_Q6_K: return {256, 210};
        default: return {0, 0};
    }
}

__device__ __forceinline__ float h16(const uint8_t* p) {       // fp16 at a 2-byte aligned address
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
}
// 6-bit (scale, min) pair j of a Q4_K / Q5_K block (Laplace src/kernels.h:82-90)
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& mn) {
    if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// Values 16 g .. 16 g + 15 of one block, in the order dequantize() writes them.
__device__ __forceinline__ void decode16(uint32_t type, const uint8_t* __restrict__ b, int g, float (&v)[16]) {
    switch (type) {
        case T_F32: {
            const float4* p = reinterpret_cast<const float4*>(b);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float4 t = __ldg(p + i); v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w; }
            break;
        }
        case T_F16: case T_BF16: {
            // 32 bytes; two 16-byte loads when the group is 16-byte aligned (rows of K % 16 == 0 values at an aligned base)
            uint32_t wds[8];
            if ((reinterpret_cast<uintptr_t>(b) & 15) == 0) {
                const uint4 a = __ldg(reinterpret_cast<const uint4*>(b)), c = __ldg(reinterpret_cast<const uint4*>(b) + 1);
                wds[0] = a.x; wds[1] = a.y; wds[2] = a.z; wds[3] = a.w; wds[4] = c.x; wds[5] = c.y; wds[6] = c.z; wds[7] = c.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    wds[i] = static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(b + 4 * i)) |
                             (static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(b + 4 * i + 2)) << 16);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (type == T_F16) {
                    v[2 * i] = __half2float(__ushort_as_half(static_cast<unsigned short>(wds[i] & 0xffffu)));
                    v[2 * i + 1] = __half2float(__ushort_as_half(static_cast<unsigned short>(wds[i] >> 16)));
                } else {
                    v[2 * i] = __uint_as_float(wds[i] << 16);
                    v[2 * i + 1] = __uint_as_float(wds[i] & 0xffff0000u);
                }
            }
            break;
        }
        case T_Q4_0: {
            const float d = h16(b);
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                const int q = g ? (b[2 + l] >> 4) : (b[2 + l] & 0xF);
                v[l] = __fmul_rn(d, static_cast<float>(q - 8));
            }
            break;
        }
        case T_Q5_0: {
            const float d = h16(b);
            const uint32_t qh = static_cast<uint32_t>(b[2]) | (static_cast<uint32_t>(b[3]) << 8) | (static_cast<uint32_t>(b[4]) << 16) |
                                (static_cast<uint32_t>(b[5]) << 24);
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                const int nib = g ? (b[6 + l] >> 4) : (b[6 + l] & 0xF);
                const int q = nib | (((qh >> (l + 16 * g)) & 1) << 4);
                v[l] = __fmul_rn(d, static_cast<float>(q - 16));
            }
            break;
        }
        case T_Q8_0: {
            const float d = h16(b);
#pragma unroll
            for (int l = 0; l < 16; ++l) v[l] = __fmul_rn(d, static_cast<float>(static_cast<int8_t>(b[2 + 16 * g + l])));
            break;
        }
        case T_Q2_K: {
            // scales[16], qs[64], d, dmin: value = d * (scale & 15) * q - dmin * (scale >> 4)
            const float d = h16(b + 80), dmin = h16(b + 82);
            const int half = g >> 3, jj = g & 7, grp = jj >> 1, lo = jj & 1;
            const float ds = __fmul_rn(d, static_cast<float>(b[g] & 0xF)), mm = __fmul_rn(dmin, static_cast<float>(b[g] >> 4));
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                const int q = (b[16 + half * 32 + lo * 16 + l] >> (grp * 2)) & 3;
                v[l] = __fsub_rn(__fmul_rn(ds, static_cast<float>(q)), mm);
            }
            break;
        }
        case T_Q3_K: {
            // hmask[32], qs[64], scales[12] (sixteen 6-bit values), d: value = d * (scale - 32) * (low2 - 4 + 4 * high bit)
            const float d = h16(b + 108);
            const uint8_t* s = b + 96;
            const int lo4 = g < 8 ? (s[g] & 0xF) : (s[g - 8] >> 4);
            const int hi2 = (s[8 + (g & 3)] >> (2 * (g >> 2))) & 3;
            const float ds = __fmul_rn(d, static_cast<float>((lo4 | (hi2 << 4)) - 32));
            const int g32 = g >> 1, li0 = 16 * (g & 1);
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                const int li = li0 + l;
                const int low2 = (b[32 + (g32 >> 2) * 32 + li] >> ((g32 & 3) * 2)) & 3;
                const int hbit = (b[li] >> g32) & 1;
                v[l] = __fmul_rn(ds, static_cast<float>(low2 - 4 + 4 * hbit));
            }
            break;
        }
        case T_Q4_K: case T_Q5_K: {
            // d, dmin, scales[12], (Q5_K: qh[32],) qs[128]: value = d * sc * q - dmin * m
            const float d = h16(b), dmin = h16(b + 2);
            const int jb = g >> 2, sub = (g >> 1) & 1, l0 = 16 * (g & 1);
            int sc, mn;
            scale_min_k4(2 * jb + sub, b + 4, sc, mn);
            const float ds = __fmul_rn(d, static_cast<float>(sc)), mm = __fmul_rn(dmin, static_cast<float>(mn));
            const uint8_t* qs = b + (type == T_Q5_K ? 48 : 16) + 32 * jb + l0;
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                int q = sub ? (qs[l] >> 4) : (qs[l] & 0xF);
                if (type == T_Q5_K) q += 16 * ((b[16 + l0 + l] >> (2 * jb + sub)) & 1);
                v[l] = __fsub_rn(__fmul_rn(ds, static_cast<float>(q)), mm);
            }
            break;
        }
        case T_Q6_K: {
            // ql[128], qh[64], int8 scales[16], d: value = d * scale * (q6 - 32)
            const float d = h16(b + 208);
            const int h = g >> 3, t = g & 7, qtr = t >> 1, l0 = 16 * (t & 1);
            const float ds = __fmul_rn(d, static_cast<float>(static_cast<int8_t>(b[192 + 8 * h + (t & 1) + 2 * qtr])));
            const uint8_t* ql = b + 64 * h + 32 * (qtr & 1) + l0;
            const uint8_t* qh = b + 128 + 32 * h + l0;
#pragma unroll
            for (int l = 0; l < 16; ++l) {
                const int nib = (qtr & 2) ? (ql[l] >> 4) : (ql[l] & 0xF);
                const int q = nib | (((qh[l] >> (2 * qtr)) & 3) << 4);
                v[l] = __fmul_rn(ds, static_cast<float>(q - 32));
            }
            break;
        }
        default:
#pragma unroll
            for (int l = 0; l < 16; ++l) v[l] = 0.f;
    }
}

__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ w, uint32_t type, float* __restrict__ dst,
                                                         long long n_groups, float scale) {
    const Geo geo = geo_of(type);
    const int gpb = geo.elems / 16;
    for (long long gi = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; gi < n_groups;
         gi += static_cast<long long>(gridDim.x) * blockDim.x) {
        float v[16];
        decode16(type, w + (gi / gpb) * geo.bytes, static_cast<int>(gi % gpb), v);
        float4* o = reinterpret_cast<float4*>(dst + gi * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            o[i] = scale == 1.0f ? make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3])
                                 : make_float4(v[4 * i] * scale, v[4 * i + 1] * scale, v[4 * i + 2] * scale, v[4 * i + 3] * scale);
    }
}

// dst[m] = dequantize(row tokens[m]) * scale; one block per token
__global__ void __launch_bounds__(256) embed_rows_kernel(const uint8_t* __restrict__ w, uint32_t type, const int* __restrict__ tokens,
                                                         int H, long long vocab, float scale, float* __restrict__ dst, int* err) {
    const Geo geo = geo_of(type);
    const int gpb = geo.elems / 16;
    const long long tok = tokens[blockIdx.x];
    if (tok < 0 || tok >= vocab) { if (threadIdx.x == 0) atomicCAS(err, DEV_OK, DEV_BAD_INDEX); return; }
    const uint8_t* row = w + tok * (static_cast<long long>(H / geo.elems) * geo.bytes);
    for (int gi = threadIdx.x; gi < H / 16; gi += blockDim.x) {
        float v[16];
        decode16(type, row + (gi / gpb) * geo.bytes, gi % gpb, v);
        float4* o = reinterpret_cast<float4*>(dst + static_cast<size_t>(blockIdx.x) * H + gi * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = make_float4(v[4 * i] * scale, v[4 * i + 1] * scale, v[4 * i + 2] * scale, v[4 * i + 3] * scale);
    }
}

// ---- K-quant blocks read from shared memory -------------------------------------------------------------------
// The fp32-activation GEMV stages each weight block at a 16-byte aligned shared address, so that a lane fetches
// the 16 quants of its group (and their high bits) with one 16-byte read each instead of 16 single-byte loads from
// global memory (which cost one L1 lookup per byte and held these types at 0.4-0.5 TB/s).
__device__ __forceinline__ uint4 lds_u4(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint32_t byte_of(const uint4& q, int l) {          // l is a compile-time constant after unrolling
    const uint32_t w = l < 4 ? q.x : l < 8 ? q.y : l < 12 ? q.z : q.w;
    return (w >> (8 * (l & 3))) & 0xFFu;
}
// The 16 quants of group g as floats (unscaled integers) plus the two factors of the group:
//   value_l = ds * q_l - mm        so        sum_l x_l * value_l = ds * (sum_l x_l q_l) - mm * (sum_l x_l).
// Four quants are cut out of a 32-bit word at a time (byte-parallel shifts and masks); the per-value work is one
// integer-to-float conversion and one FMA. Not the reference's rounding (it rounds ds * q - mm per value), which the
// fp32-activation matmul is not held to: its bar is 1e-5 relative L2 against the reference's result.
template <uint32_t TYPE>
__device__ __forceinline__ void quants16_staged(const uint8_t* __restrict__ b, int g, float (&qf)[16], float& ds, float& mm) {
    uint32_t q4[4];
    if constexpr (TYPE == T_Q5_K) {
        const uint4 head = lds_u4(b);                    // d, dmin, scales[12]
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(head.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(head.x >> 16)));
        const int jb = g >> 2, sub = (g >> 1) & 1, l0 = 16 * (g & 1), j = 2 * jb + sub;
        auto sbyte = [&](int i) { return ((i < 4 ? head.y : i < 8 ? head.z : head.w) >> (8 * (i & 3))) & 0xFFu; };
        int sc, mn;
        if (j < 4) { sc = sbyte(j) & 63; mn = sbyte(j + 4) & 63; }
        else { sc = (sbyte(j + 4) & 0xF) | ((sbyte(j - 4) >> 6) << 4); mn = (sbyte(j + 4) >> 4) | ((sbyte(j) >> 6) << 4); }
        ds = __fmul_rn(d, static_cast<float>(sc));
        mm = __fmul_rn(dmin, static_cast<float>(mn));
        const uint4 qs = lds_u4(b + 48 + 32 * jb + l0), qh = lds_u4(b + 16 + l0);
        const uint32_t qsw[4] = {qs.x, qs.y, qs.z, qs.w}, qhw[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
        for (int w = 0; w < 4; ++w)
            q4[w] = ((qsw[w] >> (4 * sub)) & 0x0f0f0f0fu) | (((qhw[w] >> j) & 0x01010101u) << 4);
    } else if constexpr (TYPE == T_Q2_K) {
        const uint32_t dd = *reinterpret_cast<const uint32_t*>(b + 80);
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(dd & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(dd >> 16)));
        const int half = g >> 3, jj = g & 7, grp = jj >> 1, lo = jj & 1;
        const uint32_t scb = b[g];
        ds = __fmul_rn(d, static_cast<float>(scb & 0xF));
        mm = __fmul_rn(dmin, static_cast<float>(scb >> 4));
        const uint4 qs = lds_u4(b + 16 + half * 32 + lo * 16);
        const uint32_t qsw[4] = {qs.x, qs.y, qs.z, qs.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) q4[w] = (qsw[w] >> (grp * 2)) & 0x03030303u;
    } else {                                             // Q3_K: value = ds * (low2 + 4 * hbit - 4)
        const uint4 tail = lds_u4(b + 96);               // scales[12], d
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(tail.w & 0xffffu)));
        auto sbyte = [&](int i) { return ((i < 4 ? tail.x : i < 8 ? tail.y : tail.z) >> (8 * (i & 3))) & 0xFFu; };
        const int lo4 = g < 8 ? (sbyte(g) & 0xF) : (sbyte(g - 8) >> 4);
        const int hi2 = (sbyte(8 + (g & 3)) >> (2 * (g >> 2))) & 3;
        ds = __fmul_rn(d, static_cast<float>((lo4 | (hi2 << 4)) - 32));
        mm = __fmul_rn(ds, 4.0f);
        const int g32 = g >> 1, li0 = 16 * (g & 1);
        const uint4 qs = lds_u4(b + 32 + (g32 >> 2) * 32 + li0), hm = lds_u4(b + li0);
        const uint32_t qsw[4] = {qs.x, qs.y, qs.z, qs.w}, hmw[4] = {hm.x, hm.y, hm.z, hm.w};
#pragma unroll
        for (int w = 0; w < 4; ++w)
            q4[w] = ((qsw[w] >> ((g32 & 3) * 2)) & 0x03030303u) | (((hmw[w] >> g32) & 0x01010101u) << 2);
    }
    // byte -> float without the conversion unit: 0x4B0000bb is the float 2^23 + bb
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        qf[4 * w]     = __uint_as_float(__byte_perm(q4[w], 0x4B000000u, 0x7440)) - 8388608.0f;
        qf[4 * w + 1] = __uint_as_float(__byte_perm(q4[w], 0x4B000000u, 0x7441)) - 8388608.0f;
        qf[4 * w + 2] = __uint_as_float(__byte_perm(q4[w], 0x4B000000u, 0x7442)) - 8388608.0f;
        qf[4 * w + 3] = __uint_as_float(__byte_perm(q4[w], 0x4B000000u, 0x7443)) - 8388608.0f;
    }
}

// x in shared memory: 16-byte piece f of a row sits at piece (f & ~3) | ((f & 3) ^ ((f >> 3) & 3)). A lane that owns 16
// consecutive values (4 pieces) reads piece i of every lane in one instruction; unswizzled, the lanes of a quarter warp
// would hit two 16-byte bank groups four times each.
__device__ __forceinline__ int x_piece(int f) { return (f & ~3) | ((f & 3) ^ ((f >> 3) & 3)); }

// y[m][j] = sum_k x[m][k] * dequantized(w[j][k]) for M <= 8 activation rows: a warp per weight row. The type is a
// template parameter (with it as a run-time argument the decoder's switch and the divisions by the groups per block sat
// inside the loop).
constexpr int F32ACT_WARPS = 8;
template <uint32_t TYPE> struct Stage {                   // staging of K-quant blocks: two blocks (512 values) per warp step
    static constexpr bool on = TYPE == T_Q2_K || TYPE == T_Q3_K || TYPE == T_Q5_K;
    static constexpr int bytes = geo_of(TYPE).bytes;
    static constexpr int pitch = (bytes + 15) & ~15;
    static constexpr int unit = TYPE == T_Q5_K ? 16 : TYPE == T_Q2_K ? 4 : 2;      // load width the block size allows
    static constexpr int units_per_block = bytes / unit;
    static constexpr int per_lane = (2 * units_per_block + 31) / 32;
    static constexpr int depth = 4;                                                // steps fetched back to back
    static constexpr int warp_bytes = on ? depth * 2 * pitch : 0;
};
template <int M, uint32_t TYPE>
__global__ void __launch_bounds__(256) gemv_f32act_kernel(const float* __restrict__ x, const uint8_t* __restrict__ w,
                                                          float* __restrict__ y, int K, int N, int x_in_smem) {
    extern __shared__ __align__(16) uint8_t f32act_smem[];
    using S = Stage<TYPE>;
    uint8_t* stage_base = f32act_smem;
    float* xs = reinterpret_cast<float*>(f32act_smem + F32ACT_WARPS * S::warp_bytes);
    constexpr Geo geo = geo_of(TYPE);
    constexpr int gpb = geo.elems / 16;
    const int groups = K / 16;
    const size_t rb = static_cast<size_t>(K / geo.elems) * geo.bytes;
    if (x_in_smem) {
        const int per_row = K / 4;
        for (int i = threadIdx.x; i < M * per_row; i += blockDim.x) {
            const int m = i / per_row, f = i - m * per_row;
            reinterpret_cast<float4*>(xs)[m * per_row + x_piece(f)] = __ldg(reinterpret_cast<const float4*>(x) + i);
        }
        __syncthreads();
        if constexpr (S::on) {
            // sum of x over every group of 16 values, once per CTA (the staged K-quant walk needs it per group and row)
            float* xsum = xs + static_cast<size_t>(M) * K;
            for (int i = threadIdx.x; i < M * groups; i += blockDim.x) {
                const int m = i / groups, gi = i - m * groups;
                const float4* base = reinterpret_cast<const float4*>(xs) + m * per_row;
                float t = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float4 v = base[x_piece(4 * gi + k)];
                    t += (v.x + v.y) + (v.z + v.w);
                }
                xsum[i] = t;
            }
            __syncthreads();
        }
    }
    const float* xa = x_in_smem ? xs : x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const bool plain_fast = (TYPE == T_F32 || TYPE == T_F16 || TYPE == T_BF16) &&
                            (reinterpret_cast<uintptr_t>(w) & (TYPE == T_F32 ? 15 : 7)) == 0;
    // staged K-quant walk: needs block addresses that are multiples of the load width
    const bool staged = S::on && (reinterpret_cast<uintptr_t>(w) & (S::unit - 1)) == 0;
    // the fp32 activations of group gi, piece i (values 16 gi + 4 i .. + 3) of row m
    auto x4 = [&](int m, int gi, int i) -> float4 {
        const float4* base = reinterpret_cast<const float4*>(xa + static_cast<size_t>(m) * K);
        return x_in_smem ? base[x_piece(4 * gi + i)] : __ldg(base + 4 * gi + i);
    };
    for (int j = blockIdx.x * wpb + warp; j < N; j += gridDim.x * wpb) {
        const uint8_t* row = w + static_cast<size_t>(j) * rb;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        if constexpr (TYPE == T_F32 || TYPE == T_F16 || TYPE == T_BF16) {
            // Plain rows: lane l takes values 128 i + 4 l .. + 3, so that a warp reads 128 consecutive values of
            // the row per step. Needs rows that start on an 8-byte (F32: 16-byte) boundary; row lengths are
            // multiples of 32 bytes.
            if (plain_fast) {
                using Wv = typename std::conditional<TYPE == T_F32, float4, uint2>::type;
                for (int k0 = lane * 4; k0 < K; k0 += 512) {
                    Wv t[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)                  // four loads in flight before the first use
                        if (k0 + 128 * u < K) t[u] = __ldg(reinterpret_cast<const Wv*>(row) + ((k0 + 128 * u) >> 2));
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int k = k0 + 128 * u;
                        if (k < K) {
                            float v0, v1, v2, v3;
                            if constexpr (TYPE == T_F32) {
                                v0 = t[u].x; v1 = t[u].y; v2 = t[u].z; v3 = t[u].w;
                            } else if constexpr (TYPE == T_F16) {
                                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t[u].x));
                                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t[u].y));
                                v0 = a.x; v1 = a.y; v2 = b.x; v3 = b.y;
                            } else {
                                v0 = __uint_as_float(t[u].x << 16); v1 = __uint_as_float(t[u].x & 0xffff0000u);
                                v2 = __uint_as_float(t[u].y << 16); v3 = __uint_as_float(t[u].y & 0xffff0000u);
                            }
#pragma unroll
                            for (int m = 0; m < M; ++m) {
                                const float4 xv = x4(m, k >> 4, (k >> 2) & 3);
                                acc[m] = fmaf(xv.w, v3, fmaf(xv.z, v2, fmaf(xv.y, v1, fmaf(xv.x, v0, acc[m]))));
                            }
                        }
                    }
                }
            }
        }
        if constexpr (S::on) {
            if (staged) {
                // Two blocks (512 values, one group of 16 per lane) per step: the warp copies them with coalesced
                // loads of the widest unit the block size allows into its staging area.
                uint8_t* st = stage_base + warp * S::warp_bytes;
                const int n_blocks = K / geo.elems, n_steps = (n_blocks + 1) / 2;
                auto fetch = [&](int step, uint32_t (&r)[S::per_lane][S::unit == 16 ? 4 : 1]) {
                    const int units = (n_blocks - 2 * step >= 2 ? 2 : 1) * S::units_per_block;
                    const uint8_t* src = row + static_cast<size_t>(2 * step) * S::bytes;
#pragma unroll
                    for (int t = 0; t < S::per_lane; ++t) {
                        const int u = lane + 32 * t;
                        if (u < units) {
                            if constexpr (S::unit == 16) {
                                const uint4 q = __ldg(reinterpret_cast<const uint4*>(src) + u);
                                r[t][0] = q.x; r[t][1] = q.y; r[t][2] = q.z; r[t][3] = q.w;
                            } else if constexpr (S::unit == 4) {
                                r[t][0] = __ldg(reinterpret_cast<const uint32_t*>(src) + u);
                            } else {
                                r[t][0] = __ldg(reinterpret_cast<const unsigned short*>(src) + u);
                            }
                        }
                    }
                };
                auto put = [&](int slot, int step, const uint32_t (&r)[S::per_lane][S::unit == 16 ? 4 : 1]) {
                    const int units = (n_blocks - 2 * step >= 2 ? 2 : 1) * S::units_per_block;
                    uint8_t* dst = st + slot * 2 * S::pitch;
#pragma unroll
                    for (int t = 0; t < S::per_lane; ++t) {
                        const int u = lane + 32 * t;
                        if (u < units) {
                            const int blk = u >= S::units_per_block ? 1 : 0;
                            uint8_t* at = dst + blk * S::pitch + (u - blk * S::units_per_block) * S::unit;
                            if constexpr (S::unit == 16) *reinterpret_cast<uint4*>(at) = make_uint4(r[t][0], r[t][1], r[t][2], r[t][3]);
                            else if constexpr (S::unit == 4) *reinterpret_cast<uint32_t*>(at) = r[t][0];
                            else *reinterpret_cast<unsigned short*>(at) = static_cast<unsigned short>(r[t][0]);
                        }
                    }
                };
                // DEPTH steps are fetched into registers back to back (loads in flight), staged, then decoded.
                constexpr int DEPTH = S::depth;
                for (int s0 = 0; s0 < n_steps; s0 += DEPTH) {
                    uint32_t regs[DEPTH][S::per_lane][S::unit == 16 ? 4 : 1];
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d)
                        if (s0 + d < n_steps) fetch(s0 + d, regs[d]);
                    __syncwarp();                               // every lane is done reading the previous batch
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d)
                        if (s0 + d < n_steps) put(d, s0 + d, regs[d]);
                    __syncwarp();                               // the batch is in shared memory
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d) {
                        const int gi = 32 * (s0 + d) + lane;
                        if (gi < groups) {
                            float qf[16], ds, mm;
                            quants16_staged<TYPE>(st + d * 2 * S::pitch + (lane >> 4) * S::pitch, lane & 15, qf, ds, mm);
#pragma unroll
                            for (int m = 0; m < M; ++m) {
                                float sq = 0.f, sx = 0.f;                 // sum x q and sum x over the group
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float4 t = x4(m, gi, i);
                                    sq = fmaf(t.x, qf[4 * i], sq); sq = fmaf(t.y, qf[4 * i + 1], sq);
                                    sq = fmaf(t.z, qf[4 * i + 2], sq); sq = fmaf(t.w, qf[4 * i + 3], sq);
                                    if (!x_in_smem) sx += (t.x + t.y) + (t.z + t.w);
                                }
                                if (x_in_smem) sx = xs[static_cast<size_t>(M) * K + m * groups + gi];
                                acc[m] = fmaf(ds, sq, fmaf(-mm, sx, acc[m]));
                            }
                        }
                    }
                }
            }
        }
#pragma unroll 2
        for (int gi = lane; gi < ((plain_fast || staged) ? 0 : groups); gi += 32) {
            float v[16];
            decode16(TYPE, row + (gi / gpb) * geo.bytes, gi % gpb, v);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 t = x4(m, gi, i);
                    s = fmaf(t.x, v[4 * i], s); s = fmaf(t.y, v[4 * i + 1], s); s = fmaf(t.z, v[4 * i + 2], s); s = fmaf(t.w, v[4 * i + 3], s);
                }
                acc[m] += s;
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float a = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0) y[static_cast<size_t>(m) * N + j] = a;
        }
    }
}

__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ y, long long n, float cap, float inv_cap) {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x)
        y[i] = __fmul_rn(tanhf(__fmul_rn(y[i], inv_cap)), cap);
}

template <int M, uint32_t TYPE>
cudaError_t launch_f32act_typed(const float* x, const uint8_t* w, float* y, int K, int N, cudaStream_t st) {
    const size_t xbytes = static_cast<size_t>(M) * K * sizeof(float);
    const int in_smem = xbytes <= 96 * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_f32act_kernel<M, TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int wpb = F32ACT_WARPS;
    long long blocks = (static_cast<long long>(N) + wpb - 1) / wpb;
    // One wave: as many CTAs as are resident at once (registers and the x copy in shared memory decide), each walking
    // rows at the grid's stride. A grid of 8 CTAs per SM where 6 fit ran a second, one-third-full wave.
    static size_t occ_for = ~size_t(0);
    static int occ = 1;
    const size_t dyn = (in_smem ? xbytes + (Stage<TYPE>::on ? xbytes / 16 : 0) : 0) + static_cast<size_t>(F32ACT_WARPS) * Stage<TYPE>::warp_bytes;
    if (occ_for != dyn) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_f32act_kernel<M, TYPE>, 256, dyn);
        if (e != cudaSuccess) return e;
        occ = n < 1 ? 1 : n;
        occ_for = dyn;
    }
    const long long cap = static_cast<long long>(ctx().sm_count) * occ;
    if (blocks > cap) blocks = cap;
    gemv_f32act_kernel<M, TYPE><<<static_cast<int>(blocks), 256, dyn, st>>>(x, w, y, K, N, in_smem);
    return cudaGetLastError();
}

template <int M>
cudaError_t launch_f32act(const float* x, const uint8_t* w, uint32_t type, float* y, int K, int N, cudaStream_t st) {
    switch (type) {
        case T_F32:  return launch_f32act_typed<M, T_F32>(x, w, y, K, N, st);
        case T_F16:  return launch_f32act_typed<M, T_F16>(x, w, y, K, N, st);
        case T_BF16: return launch_f32act_typed<M, T_BF16>(x, w, y, K, N, st);
        case T_Q2_K: return launch_f32act_typed<M, T_Q2_K>(x, w, y, K, N, st);
        case T_Q3_K: return launch_f32act_typed<M, T_Q3_K>(x, w, y, K, N, st);
        case T_Q5_K: return launch_f32act_typed<M, T_Q5_K>(x, w, y, K, N, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

bool f32act_type(uint32_t type) {
    return type == T_F32 || type == T_F16 || type == T_BF16 || type == T_Q2_K || type == T_Q3_K || type == T_Q5_K;
}
bool dequant_type(uint32_t type) { return geo_of(type).elems != 0; }
size_t any_row_bytes(uint32_t type, long long K) {
    const Geo g = geo_of(type);
    return g.elems ? static_cast<size_t>(K / g.elems) * g.bytes : 0;
}
int any_block_elems(uint32_t type) {
    const Geo g = geo_of(type);
    return (type == T_F32 || type == T_F16 || type == T_BF16) ? 16 : g.elems;
}

int launch_gemm_f32act(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, cudaStream_t st) {
    if (!f32act_type(type)) return LAPLACE_UNSUPPORTED;
    const Geo g = geo_of(type);
    if (K % g.elems) {
        if (type == T_F32 || type == T_F16 || type == T_BF16) return LAPLACE_UNSUPPORTED;      // rows are walked 16 values at a time
        return fail(LAPLACE_ERR_ARG, "gemm: K=%d is not a multiple of %d for type %u", K, g.elems, type);
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & (type == T_F32 ? 15 : 1)))
        return fail(LAPLACE_ERR_ARG, "gemm: x must be 16-byte aligned, weights 2-byte (F32: 16-byte) aligned");
    Context& c = ctx();
    for (int m0 = 0; m0 < M; m0 += 8) {
        const int mm = M - m0 < 8 ? M - m0 : 8;
        const float* xp = x + static_cast<size_t>(m0) * K;
        float* yp = y + static_cast<size_t>(m0) * N;
        cudaError_t e = cudaErrorInvalidValue;
        switch (mm) {
            case 1: e = launch_f32act<1>(xp, w, type, yp, K, N, st); break;
            case 2: e = launch_f32act<2>(xp, w, type, yp, K, N, st); break;
            case 3: e = launch_f32act<3>(xp, w, type, yp, K, N, st); break;
            case 4: e = launch_f32act<4>(xp, w, type, yp, K, N, st); break;
            case 5: e = launch_f32act<5>(xp, w, type, yp, K, N, st); break;
            case 6: e = launch_f32act<6>(xp, w, type, yp, K, N, st); break;
            case 7: e = launch_f32act<7>(xp, w, type, yp, K, N, st); break;
            case 8: e = launch_f32act<8>(xp, w, type, yp, K, N, st); break;
        }
        c.launches++;
        c.last_path = 4;
        if (e != cudaSuccess) return cuda_check(e, "gemv_f32act launch");
    }
    return LAPLACE_OK;
}

int launch_dequantize(const uint8_t* w, uint32_t type, float* dst, long long n, float scale, cudaStream_t st) {
    const Geo g = geo_of(type);
    if (!g.elems) return LAPLACE_UNSUPPORTED;
    if (!w || !dst || n <= 0 || n % g.elems) return fail(LAPLACE_ERR_ARG, "dequantize: n=%lld is not a positive multiple of %d", n, g.elems);
    if ((reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(w) & (type == T_F32 ? 15 : 1)))
        return fail(LAPLACE_ERR_ARG, "dequantize: dst must be 16-byte aligned, blocks 2-byte (F32: 16-byte) aligned");
    const long long groups = n / 16;
    long long blocks = (groups + 255) / 256;
    if (blocks > static_cast<long long>(ctx().sm_count) * 16) blocks = static_cast<long long>(ctx().sm_count) * 16;
    dequantize_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(w, type, dst, groups, scale);
    ctx().launches++;
    return cuda_check(cudaGetLastError(), "dequantize launch");
}

int launch_embed_rows(const uint8_t* w, uint32_t type, const int* tokens, int M, int H, long long vocab, float scale, float* dst,
                      cudaStream_t st) {
    const Geo g = geo_of(type);
    if (!g.elems) return LAPLACE_UNSUPPORTED;
    if (!w || !tokens || !dst || M <= 0 || H <= 0 || H % g.elems || vocab <= 0)
        return fail(LAPLACE_ERR_ARG, "embed_rows: M=%d H=%d (a multiple of %d expected) vocab=%lld", M, H, g.elems, vocab);
    if ((reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(w) & (type == T_F32 ? 15 : 1)))
        return fail(LAPLACE_ERR_ARG, "embed_rows: dst must be 16-byte aligned, blocks 2-byte (F32: 16-byte) aligned");
    embed_rows_kernel<<<M, 256, 0, st>>>(w, type, tokens, H, vocab, scale, dst, ctx().d_err);
    ctx().launches++;
    return cuda_check(cudaGetLastError(), "embed_rows launch");
}

int launch_softcap(float* y, long long n, float cap, cudaStream_t st) {
    if (!y || n <= 0 || !(cap > 0.0f)) return fail(LAPLACE_ERR_ARG, "softcap: n=%lld cap=%g", n, static_cast<double>(cap));
    long long blocks = (n + 255) / 256;
    if (blocks > static_cast<long long>(ctx().sm_count) * 16) blocks = static_cast<long long>(ctx().sm_count) * 16;
    softcap_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(y, n, cap, 1.0f / cap);
    ctx().launches++;
    return cuda_check(cudaGetLastError(), "softcap launch");
}

}  // namespace lp
