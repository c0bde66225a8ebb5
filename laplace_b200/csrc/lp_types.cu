// lp_types.cu - the weight types that have no int8 kernel in the reference, and dequantize() on the device.
//
// Laplace serves Q4_0 / Q5_0 / Q8_0 / Q4_K / Q6_K matmuls through its int8 back-end and everything else -
// F32, F16, BF16, Q2_K, Q3_K, Q5_K - through the scalar path with fp32 activations
// (gemm_fallback, src/matmul.cpp:336-352: y[m][j] = dot_row_<type>(x[m], row j)). dequantize() (src/matmul.cpp:504-675)
// turns blocks into floats for token-embedding lookups (src/model.cpp:366-378). Here:
//   dequantize_kernel        every type, 16 values per thread, the reference's expressions with separate roundings
//                            (d * sc * q - dmin * m and the like), so the result is bit-identical to dequantize()
//   embed_rows_kernel        rows tokens[m] of the embedding table, times the model's embedding scale
//   gemv_f32act_kernel       fp32 activations against on-the-fly dequantized rows: one warp per weight row, lanes
//                            over groups of 16 values; HBM-bound, a few hundred GB/s to a few TB/s depending on the
//                            type's bytes per value - these types carry embeddings, LM heads and the odd tensor of a
//                            mixed-precision file, not the bulk of the weights
//   softcap_kernel           logits = tanh(logits / cap) * cap (src/model.cpp:399-406)
#include <cuda_bf16.h>

#include "lp_common.cuh"

namespace lp {
namespace {

constexpr uint32_t T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q5_0 = 6, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12,
                   T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30;

struct Geo { int elems, bytes; };       // per block; plain types are handled as "blocks" of 16 values
__host__ __device__ inline Geo geo_of(uint32_t t) {
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

// y[m][j] = sum_k x[m][k] * dequantized(w[j][k]) for M <= 8 activation rows: a warp per weight row.
template <int M>
__global__ void __launch_bounds__(256) gemv_f32act_kernel(const float* __restrict__ x, const uint8_t* __restrict__ w, uint32_t type,
                                                          float* __restrict__ y, int K, int N, int x_in_smem) {
    extern __shared__ float xs[];
    const Geo geo = geo_of(type);
    const int gpb = geo.elems / 16, groups = K / 16;
    const size_t rb = static_cast<size_t>(K / geo.elems) * geo.bytes;
    if (x_in_smem) {
        for (int i = threadIdx.x; i < M * K / 4; i += blockDim.x) reinterpret_cast<float4*>(xs)[i] = __ldg(reinterpret_cast<const float4*>(x) + i);
        __syncthreads();
    }
    const float* xa = x_in_smem ? xs : x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (int j = blockIdx.x * wpb + warp; j < N; j += gridDim.x * wpb) {
        const uint8_t* row = w + static_cast<size_t>(j) * rb;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        for (int gi = lane; gi < groups; gi += 32) {
            float v[16];
            decode16(type, row + (gi / gpb) * geo.bytes, gi % gpb, v);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float4* xp = reinterpret_cast<const float4*>(xa + static_cast<size_t>(m) * K + gi * 16);
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 t = x_in_smem ? xp[i] : __ldg(xp + i);
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

template <int M>
cudaError_t launch_f32act(const float* x, const uint8_t* w, uint32_t type, float* y, int K, int N, cudaStream_t st) {
    const size_t xbytes = static_cast<size_t>(M) * K * sizeof(float);
    const int in_smem = xbytes <= 96 * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_f32act_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int wpb = 8;
    long long blocks = (static_cast<long long>(N) + wpb - 1) / wpb;
    const long long cap = static_cast<long long>(ctx().sm_count) * (in_smem && xbytes > 48 * 1024 ? 2 : 8);
    if (blocks > cap) blocks = cap;
    gemv_f32act_kernel<M><<<static_cast<int>(blocks), 256, in_smem ? xbytes : 0, st>>>(x, w, type, y, K, N, in_smem);
    return cudaGetLastError();
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
