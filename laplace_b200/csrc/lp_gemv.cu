// lp_gemv.cu - decode-time streaming GEMV (1..8 activation rows) for Q4_0,
// Q8_0, Q4_K and Q6_K weights, with the activation quantizer fused into the
// prologue. Replaces the row loop + dot kernels of Laplace's NEON back-end
// (src/matmul_simd.cpp:143-342, 348-455, 506-544) for small M.
//
// Shape of the kernel (one persistent CTA per SM):
//   * warp 16 is the producer: it issues 1-D bulk copies (TMA engine,
//     cp.async.bulk, no multicast) that bring 16 consecutive weight rows - one
//     contiguous byte range of the GGUF tensor, or one K-slice per row when
//     rows are long - into a ring of shared-memory stages, each guarded by a
//     full/empty mbarrier pair;
//   * while the first stages are in flight, the 16 consumer warps quantize the
//     fp32 activations into shared memory (per 32 values: d = amax/127, int8,
//     d*sum), so the quantized activations never touch HBM;
//   * consumers unpack nibbles / 6-bit fields in registers, take exact int32
//     block sums with dp4a, apply the fp16 block scales in fp32, reduce across
//     the warp with shuffles and write y.
// HBM traffic is the packed weights once, plus x and y. Every wait is bounded:
// a wait that gives up raises a status word and the CTA drains and returns.
#include "lp_common.cuh"

namespace lp {

namespace {

constexpr int CONSUMER_WARPS = 16;
constexpr int THREADS        = (CONSUMER_WARPS + 1) * 32;
constexpr int MAX_STAGES     = 8;
constexpr int REC_BYTES      = 80;   // activation record: 64 int8 + d0,d1,sum0,sum1 (fp32)

struct KParams {
    const float*   x;
    const uint8_t* w;
    float*         y;
    const int*     expert_idx;
    int*           err;
    int            K, N;
    int            n_seg;
    int            act_rows;        // rows of x quantized into shared memory
    int            per_seg_x;
    uint32_t       rb;              // bytes per weight row
    int            n_slices;        // K-slices per row (1: a tile is 16 whole rows, one copy)
    uint32_t       slice_bytes;     // bytes of a full slice of one row (16-byte multiple when n_slices > 1)
    int            slice_items;     // items of a full slice
    uint32_t       slot_bytes;      // per-row slot in a stage when n_slices > 1
    int            n_stages;
    uint32_t       stage_bytes;     // multiple of 16, includes alignment slack
    uint32_t       act_row_stride;  // bytes between quantized activation rows
    uint32_t       isum_row_stride; // bytes between rows of the int16 half-sums
    uint32_t       off_isum, off_stages;
};

// Shared-memory map: [0,64) full barriers, [64,128) empty barriers, [128,132)
// abort flag, then activations, half-sums, stages.
constexpr uint32_t OFF_FULL = 0, OFF_EMPTY = 64, OFF_ABORT = 128;
constexpr uint32_t OFF_ACT = 256;

// ------------------------------------------------------------------ tiles
// A tile is up to 16 consecutive weight rows of one segment (one per consumer
// warp), restricted to one K-slice. Slices of a row group come back to back so
// a warp keeps its row's accumulators in registers across them.
struct Tile {
    long long src_off;   // byte offset of the first row (start of the row, not of the slice) from p.w
    int seg, j0, nrows, slice;
};

struct TileWalker {
    long long g, g_end;
    int N, n_slices, slice;
    uint32_t rb;
    const int* expert_idx;
    __device__ bool next(Tile& t) {
        if (g >= g_end) return false;
        int seg = static_cast<int>(g / N);
        int j0 = static_cast<int>(g - static_cast<long long>(seg) * N);
        long long left = g_end - g;
        int nrows = CONSUMER_WARPS;
        if (nrows > N - j0) nrows = N - j0;
        if (nrows > left) nrows = static_cast<int>(left);
        long long e = expert_idx ? expert_idx[seg] : 0;
        t.src_off = (e * N + j0) * static_cast<long long>(rb);
        t.seg = seg; t.j0 = j0; t.nrows = nrows; t.slice = slice;
        if (++slice == n_slices) { slice = 0; g += nrows; }
        return true;
    }
};

// ------------------------------------------------------ per-type item code
// An "item" is the unit one lane processes at a time; items of a row are
// numbered along K. Each traits struct gives items per row and the dot.

template <uint32_t TYPE> struct Traits;

// Q4_K: item = one 64-value chunk (32 bytes of nibbles) of a super-block.
// Activation record i holds exactly the two 32-value blocks of item i.
template <> struct Traits<LAPLACE_TYPE_Q4_K> {
    __device__ static int items(int K) { return K / 64; }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M], float (&acc2)[M]) {
        const uint32_t blk = row + (i >> 2) * Q4_K_BYTES;
        const int c = i & 3;
        const uint4 hdr = lds128(blk);
        const uint4 qa = lds128(blk + 16 + 32 * c);
        const uint4 qb = lds128(blk + 32 + 32 * c);
        // 6-bit scale/min pairs of sub-blocks 2c and 2c+1 (Laplace src/kernels.h:82-90)
        uint32_t scp, mnp;
        if (c < 2) {
            scp = (hdr.y >> (16 * c)) & 0x3f3fu;
            mnp = (hdr.z >> (16 * c)) & 0x3f3fu;
        } else {
            const int s = 16 * (c - 2);
            const uint32_t a = (hdr.w >> s) & 0xffffu, b = (hdr.y >> s) & 0xffffu, cc = (hdr.z >> s) & 0xffffu;
            scp = (a & 0x0f0fu) | ((b >> 2) & 0x3030u);
            mnp = ((a >> 4) & 0x0f0fu) | ((cc >> 2) & 0x3030u);
        }
        const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
        const float d1 = d * static_cast<float>(scp & 0xff), d2 = d * static_cast<float>(scp >> 8);
        const float m1 = dmin * static_cast<float>(mnp & 0xff), m2 = dmin * static_cast<float>(mnp >> 8);
        const uint32_t wq[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t rec = act + m * astride + i * REC_BYTES;
            const uint4 x0 = lds128(rec), x1 = lds128(rec + 16), x2 = lds128(rec + 32), x3 = lds128(rec + 48);
            const uint4 sc = lds128(rec + 64);
            const uint32_t xa[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const uint32_t xb[8] = {x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w};
            int u1 = 0, u2 = 0;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                u1 = dp4a_us(wq[t] & 0x0f0f0f0fu, xa[t], u1);
                u2 = dp4a_us(wq[t] & 0xf0f0f0f0u, xb[t], u2);   // 16 x the high-nibble sum
            }
            u2 >>= 4;                                            // exact: a multiple of 16
            acc[m] = fmaf(d1 * __uint_as_float(sc.x), static_cast<float>(u1), acc[m]);
            acc[m] = fmaf(d2 * __uint_as_float(sc.y), static_cast<float>(u2), acc[m]);
            acc2[m] = fmaf(m1, __uint_as_float(sc.z), acc2[m]);
            acc2[m] = fmaf(m2, __uint_as_float(sc.w), acc2[m]);
        }
    }
};

// Q4_0: item = one 18-byte block. acc2 collects d_w * 8 * sum_x.
template <> struct Traits<LAPLACE_TYPE_Q4_0> {
    __device__ static int items(int K) { return K / 32; }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M], float (&acc2)[M]) {
        const uint32_t blk = row + i * Q4_0_BYTES;
        const float d = half_bits_to_float(lds16(blk));
        uint32_t wq[4];
        lds16B_align2(blk + 2, wq);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t rec = act + m * astride + (i >> 1) * REC_BYTES;
            const uint32_t q = rec + 32 * (i & 1);
            const uint4 x0 = lds128(q), x1 = lds128(q + 16);
            const float dx = __uint_as_float(lds32(rec + 64 + 4 * (i & 1)));
            const float sx = __uint_as_float(lds32(rec + 72 + 4 * (i & 1)));
            const uint32_t xl[4] = {x0.x, x0.y, x0.z, x0.w}, xh[4] = {x1.x, x1.y, x1.z, x1.w};
            int ul = 0, uh = 0;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                ul = dp4a_us(wq[t] & 0x0f0f0f0fu, xl[t], ul);
                uh = dp4a_us(wq[t] & 0xf0f0f0f0u, xh[t], uh);
            }
            const int u = ul + (uh >> 4);
            acc[m] = fmaf(d * dx, static_cast<float>(u), acc[m]);
            acc2[m] = fmaf(d * 8.0f, sx, acc2[m]);
        }
    }
};

// Q8_0: item = one 34-byte block.
template <> struct Traits<LAPLACE_TYPE_Q8_0> {
    __device__ static int items(int K) { return K / 32; }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M], float (&)[M]) {
        const uint32_t blk = row + i * Q8_0_BYTES;
        const float d = half_bits_to_float(lds16(blk));
        uint32_t w0[4], w1[4];
        lds16B_align2(blk + 2, w0);
        lds16B_align2(blk + 18, w1);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t rec = act + m * astride + (i >> 1) * REC_BYTES;
            const uint32_t q = rec + 32 * (i & 1);
            const uint4 x0 = lds128(q), x1 = lds128(q + 16);
            const float dx = __uint_as_float(lds32(rec + 64 + 4 * (i & 1)));
            int u = 0;
            u = dp4a_ss(w0[0], x0.x, u); u = dp4a_ss(w0[1], x0.y, u);
            u = dp4a_ss(w0[2], x0.z, u); u = dp4a_ss(w0[3], x0.w, u);
            u = dp4a_ss(w1[0], x1.x, u); u = dp4a_ss(w1[1], x1.y, u);
            u = dp4a_ss(w1[2], x1.z, u); u = dp4a_ss(w1[3], x1.w, u);
            acc[m] = fmaf(d * dx, static_cast<float>(u), acc[m]);
        }
    }
};

// Q6_K: item = (super-block, half, 16-value group s). It owns positions
// l = 16s..16s+15 of ql[l], ql[l+32], qh[l] in that half, i.e. values
// 16s..16s+15 of the four activation blocks half*4+g, g = 0..3, and the four
// sub-scales sc[8*half + 2g + s]. The dot uses the unsigned 6-bit values and
// subtracts 32 * (sum of the 16 activations): the same integer as summing
// (q6 - 32) * x (Laplace src/matmul_simd.cpp:300-335).
template <> struct Traits<LAPLACE_TYPE_Q6_K> {
    __device__ static int items(int K) { return K / 64; }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t isum,
                                uint32_t isum_stride, float (&acc)[M], float (&)[M]) {
        const int s = i & 1, half = (i >> 1) & 1, sb = i >> 2;
        const uint32_t blk = row + sb * Q6_K_BYTES;
        uint32_t qa[4], qb[4], qh[4];
        lds16B_align2(blk + 64 * half + 16 * s, qa);
        lds16B_align2(blk + 64 * half + 32 + 16 * s, qb);
        lds16B_align2(blk + 128 + 32 * half + 16 * s, qh);
        const float d = half_bits_to_float(lds16(blk + 208));
        uint32_t v[4][4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            v[0][t] = (qa[t] & 0x0f0f0f0fu) | ((qh[t] << 4) & 0x30303030u);
            v[1][t] = (qb[t] & 0x0f0f0f0fu) | ((qh[t] << 2) & 0x30303030u);
            v[2][t] = ((qa[t] >> 4) & 0x0f0f0f0fu) | (qh[t] & 0x30303030u);
            v[3][t] = ((qb[t] >> 4) & 0x0f0f0f0fu) | ((qh[t] >> 2) & 0x30303030u);
        }
        float scf[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) scf[g] = static_cast<float>(lds_s8(blk + 192 + 8 * half + 2 * g + s));
#pragma unroll
        for (int m = 0; m < M; ++m) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int ab = sb * 8 + half * 4 + g;   // activation block
                const uint32_t rec = act + m * astride + (ab >> 1) * REC_BYTES;
                const uint4 xq = lds128(rec + 32 * (ab & 1) + 16 * s);
                const float dx = __uint_as_float(lds32(rec + 64 + 4 * (ab & 1)));
                const int hs = static_cast<short>(lds16(isum + m * isum_stride + ab * 4 + 2 * s));
                int u = 0;
                u = dp4a_us(v[g][0], xq.x, u); u = dp4a_us(v[g][1], xq.y, u);
                u = dp4a_us(v[g][2], xq.z, u); u = dp4a_us(v[g][3], xq.w, u);
                u -= 32 * hs;
                acc[m] = fmaf(d * dx * scf[g], static_cast<float>(u), acc[m]);
            }
        }
    }
};

// ------------------------------------------------------------------ kernel
template <uint32_t TYPE, int M>
__global__ void __launch_bounds__(THREADS, 1) gemv_stream_kernel(const KParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_ABORT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.n_stages; ++s) {
            mbar_init(sbase + OFF_FULL + 8 * s, 1);
            mbar_init(sbase + OFF_EMPTY + 8 * s, CONSUMER_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // This CTA's contiguous share of the n_seg * N weight rows.
    const long long total = static_cast<long long>(p.n_seg) * p.N;
    TileWalker walk;
    walk.g = total * blockIdx.x / gridDim.x;
    walk.g_end = total * (blockIdx.x + 1) / gridDim.x;
    walk.N = p.N; walk.n_slices = p.n_slices; walk.slice = 0; walk.rb = p.rb; walk.expert_idx = p.expert_idx;

    const uint32_t stages = sbase + p.off_stages;

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer warp ----------------
        Tile t;
        int issued = 0;
        bool ok = true;
        while (ok && walk.next(t)) {
            const int s = issued % p.n_stages;
            const uint32_t ph = (issued / p.n_stages) & 1;
            const uint32_t full = sbase + OFF_FULL + 8 * s;
            if (lane == 0) {
                if (!mbar_wait_bounded(sbase + OFF_EMPTY + 8 * s, ph ^ 1) || *abort_flag) {
                    if (!*abort_flag) { atomicExch(p.err, DEV_TIMEOUT_EMPTY); *abort_flag = 1; }
                    ok = false;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const uint32_t stage = stages + s * p.stage_bytes;
            if (p.n_slices == 1) {
                // 16 whole rows are one contiguous byte range: a single copy
                if (lane == 0) {
                    const uint8_t* src = p.w + t.src_off;
                    const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15u);
                    const uint32_t bytes = (mis + static_cast<uint32_t>(t.nrows) * p.rb + 15u) & ~15u;
                    mbar_expect_tx(full, bytes);
                    bulk_g2s(stage, src - mis, bytes, full);
                }
            } else {
                // one copy per row: the slice of that row, into the row's slot
                const uint32_t off = static_cast<uint32_t>(t.slice) * p.slice_bytes;
                const uint32_t len = (p.rb - off) < p.slice_bytes ? (p.rb - off) : p.slice_bytes;
                const uint8_t* src = p.w + t.src_off + static_cast<long long>(lane) * p.rb + off;
                const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15u);
                uint32_t bytes = lane < t.nrows ? ((mis + len + 15u) & ~15u) : 0u;
                uint32_t sum = bytes;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (lane == 0) mbar_expect_tx(full, sum);
                __syncwarp();
                if (lane < t.nrows) bulk_g2s(stage + lane * p.slot_bytes, src - mis, bytes, full);
            }
            ++issued;
        }
        // Copies still in flight must land before the CTA gives its shared memory back.
        if (lane == 0) {
            const int pending = issued < p.n_stages ? issued : p.n_stages;
            for (int k = 0; k < pending; ++k) {
                const int tix = issued - 1 - k;
                if (!mbar_wait_bounded(sbase + OFF_FULL + 8 * (tix % p.n_stages), (tix / p.n_stages) & 1))
                    atomicExch(p.err, DEV_TIMEOUT_DRAIN);
            }
        }
    } else {
        // ---------------- consumer warps ----------------
        // (1) quantize the activations into shared memory while the ring fills
        {
            const int bpr = p.K >> 5;
            const int groups = (CONSUMER_WARPS * 32) / 8;
            const int grp = threadIdx.x >> 3, t8 = threadIdx.x & 7;
            const int nblk = p.act_rows * bpr;
            // whole warps iterate together so the 8-lane shuffles stay converged
            for (int base = 0; base < nblk; base += groups) {
                const int b = base + grp;
                const bool live = b < nblk;
                const int m = live ? b / bpr : 0, kb = live ? b - m * bpr : 0;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) v = __ldg(reinterpret_cast<const float4*>(p.x + static_cast<size_t>(m) * p.K + kb * 32) + t8);
                uint32_t packed; int hs;
                const float d = quantize_block_8lanes(v, packed, hs);
                const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
                if (live) {
                    uint8_t* rec = smem + OFF_ACT + m * p.act_row_stride + (kb >> 1) * REC_BYTES;
                    reinterpret_cast<uint32_t*>(rec + 32 * (kb & 1))[t8] = packed;
                    if (t8 == 0) {
                        const short lo = static_cast<short>(hs), hi = static_cast<short>(hs_hi);
                        reinterpret_cast<float*>(rec + 64)[kb & 1] = d;
                        reinterpret_cast<float*>(rec + 72)[kb & 1] =
                            d * static_cast<float>(static_cast<int>(lo) + static_cast<int>(hi));
                        if (p.isum_row_stride) {
                            short* is = reinterpret_cast<short*>(smem + p.off_isum + m * p.isum_row_stride + kb * 4);
                            is[0] = lo; is[1] = hi;
                        }
                    }
                }
            }
            named_bar_sync(1, CONSUMER_WARPS * 32);
        }

        // (2) stream tiles: warp r owns row r of every tile
        const int n_items = Traits<TYPE>::items(p.K);
        const uint32_t act0 = sbase + OFF_ACT, isum0 = sbase + p.off_isum;
        float acc[M], acc2[M];
#pragma unroll
        for (int m = 0; m < M; ++m) { acc[m] = 0.f; acc2[m] = 0.f; }
        Tile t;
        int tix = 0;
        while (walk.next(t)) {
            const int s = tix % p.n_stages;
            const uint32_t ph = (tix / p.n_stages) & 1;
            if (!mbar_wait_bounded(sbase + OFF_FULL + 8 * s, ph) || *abort_flag) {
                if (!*abort_flag) { atomicExch(p.err, DEV_TIMEOUT_FULL); *abort_flag = 1; }
                break;
            }
            if (warp < t.nrows) {
                const uint32_t stage = stages + s * p.stage_bytes;
                uint32_t row;      // shared address where byte 0 of this warp's weight row would sit
                if (p.n_slices == 1) {
                    const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.w + t.src_off) & 15u);
                    row = stage + mis + warp * p.rb;
                } else {
                    const uint32_t off = static_cast<uint32_t>(t.slice) * p.slice_bytes;
                    const uint32_t mis = static_cast<uint32_t>(
                        reinterpret_cast<uintptr_t>(p.w + t.src_off + static_cast<long long>(warp) * p.rb + off) & 15u);
                    row = stage + warp * p.slot_bytes + mis - off;
                }
                const int arow = p.per_seg_x ? t.seg : 0;
                const uint32_t act = act0 + arow * p.act_row_stride;
                const uint32_t isum = isum0 + arow * p.isum_row_stride;
                const int i0 = t.slice * p.slice_items;
                const int i1 = (i0 + p.slice_items) < n_items ? (i0 + p.slice_items) : n_items;
                for (int i = i0 + lane; i < i1; i += 32)
                    Traits<TYPE>::template item<M>(row, i, act, p.act_row_stride, isum, p.isum_row_stride, acc, acc2);
                if (t.slice == p.n_slices - 1) {
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        float a = acc[m], b = acc2[m];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            a += __shfl_xor_sync(0xffffffffu, a, o);
                            b += __shfl_xor_sync(0xffffffffu, b, o);
                        }
                        if (lane == 0)
                            p.y[(static_cast<size_t>(t.seg) * M + m) * p.N + t.j0 + warp] = a - b;
                        acc[m] = 0.f; acc2[m] = 0.f;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + OFF_EMPTY + 8 * s);
            ++tix;
        }
    }
    __syncthreads();
}

template <uint32_t TYPE>
cudaError_t launch_typed(int M, const KParams& p, dim3 grid, size_t smem, cudaStream_t st) {
#define LP_CASE(MM)                                                                                  \
    case MM: {                                                                                       \
        auto k = gemv_stream_kernel<TYPE, MM>;                                                       \
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return e;                                                              \
        k<<<grid, THREADS, smem, st>>>(p);                                                           \
        return cudaGetLastError();                                                                   \
    }
    switch (M) {
        LP_CASE(1) LP_CASE(2) LP_CASE(3) LP_CASE(4) LP_CASE(5) LP_CASE(6) LP_CASE(7) LP_CASE(8)
        default: return cudaErrorInvalidValue;
    }
#undef LP_CASE
}

}  // namespace

int launch_gemv_stream(const GemvArgs& a, cudaStream_t st) {
    Context& c = ctx();
    if (a.M < 1 || a.M > 8) return fail(LAPLACE_ERR_ARG, "gemv: M=%d outside 1..8", a.M);
    const int epb = block_elems(a.type);
    if (!epb) return LAPLACE_UNSUPPORTED;
    if (a.K <= 0 || a.K % epb) return fail(LAPLACE_ERR_ARG, "gemv: K=%d is not a multiple of %d", a.K, epb);
    if (a.N <= 0 || a.n_seg <= 0) return fail(LAPLACE_ERR_ARG, "gemv: N=%d n_seg=%d", a.N, a.n_seg);
    if (reinterpret_cast<uintptr_t>(a.w) & 1) return fail(LAPLACE_ERR_ARG, "gemv: weight pointer not 2-byte aligned");
    if (reinterpret_cast<uintptr_t>(a.x) & 15) return fail(LAPLACE_ERR_ARG, "gemv: x not 16-byte aligned");

    KParams p{};
    p.x = a.x; p.w = a.w; p.y = a.y; p.expert_idx = a.expert_idx; p.err = c.d_err;
    p.K = a.K; p.N = a.N; p.n_seg = a.n_seg; p.per_seg_x = a.per_seg_x;
    p.act_rows = a.per_seg_x ? a.n_seg : a.M;
    p.rb = static_cast<uint32_t>(row_bytes(a.type, a.K));
    if (a.type == LAPLACE_TYPE_Q4_K && (reinterpret_cast<uintptr_t>(a.w) & 15))
        return fail(LAPLACE_ERR_ARG, "gemv: Q4_K weights must be 16-byte aligned on the device");

    p.act_row_stride = static_cast<uint32_t>((a.K + 63) / 64) * REC_BYTES;
    p.isum_row_stride = a.type == LAPLACE_TYPE_Q6_K ? static_cast<uint32_t>(a.K / 32) * 4 : 0;   // only Q6_K reads them
    const size_t act_bytes = static_cast<size_t>(p.act_rows) * p.act_row_stride;
    const size_t isum_bytes = (static_cast<size_t>(p.act_rows) * p.isum_row_stride + 15) & ~size_t(15);
    p.off_isum = static_cast<uint32_t>(OFF_ACT + act_bytes);
    p.off_stages = static_cast<uint32_t>((p.off_isum + isum_bytes + 127) & ~size_t(127));

    // K-slicing. A stage holds one slice of 16 rows. Aim at ~2.5 KB per row
    // (a ~40 KB stage) but shrink the slice when the quantized activations
    // leave little room, so that at least 3 stages fit. Slice boundaries sit on
    // multiples of 8 blocks (any super-block for Q4_K), which keeps them
    // 16-byte aligned relative to the start of the row.
    int unit_blocks, items_per_block;
    switch (a.type) {
        case LAPLACE_TYPE_Q4_K: unit_blocks = 1; items_per_block = 4; break;
        case LAPLACE_TYPE_Q6_K: unit_blocks = 8; items_per_block = 4; break;
        default:                unit_blocks = 8; items_per_block = 1; break;   // Q4_0, Q8_0
    }
    const uint32_t bpb = static_cast<uint32_t>(block_bytes(a.type));
    const int n_blocks = a.K / epb;
    const size_t budget = c.smem_optin;
    if (p.off_stages + 4096 > budget)
        return fail(LAPLACE_ERR_LIMIT, "gemv: M=%d K=%d: activations alone fill shared memory", a.M, a.K);
    const size_t ring = budget - p.off_stages;
    size_t target = ring / (3 * CONSUMER_WARPS);      // per-row bytes that allow 3 stages
    if (target > 2560) target = 2560;
    if (p.rb + 4 <= target) {
        p.n_slices = 1;
        p.slice_bytes = p.rb;
        p.slice_items = n_blocks * items_per_block;
        p.slot_bytes = p.rb;
        p.stage_bytes = static_cast<uint32_t>((static_cast<size_t>(CONSUMER_WARPS) * p.rb + 64 + 15) & ~size_t(15));
    } else {
        int units = target > 48 ? static_cast<int>((target - 48) / (bpb * unit_blocks)) : 0;
        if (units < 1) units = 1;
        const int slice_blocks = units * unit_blocks;
        p.n_slices = (n_blocks + slice_blocks - 1) / slice_blocks;
        p.slice_bytes = static_cast<uint32_t>(slice_blocks) * bpb;
        p.slice_items = slice_blocks * items_per_block;
        p.slot_bytes = (p.slice_bytes + 15 + 16 + 15) & ~15u;      // misalignment + read-ahead slack
        p.stage_bytes = CONSUMER_WARPS * p.slot_bytes;
    }
    int stages = static_cast<int>(ring / p.stage_bytes);
    if (stages < 2)
        return fail(LAPLACE_ERR_LIMIT, "gemv: M=%d K=%d needs more shared memory than one SM has", a.M, a.K);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    p.n_stages = stages;
    const size_t smem = p.off_stages + static_cast<size_t>(stages) * p.stage_bytes;

    const long long total_rows = static_cast<long long>(a.n_seg) * a.N;
    long long tiles = (total_rows + CONSUMER_WARPS - 1) / CONSUMER_WARPS;
    int grid = c.sm_count;
    if (tiles < grid) grid = static_cast<int>(tiles);

    cudaError_t e;
    switch (a.type) {
        case LAPLACE_TYPE_Q4_K: e = launch_typed<LAPLACE_TYPE_Q4_K>(a.M, p, dim3(grid), smem, st); break;
        case LAPLACE_TYPE_Q6_K: e = launch_typed<LAPLACE_TYPE_Q6_K>(a.M, p, dim3(grid), smem, st); break;
        case LAPLACE_TYPE_Q4_0: e = launch_typed<LAPLACE_TYPE_Q4_0>(a.M, p, dim3(grid), smem, st); break;
        case LAPLACE_TYPE_Q8_0: e = launch_typed<LAPLACE_TYPE_Q8_0>(a.M, p, dim3(grid), smem, st); break;
        default: return LAPLACE_UNSUPPORTED;
    }
    c.launches++;
    c.last_path = 1;
    return cuda_check(e, "gemv_stream launch");
}

}  // namespace lp
