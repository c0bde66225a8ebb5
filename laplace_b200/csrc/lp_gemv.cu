// lp_gemv.cu - decode-time streaming GEMV (1..8 activation rows) for Q4_0,
// Q5_0, Q8_0, Q4_K and Q6_K weights, with the activation quantizer fused into the
// prologue. Replaces the row loop + dot kernels of Laplace's NEON back-end
// (src/matmul_simd.cpp:143-342, 348-455, 506-544) for small M.
//
// Shape of the kernel (one persistent CTA per SM):
//   * every consumer warp owns a private ring of shared-memory slots that a
//     producer warp fills with its weight rows by 1-D bulk copies (TMA engine,
//     cp.async.bulk to this CTA only), a full/empty mbarrier pair per slot. A row
//     is one contiguous byte range of the GGUF tensor; long rows are cut into
//     K-slices on 16-byte boundaries. Consumers never wait for each other
//     after the prologue, and a CTA keeps ~220 KB of weight bytes in flight;
//   * while the first copies are in flight, all warps quantize the fp32
//     activations into shared memory (per 32 values: d = amax/127, int8,
//     d*sum), so the quantized activations never touch HBM;
//   * lanes unpack nibbles / 6-bit fields in registers, take exact int32 block
//     sums with dp4a, apply the fp16 block scales in fp32, reduce across the
//     warp with shuffles and write y.
// HBM traffic is the packed weights once, plus x and y. Every wait is bounded:
// a wait that gives up raises a status word, the warp drains its own copies
// and leaves.
//
// Variants inside the same kernel template:
//   * RESIDENT (Q4_K, K <= 4096): activation records live in registers; with 2..8
//     activation rows a warp keeps two of them and ceil(M/2) warps share a ring;
//   * fused all-gather (PeerOut): results are staged in shared memory and one warp
//     writes the CTA's column range to every GPU's buffer with coalesced peer stores;
//     step flags are announced by the next launch's prologue (no fence on the critical
//     path) and polled with relaxed loads while the kernel streams. The same staging
//     writes y into pinned host memory for host-pointer calls.
#include <cstdio>

#include "lp_common.cuh"

namespace lp {

namespace {

constexpr int MAX_SLOTS = 4;
constexpr int MAX_MATS = 8;
constexpr int PRODUCER_WARPS = 4;   // a lane issues a bulk copy in ~100 cycles; four warps issue in parallel
constexpr int REC_BYTES = 176;   // activation record per 128 values: 128 int8, d[4], sum[4], 16 pad
                                 // (44 words: consecutive lanes fall in distinct bank groups)

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
    int            act_regs;        // 32-value-block types, one activation row, K <= 4096: activations in registers
    uint32_t       rb;              // bytes per weight row
    int            rows_per_unit;   // whole rows per bulk copy (when n_slices == 1)
    int            n_slices;        // K-slices per row
    uint32_t       slice_bytes;     // bytes of a full slice (16-byte multiple when n_slices > 1)
    int            slice_items;     // items of a full slice
    uint32_t       slot_bytes;      // one slot of a warp's ring
    int            n_slots;
    uint32_t       act_row_stride;  // bytes between quantized activation rows
    uint32_t       isum_row_stride; // bytes between rows of the int16 half-sums (Q6_K only, else 0)
    uint32_t       off_isum, off_ring;
    int            rows_q, rows_r;  // CTA b owns rows_q (+1 if b < rows_r) rows
    // several matrices that share x (same type and K): global row g belongs to matrix i with mat_end[i-1] <= g < mat_end[i]
    int            n_mats;          // 0: one matrix (w, y, N)
    const uint8_t* mat_w[MAX_MATS];
    float*         mat_y[MAX_MATS];
    int            mat_end[MAX_MATS];
    int            mat_n[MAX_MATS];
    // optional RMSNorm of x in front of the quantizer (Laplace src/ops.cpp:34-74): x_norm = x * inv * norm_w
    const float*   norm_w;
    float          norm_eps;
    float*         x_norm_out;      // optional: the normalised rows, written by CTA 0
    PeerOut        peers;           // peers.world == 0: results go to y
    uint32_t       off_stage;       // fused all-gather: this CTA's results are staged here, [M][stage_ld] floats
    int            stage_ld;
};

// Result store: to y, or (fused all-gather) into this CTA's staging area in shared memory, from where
// one warp writes the CTA's contiguous column range to every GPU in 128-byte coalesced stores.
// `row` counts result rows, `col` the column inside this GPU's slice, `cta_col0` the CTA's first column.
// EXT: the instantiation that serves several matrices and the RMSNorm prologue; the plain one carries none of that code.
template <bool PEERS, bool EXT>
__device__ __forceinline__ void store_result(const KParams& p, uint8_t* smem, int cta_col0, size_t row, int col, float v, int mat = 0) {
    if (EXT && p.n_mats) p.mat_y[mat][row * p.mat_n[mat] + col] = v;
    else if (!PEERS || p.peers.world == 0) p.y[row * p.N + col] = v;
    else reinterpret_cast<float*>(smem + p.off_stage)[row * p.stage_ld + (col - cta_col0)] = v;
}

// Shared-memory map: [0, 64 * warps) slot barriers (per consumer warp: 4 "full"
// then 4 "empty"), then activations, half-sums, the rings.
constexpr uint32_t OFF_ACT = 2048;

// ------------------------------------------------------ per-type item code
// An "item" is the unit one lane processes at a time; items of a row are
// numbered along K. `row` is the shared address where byte 0 of the weight row
// would sit; `act` the address of the activation row's first record.

__device__ __forceinline__ uint32_t act_q(uint32_t act, int blk) {        // 32 int8 of activation block blk
    return act + (blk >> 2) * REC_BYTES + (blk & 3) * 32;
}
__device__ __forceinline__ uint32_t act_d(uint32_t act, int blk) {        // its fp32 scale; +16 is d*sum
    return act + (blk >> 2) * REC_BYTES + 128 + (blk & 3) * 4;
}

template <uint32_t TYPE> struct Traits;

// Q4_K: item = half a super-block: 128 values, 64 bytes of nibbles, the four
// sub-blocks 4h..4h+3, which are exactly activation record i.
struct Q4KAct {            // one activation record in registers
    uint32_t q[32];        // 128 int8
    float    d[4], s[4];   // per 32 values: scale, scale * integer sum
};
__device__ __forceinline__ void q4k_load_act(uint32_t rec, Q4KAct& a) {
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const uint4 v = lds128(rec + 16 * t);
        a.q[4 * t] = v.x; a.q[4 * t + 1] = v.y; a.q[4 * t + 2] = v.z; a.q[4 * t + 3] = v.w;
    }
    const uint4 dx = lds128(rec + 128), sx = lds128(rec + 144);
    a.d[0] = __uint_as_float(dx.x); a.d[1] = __uint_as_float(dx.y); a.d[2] = __uint_as_float(dx.z); a.d[3] = __uint_as_float(dx.w);
    a.s[0] = __uint_as_float(sx.x); a.s[1] = __uint_as_float(sx.y); a.s[2] = __uint_as_float(sx.z); a.s[3] = __uint_as_float(sx.w);
}
struct Q4KWts {            // half a super-block of weights in registers
    uint32_t q[16];        // 64 bytes of nibbles
    uint32_t sc4, mn4;     // 6-bit scales / mins of sub-blocks 4h..4h+3, one per byte
    float    d, dmin;
};
__device__ __forceinline__ void q4k_load_wts(uint32_t row, int i, Q4KWts& w) {
    const uint32_t blk = row + (i >> 1) * Q4_K_BYTES;
    const int h = i & 1;
    const uint4 hdr = lds128(blk);
    const uint32_t qaddr = blk + 16 + 64 * h;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const uint4 v = lds128(qaddr + 16 * t);
        w.q[4 * t] = v.x; w.q[4 * t + 1] = v.y; w.q[4 * t + 2] = v.z; w.q[4 * t + 3] = v.w;
    }
    // Laplace src/kernels.h:82-90, four sub-blocks at a time
    if (h == 0) {
        w.sc4 = hdr.y & 0x3f3f3f3fu;
        w.mn4 = hdr.z & 0x3f3f3f3fu;
    } else {
        w.sc4 = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
        w.mn4 = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
    }
    w.d = half_bits_to_float(hdr.x);
    w.dmin = half_bits_to_float(hdr.x >> 16);
}
__device__ __forceinline__ float q4k_dot(const Q4KWts& w, const Q4KAct& x) {
    float a = 0.f, am = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {                      // 64-value chunk: low nibbles, then high
        int u1a = 0, u1b = 0, u2a = 0, u2b = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            u1a = dp4a_us(w.q[8 * c + t] & 0x0f0f0f0fu, x.q[16 * c + t], u1a);
            u1b = dp4a_us(w.q[8 * c + 4 + t] & 0x0f0f0f0fu, x.q[16 * c + 4 + t], u1b);
            u2a = dp4a_us(w.q[8 * c + t] & 0xf0f0f0f0u, x.q[16 * c + 8 + t], u2a);      // 16 x the high-nibble sum
            u2b = dp4a_us(w.q[8 * c + 4 + t] & 0xf0f0f0f0u, x.q[16 * c + 12 + t], u2b);
        }
        const int u1 = u1a + u1b, u2 = (u2a + u2b) >> 4;                                // exact: a multiple of 16
        const float d1 = w.d * static_cast<float>((w.sc4 >> (16 * c)) & 0xff);
        const float d2 = w.d * static_cast<float>((w.sc4 >> (16 * c + 8)) & 0xff);
        const float m1 = w.dmin * static_cast<float>((w.mn4 >> (16 * c)) & 0xff);
        const float m2 = w.dmin * static_cast<float>((w.mn4 >> (16 * c + 8)) & 0xff);
        a = fmaf(d1 * x.d[2 * c], static_cast<float>(u1), a);
        a = fmaf(d2 * x.d[2 * c + 1], static_cast<float>(u2), a);
        am = fmaf(m1, x.s[2 * c], am);
        am = fmaf(m2, x.s[2 * c + 1], am);
    }
    return a - am;
}
// The same for two activation rows at once: the masked nibbles and the scale products of the
// weight item are formed once and meet both rows (each result is bit-identical to q4k_dot's).
__device__ __forceinline__ float2 q4k_dot2(const Q4KWts& w, const Q4KAct& x, const Q4KAct& z) {
    float a = 0.f, am = 0.f, b = 0.f, bm = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        int u1a = 0, u1b = 0, u2a = 0, u2b = 0, v1a = 0, v1b = 0, v2a = 0, v2b = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint32_t l0 = w.q[8 * c + t] & 0x0f0f0f0fu, l1 = w.q[8 * c + 4 + t] & 0x0f0f0f0fu;
            const uint32_t h0 = w.q[8 * c + t] & 0xf0f0f0f0u, h1 = w.q[8 * c + 4 + t] & 0xf0f0f0f0u;
            u1a = dp4a_us(l0, x.q[16 * c + t], u1a);      v1a = dp4a_us(l0, z.q[16 * c + t], v1a);
            u1b = dp4a_us(l1, x.q[16 * c + 4 + t], u1b);  v1b = dp4a_us(l1, z.q[16 * c + 4 + t], v1b);
            u2a = dp4a_us(h0, x.q[16 * c + 8 + t], u2a);  v2a = dp4a_us(h0, z.q[16 * c + 8 + t], v2a);
            u2b = dp4a_us(h1, x.q[16 * c + 12 + t], u2b); v2b = dp4a_us(h1, z.q[16 * c + 12 + t], v2b);
        }
        const int u1 = u1a + u1b, u2 = (u2a + u2b) >> 4, v1 = v1a + v1b, v2 = (v2a + v2b) >> 4;
        const float d1 = w.d * static_cast<float>((w.sc4 >> (16 * c)) & 0xff);
        const float d2 = w.d * static_cast<float>((w.sc4 >> (16 * c + 8)) & 0xff);
        const float m1 = w.dmin * static_cast<float>((w.mn4 >> (16 * c)) & 0xff);
        const float m2 = w.dmin * static_cast<float>((w.mn4 >> (16 * c + 8)) & 0xff);
        a = fmaf(d1 * x.d[2 * c], static_cast<float>(u1), a);
        a = fmaf(d2 * x.d[2 * c + 1], static_cast<float>(u2), a);
        am = fmaf(m1, x.s[2 * c], am);
        am = fmaf(m2, x.s[2 * c + 1], am);
        b = fmaf(d1 * z.d[2 * c], static_cast<float>(v1), b);
        b = fmaf(d2 * z.d[2 * c + 1], static_cast<float>(v2), b);
        bm = fmaf(m1, z.s[2 * c], bm);
        bm = fmaf(m2, z.s[2 * c + 1], bm);
    }
    return make_float2(a - am, b - bm);
}
template <> struct Traits<LAPLACE_TYPE_Q4_K> {
    static constexpr int ITEMS_PER_BLOCK = 2;
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M]) {
        Q4KWts w;
        q4k_load_wts(row, i, w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            Q4KAct x;
            q4k_load_act(act + m * astride + i * REC_BYTES, x);
            acc[m] += q4k_dot(w, x);
        }
    }
};

// Q4_0: item = one 18-byte block. The second term is d_w * 8 * sum_x.
// (The 32-value-block types split an item into load_w, the weight side, and dot, one activation block against it, so
// that the row loop can keep a lane's activation blocks in registers, see ACT_REGS in the kernel.)
template <> struct Traits<LAPLACE_TYPE_Q4_0> {
    static constexpr int ITEMS_PER_BLOCK = 1;
    struct W { float d; uint32_t q[4]; };
    __device__ static __forceinline__ void load_w(uint32_t row, int i, W& w) {
        const uint32_t blk = row + i * Q4_0_BYTES;
        w.d = half_bits_to_float(lds16(blk));
        lds16B_align2(blk + 2, w.q);
    }
    __device__ static __forceinline__ float dot(const W& w, const uint4& x0, const uint4& x1, float dx, float sx, float acc) {
        const uint32_t xl[4] = {x0.x, x0.y, x0.z, x0.w}, xh[4] = {x1.x, x1.y, x1.z, x1.w};
        int ul = 0, uh = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            ul = dp4a_us(w.q[t] & 0x0f0f0f0fu, xl[t], ul);
            uh = dp4a_us(w.q[t] & 0xf0f0f0f0u, xh[t], uh);
        }
        const int u = ul + (uh >> 4);
        return fmaf(w.d * dx, static_cast<float>(u), acc) - w.d * 8.0f * sx;
    }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M]) {
        W w;
        load_w(row, i, w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t q = act_q(act + m * astride, i), ds = act_d(act + m * astride, i);
            const uint4 x0 = lds128(q), x1 = lds128(q + 16);
            acc[m] = dot(w, x0, x1, __uint_as_float(lds32(ds)), __uint_as_float(lds32(ds + 16)), acc[m]);
        }
    }
};

// Q5_0: item = one 22-byte block: fp16 d, 32 fifth bits (bit l of the little-endian word belongs to value l), 16
// bytes of nibbles packed as in Q4_0. The signed weight is (nibble | bit << 4) - 16; since 0 <= nibble <= 15 that
// is the byte nibble | (bit ? 0x00 : 0xF0), built four values at a time: the four bits are spread to one per byte
// by a multiply (x * 0x00204081 puts bit i at position 8i), inverted, and multiplied by 0xF0, which stays
// inside each byte (Laplace src/matmul_simd.cpp:184-224).
template <> struct Traits<LAPLACE_TYPE_Q5_0> {
    static constexpr int ITEMS_PER_BLOCK = 1;
    __device__ static __forceinline__ uint32_t sign_fill(uint32_t four_bits) {
        return (((four_bits * 0x00204081u) & 0x01010101u) ^ 0x01010101u) * 0xF0u;
    }
    struct W { float d; uint32_t lo[4], hi[4]; };
    __device__ static __forceinline__ void load_w(uint32_t row, int i, W& w) {
        const uint32_t blk = row + i * Q5_0_BYTES;
        w.d = half_bits_to_float(lds16(blk));
        const uint32_t qh = lds16(blk + 2) | (lds16(blk + 4) << 16);
        uint32_t wq[4];
        lds16B_align2(blk + 6, wq);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            w.lo[t] = (wq[t] & 0x0f0f0f0fu) | sign_fill((qh >> (4 * t)) & 15u);
            w.hi[t] = ((wq[t] >> 4) & 0x0f0f0f0fu) | sign_fill((qh >> (16 + 4 * t)) & 15u);
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const uint4& x0, const uint4& x1, float dx, float, float acc) {
        int ua = 0, ub = 0;
        ua = dp4a_ss(w.lo[0], x0.x, ua); ub = dp4a_ss(w.lo[1], x0.y, ub);
        ua = dp4a_ss(w.lo[2], x0.z, ua); ub = dp4a_ss(w.lo[3], x0.w, ub);
        ua = dp4a_ss(w.hi[0], x1.x, ua); ub = dp4a_ss(w.hi[1], x1.y, ub);
        ua = dp4a_ss(w.hi[2], x1.z, ua); ub = dp4a_ss(w.hi[3], x1.w, ub);
        return fmaf(w.d * dx, static_cast<float>(ua + ub), acc);
    }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M]) {
        W w;
        load_w(row, i, w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t q = act_q(act + m * astride, i);
            const uint4 x0 = lds128(q), x1 = lds128(q + 16);
            acc[m] = dot(w, x0, x1, __uint_as_float(lds32(act_d(act + m * astride, i))), 0.f, acc[m]);
        }
    }
};

// Q8_0: item = one 34-byte block.
template <> struct Traits<LAPLACE_TYPE_Q8_0> {
    static constexpr int ITEMS_PER_BLOCK = 1;
    struct W { float d; uint32_t lo[4], hi[4]; };
    __device__ static __forceinline__ void load_w(uint32_t row, int i, W& w) {
        const uint32_t blk = row + i * Q8_0_BYTES;
        w.d = half_bits_to_float(lds16(blk));
        lds16B_align2(blk + 2, w.lo);
        lds16B_align2(blk + 18, w.hi);
    }
    __device__ static __forceinline__ float dot(const W& w, const uint4& x0, const uint4& x1, float dx, float, float acc) {
        int ua = 0, ub = 0;
        ua = dp4a_ss(w.lo[0], x0.x, ua); ub = dp4a_ss(w.lo[1], x0.y, ub);
        ua = dp4a_ss(w.lo[2], x0.z, ua); ub = dp4a_ss(w.lo[3], x0.w, ub);
        ua = dp4a_ss(w.hi[0], x1.x, ua); ub = dp4a_ss(w.hi[1], x1.y, ub);
        ua = dp4a_ss(w.hi[2], x1.z, ua); ub = dp4a_ss(w.hi[3], x1.w, ub);
        return fmaf(w.d * dx, static_cast<float>(ua + ub), acc);
    }
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t, uint32_t,
                                float (&acc)[M]) {
        W w;
        load_w(row, i, w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t q = act_q(act + m * astride, i);
            const uint4 x0 = lds128(q), x1 = lds128(q + 16);
            acc[m] = dot(w, x0, x1, __uint_as_float(lds32(act_d(act + m * astride, i))), 0.f, acc[m]);
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
    static constexpr int ITEMS_PER_BLOCK = 4;
    template <int M>
    __device__ static void item(uint32_t row, int i, uint32_t act, uint32_t astride, uint32_t isum,
                                uint32_t isum_stride, float (&acc)[M]) {
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
            // the four activation blocks half*4+g share record sb*2+half
            const uint32_t rec = act + m * astride + (sb * 2 + half) * REC_BYTES;
            const uint4 dx = lds128(rec + 128);
            const float dxs[4] = {__uint_as_float(dx.x), __uint_as_float(dx.y), __uint_as_float(dx.z), __uint_as_float(dx.w)};
            const uint32_t hs_base = isum + m * isum_stride + (sb * 8 + half * 4) * 4 + 2 * s;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const uint4 xq = lds128(rec + 32 * g + 16 * s);
                const int hs = static_cast<short>(lds16(hs_base + 4 * g));
                int ua = 0, ub = 0;
                ua = dp4a_us(v[g][0], xq.x, ua); ub = dp4a_us(v[g][1], xq.y, ub);
                ua = dp4a_us(v[g][2], xq.z, ua); ub = dp4a_us(v[g][3], xq.w, ub);
                const int u = ua + ub - 32 * hs;
                acc[m] = fmaf(d * dxs[g] * scf[g], static_cast<float>(u), acc[m]);
            }
        }
    }
};

// ------------------------------------------------------------------ kernel
// A unit is what one bulk copy brings: up to rows_per_unit consecutive whole
// rows of one segment, or one K-slice of one row. Producer lane w and consumer
// warp w walk the same sequence of units over w's contiguous range of rows.
struct Unit {
    const uint8_t* src;  // first byte to copy
    uint32_t  len;       // bytes the unit needs
    int       seg, j, nrows, slice, mat;
};
struct Walker {
    int g, g_end, slice;
    template <bool EXT>
    __device__ bool next(const KParams& p, Unit& u) {
        if (g >= g_end) return false;
        int seg = 0, j = g, mat = 0, n_here = p.N;
        long long rowidx = g;
        const uint8_t* base = p.w;
        if (p.expert_idx) {
            seg = g / p.N;
            j = g - seg * p.N;
            rowidx = static_cast<long long>(p.expert_idx[seg]) * p.N + j;
        } else if (EXT && p.n_mats) {
            while (g >= p.mat_end[mat]) ++mat;
            j = g - (mat ? p.mat_end[mat - 1] : 0);
            rowidx = j;
            base = p.mat_w[mat];
            n_here = p.mat_n[mat];
        }
        u.seg = seg; u.j = j; u.slice = slice; u.mat = mat;
        if (p.n_slices > 1) {
            const uint32_t off = static_cast<uint32_t>(slice) * p.slice_bytes;
            u.nrows = 1;
            u.len = (p.rb - off) < p.slice_bytes ? (p.rb - off) : p.slice_bytes;
            u.src = base + rowidx * p.rb + off;
            if (++slice == p.n_slices) { slice = 0; ++g; }
        } else {
            int n = p.rows_per_unit;
            if (n > g_end - g) n = g_end - g;
            if (n > n_here - j) n = n_here - j;        // a copy never crosses into another expert or matrix
            u.nrows = n;
            u.len = static_cast<uint32_t>(n) * p.rb;
            u.src = base + rowidx * p.rb;
            g += n;
        }
        return true;
    }
};

// WARPS consumer warps plus PRODUCER_WARPS producer warps. One producer lane
// serves one consumer: it waits for a slot of that consumer's ring to be
// released and issues the next bulk copy into it. Issuing a bulk copy holds the
// issuing lane for ~100 cycles (lanes of one warp take turns) and the SM's copy
// engine takes roughly one copy per 50 cycles, so consumers never issue copies
// themselves, several warps issue in parallel, and copies are made as large as
// the ring allows (two 2.3 KB rows per copy move ~1.5x faster than one).
//
// RESIDENT: Q4_K, one item per lane and row (K <= 4096): the lane's activation
// record never changes, so it lives in registers for the whole kernel and the
// row loop reads only weights from shared memory. With M > 1 a warp keeps TWO
// activation rows in registers and G = ceil(M / 2) warps form a group that
// shares one ring: every warp of the group meets every weight row of the group
// with its own two rows of x, so shared memory serves each weight row G times
// instead of each activation row once per weight row.
template <uint32_t TYPE, int M, int WARPS, bool RESIDENT, int PW = PRODUCER_WARPS, bool PEERS = true, bool EXT = false>
__global__ void __launch_bounds__((WARPS + PW + (PEERS ? 1 : 0)) * 32, 1) gemv_stream_kernel(const KParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // This CTA's contiguous share of the n_seg * N weight rows (fewer than 2^31),
    // cut again into one contiguous range per consumer warp.
    const int bx = static_cast<int>(blockIdx.x);
    const int g0 = bx * p.rows_q + (bx < p.rows_r ? bx : p.rows_r);
    const int cta_rows = p.rows_q + (bx < p.rows_r ? 1 : 0);
    constexpr int RW = (RESIDENT && M > 1) ? 2 : 1;          // activation rows a warp keeps in registers
    // register-held activations for the 32-value-block types (one activation row, 20 consumer warps: 89 registers a thread)
    constexpr bool ACT_REGS = !RESIDENT && M == 1 && WARPS == 20 &&
                              (TYPE == LAPLACE_TYPE_Q4_0 || TYPE == LAPLACE_TYPE_Q5_0 || TYPE == LAPLACE_TYPE_Q8_0);
    constexpr int G = RESIDENT ? (M + RW - 1) / RW : 1;       // warps per ring group
    constexpr int GROUPS = WARPS / G;
    static_assert(WARPS % G == 0, "consumer warps must split into whole groups");
    auto walker_of = [&](int w) {
        const int q = cta_rows / GROUPS, r = cta_rows - q * GROUPS;
        Walker wk;
        wk.g = g0 + w * q + (w < r ? w : r);
        wk.g_end = wk.g + q + (w < r ? 1 : 0);
        wk.slice = 0;
        return wk;
    };
    auto bar_full = [&](int w, int slot) { return sbase + w * 64 + 8 * slot; };
    auto bar_empty = [&](int w, int slot) { return sbase + w * 64 + 32 + 8 * slot; };
    auto ring_of = [&](int w) { return sbase + p.off_ring + w * (p.n_slots * p.slot_bytes); };

    if (PEERS && warp == WARPS + PW) {
        // ------------------------------ fused all-gather: its own warp -----------------------------
        // Everything the exchange needs besides the results themselves happens here, beside the warps that stream:
        // reading the step counter, announcing the previous step (a system-scope fence), watching the other GPUs'
        // flags, advancing the counter, and at the end the coalesced stores of this CTA's column range into every
        // GPU's buffer. (Done by consumer warp 0, these steps lengthened every launch by almost 3 us.)
        if (!p.peers.world) return;
        asm volatile("griddepcontrol.wait;" ::: "memory");     // the previous launch's stores and counter update are complete
        const bool chained = p.peers.step_ctr != nullptr;
        // This launch is step (counter + 1); its results go to slot (step & 3) of every buffer.
        int prev = 0;
        if (chained) {
            prev = *reinterpret_cast<volatile const int*>(p.peers.step_ctr);
            if (lane == 0) {
                asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" :: "l"(p.peers.done_ctr) : "memory");   // "this CTA has read the counter"
                // The previous launch's slices are complete (grid dependency), so one thread of the grid announces
                // them: flag [rank] of every GPU is raised to the previous step.
                if (blockIdx.x == gridDim.x - 1) {
                    __threadfence_system();
                    for (int r = 0; r < p.peers.world; ++r)
                        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" :: "l"(p.peers.flags[r] + p.peers.rank), "r"(prev) : "memory");
                }
            }
        }
        const size_t slot_off = chained ? static_cast<size_t>((prev + 1) & 3) * static_cast<size_t>(p.n_seg) * M * p.peers.ld : 0;
        // This step overwrites slot (s & 3), i.e. the slices of step s - 4. A GPU raises its flag to s' - 1 when
        // its step-s' kernel starts, and everything it enqueued before that kernel - the readers of steps up to
        // s' - 2 among them - has finished by then (stream order). So a flag of s - 3 or more says that GPU is done
        // reading step s - 4. Lane r watches GPU r; the GPUs run within a step or two of one another, so the flags
        // have normally been there for a long time.
        bool seen = !(chained && lane < p.peers.world);
        bool bumped = !(chained && blockIdx.x == 0 && lane == 0);
        for (uint32_t it = 0; it < (1u << 21); ++it) {
            if (!seen) {
                int v;
                asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.peers.flags[p.peers.rank] + lane) : "memory");
                seen = v - (prev - 2) >= 0;
            }
            if (!bumped && *reinterpret_cast<volatile unsigned*>(p.peers.done_ctr) == gridDim.x) {
                // every CTA of this launch has read the old value: one thread of the grid advances the step counter
                *reinterpret_cast<volatile unsigned*>(p.peers.done_ctr) = 0u;
                *reinterpret_cast<volatile int*>(p.peers.step_ctr) = prev + 1;
                bumped = true;
            }
            if (__all_sync(0xffffffffu, seen && bumped)) break;
            if (it > 64) __nanosleep(100);
        }
        if (!(seen && bumped)) report_status(p.err, DEV_TIMEOUT_PEER);
        named_bar_sync(3, (WARPS + 1) * 32);                    // all consumer warps of this CTA have staged their results
        // No fence follows the stores: they are complete when the grid is, and the NEXT launch (or the closing wait
        // kernel) announces them.
        const float* stage = reinterpret_cast<const float*>(smem + p.off_stage);
        for (int m = 0; m < M; ++m) {
            const size_t at = slot_off + static_cast<size_t>(m) * p.peers.ld + p.peers.col0 + g0;
            for (int i = lane; i < cta_rows; i += 32) {
                const float v = stage[m * p.stage_ld + i];
                for (int r = 0; r < p.peers.world; ++r) p.peers.y[r][at + i] = v;
            }
        }
        return;
    }
    if (warp >= WARPS) {
        // ------------------------------ producer warps -----------------------------
        constexpr int PER = (GROUPS + PW - 1) / PW;   // ring groups served per producer warp
        const int w = (warp - WARPS) * PER + lane;
        const bool serving = lane < PER && w < GROUPS;
        if (serving) {
            for (int s = 0; s < p.n_slots; ++s) { mbar_init(bar_full(w, s), 1); mbar_init(bar_empty(w, s), G); }
        }
        fence_barrier_init();
        __syncwarp();
        // Order against the activations: the consumers' loads of x must enter the
        // memory pipeline before any bulk copy, and the bulk of the copies only
        // once x has arrived - a load issued behind ~220 KB of queued copy
        // traffic waits microseconds for its turn.
        named_bar_sync(2, (WARPS + PW) * 32);   // consumers are issuing their loads of x
        const uint32_t ring = ring_of(w);
        Walker wk = walker_of(serving ? w : 0);
        if (!serving) wk.g_end = wk.g;
        Unit un;
        bool have = wk.template next<EXT>(p, un);
        int ui = 0;
        uint32_t idle = 0;
        bool gave_up = false;
        bool first_round = true;
        while (__any_sync(0xffffffffu, have)) {
            if (first_round && __all_sync(0xffffffffu, !have || ui >= 1)) {
                first_round = false;
                named_bar_sync(1, (WARPS + PW) * 32);       // x is quantized in shared memory; barriers visible
            }
            bool issued = false;
            if (have) {
                const int slot = ui % p.n_slots, round = ui / p.n_slots;
                if (round == 0 || mbar_try_wait(bar_empty(w, slot), (round - 1) & 1)) {
                    const uint8_t* src = un.src;
                    const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15u);
                    const uint32_t bytes = (mis + un.len + 15u) & ~15u;
                    mbar_expect_tx(bar_full(w, slot), bytes);
                    bulk_g2s(ring + slot * p.slot_bytes, src - mis, bytes, bar_full(w, slot));
                    ++ui;
                    issued = true;
                    have = wk.template next<EXT>(p, un);
                }
            }
            if (__any_sync(0xffffffffu, issued)) {
                idle = 0;
            } else {
                __nanosleep(64);
                if (++idle > (1u << 22)) { gave_up = true; break; }      // a consumer never released its slot
            }
        }
        if (first_round) named_bar_sync(1, (WARPS + PW) * 32);   // nothing to copy at all
        if (gave_up && lane == 0) report_status(p.err, DEV_TIMEOUT_EMPTY);
        // Copies still in flight must land before the CTA gives its shared memory back.
        if (serving) {
            const int pending = ui < p.n_slots ? ui : p.n_slots;
            for (int k = 0; k < pending; ++k) {
                const int v = ui - 1 - k;
                if (!mbar_wait_bounded(bar_full(w, v % p.n_slots), (v / p.n_slots) & 1)) report_status(p.err, DEV_TIMEOUT_DRAIN);
            }
        }
        return;
    }

    // -------------------------------- consumer warps --------------------------------
    // x may be produced, and y read, by the kernel before this one in the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // (1) quantize the activations into shared memory while the rings fill. Each
    // group of 8 lanes owns 32-value blocks grp, grp + GROUPS, ...
    {
        const int bpr = p.K >> 5;
        constexpr int GROUPS = WARPS * 4;
        const int grp = threadIdx.x >> 3, t8 = threadIdx.x & 7;
        const int nblk = p.act_rows * bpr;
        // Tell the producers first: they need ~100 cycles from here to their
        // first copy, the loads below are issued within a few.
        asm volatile("bar.arrive 2, %0;" :: "r"((WARPS + PW) * 32) : "memory");
        auto load_raw = [&](int b) -> float4 {
            if (b >= nblk) return make_float4(0.f, 0.f, 0.f, 0.f);
            const int m = b / bpr, kb = b - m * bpr;
            return __ldg(reinterpret_cast<const float4*>(p.x + static_cast<size_t>(m) * p.K + kb * 32) + t8);
        };
        auto load_w = [&](int b) -> float4 {                 // the norm weights of block b, fetched as early as x
            if (!(EXT && p.norm_w) || b >= nblk) return make_float4(0.f, 0.f, 0.f, 0.f);
            return __ldg(reinterpret_cast<const float4*>(p.norm_w + (b % bpr) * 32) + t8);
        };
        float4 nxt = load_raw(grp), nxt2 = load_raw(grp + GROUPS);                   // two rounds ahead
        float4 wnxt = load_w(grp), wnxt2 = load_w(grp + GROUPS);
        // Optional RMSNorm in front of the quantizer (Laplace src/ops.cpp:34-74: inv = 1 / sqrt(mean(x^2) + eps),
        // x_norm = x * inv * w, the two multiplies in that order). Every CTA needs every row, so every CTA computes
        // the row sums itself, from the very values its threads are about to quantize (each 32-value block belongs
        // to one 8-lane group, so every element is counted once): per-thread partial sums, shuffles, one table of
        // per-warp sums in the (not yet used) activation area, added in warp order.
        float inv_row[M];
#pragma unroll
        for (int m = 0; m < M; ++m) inv_row[m] = 1.0f;
        if (EXT && p.norm_w) {
            float part[M];
#pragma unroll
            for (int m = 0; m < M; ++m) part[m] = 0.f;
            auto add_sq = [&](const float4& v, int b) {
                const float sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
                const int mrow = b < nblk ? b / bpr : 0;
#pragma unroll
                for (int m = 0; m < M; ++m) part[m] += m == mrow ? sq : 0.f;          // values past the end are zeros
            };
            add_sq(nxt, grp);
            add_sq(nxt2, grp + GROUPS);
            for (int b = grp + 2 * GROUPS; b < nblk; b += GROUPS) add_sq(load_raw(b), b);      // read again by the loop below
            float* red = reinterpret_cast<float*>(smem + OFF_ACT);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float s = part[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) red[warp * M + m] = s;
            }
            named_bar_sync(3, WARPS * 32);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float ms = 0.f;
                for (int w = 0; w < WARPS; ++w) ms += red[w * M + m];
                inv_row[m] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ms, static_cast<float>(p.K)), p.norm_eps)));
            }
            named_bar_sync(3, WARPS * 32);            // the table has been read: the area may take the quantized rows
        }
        // x as the quantizer sees it
        auto finish_x = [&](float4 v, const float4& w, int b) -> float4 {
            if (EXT && p.norm_w && b < nblk) {
                const int m = b / bpr, kb = b - m * bpr;
                float inv = inv_row[0];
#pragma unroll
                for (int mm = 1; mm < M; ++mm) inv = m == mm ? inv_row[mm] : inv;
                v.x = __fmul_rn(__fmul_rn(v.x, inv), w.x); v.y = __fmul_rn(__fmul_rn(v.y, inv), w.y);
                v.z = __fmul_rn(__fmul_rn(v.z, inv), w.z); v.w = __fmul_rn(__fmul_rn(v.w, inv), w.w);
                if (p.x_norm_out && blockIdx.x == 0)
                    reinterpret_cast<float4*>(p.x_norm_out + static_cast<size_t>(m) * p.K + kb * 32)[t8] = v;
            }
            return v;
        };
        // whole warps iterate together so the 8-lane shuffles stay converged
        for (int base = 0; base < nblk; base += GROUPS) {
            const int b = base + grp;
            const bool live = b < nblk;
            const int m = live ? b / bpr : 0, kb = live ? b - m * bpr : 0;
            const float4 v = finish_x(nxt, wnxt, b);
            nxt = nxt2;
            nxt2 = load_raw(b + 2 * GROUPS);
            if (EXT) { wnxt = wnxt2; wnxt2 = load_w(b + 2 * GROUPS); }
            uint32_t packed; int hs;
            const float d = quantize_block_8lanes(v, packed, hs);
            const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
            if (live) {
                uint8_t* rec = smem + OFF_ACT + m * p.act_row_stride + (kb >> 2) * REC_BYTES;
                reinterpret_cast<uint32_t*>(rec + 32 * (kb & 3))[t8] = packed;
                if (t8 == 0) {
                    const short lo = static_cast<short>(hs), hi = static_cast<short>(hs_hi);
                    reinterpret_cast<float*>(rec + 128)[kb & 3] = d;
                    reinterpret_cast<float*>(rec + 144)[kb & 3] =
                        d * static_cast<float>(static_cast<int>(lo) + static_cast<int>(hi));
                    if (p.isum_row_stride) {
                        short* is = reinterpret_cast<short*>(smem + p.off_isum + m * p.isum_row_stride + kb * 4);
                        is[0] = lo; is[1] = hi;
                    }
                }
            }
        }
        named_bar_sync(1, (WARPS + PW) * 32);      // all consumers + the producer's arrive
    }

    // (2) stream this warp's (group's) units
    const int grp = warp / G, sub = warp - grp * G;
    Walker wk = walker_of(grp);
    Unit un;
    const uint32_t ring = ring_of(grp);
    const int n_items = (p.K / block_elems(TYPE)) * Traits<TYPE>::ITEMS_PER_BLOCK;
    const uint32_t act0 = sbase + OFF_ACT, isum0 = sbase + p.off_isum;
    int u = 0;
    bool ok = true;

    if constexpr (RESIDENT && M > 1) {
        // two activation rows in registers; every weight row of the group's ring meets both
        const int m0 = 2 * sub, m1 = (m0 + 1 < M) ? m0 + 1 : m0;
        const bool has_item = lane < n_items;
        Q4KAct x0, x1;
        if (has_item) {
            q4k_load_act(act0 + m0 * p.act_row_stride + lane * REC_BYTES, x0);
            q4k_load_act(act0 + m1 * p.act_row_stride + lane * REC_BYTES, x1);
        }
        for (; wk.template next<EXT>(p, un); ++u) {
            const int slot = u % p.n_slots;
            if (!mbar_wait_bounded(bar_full(grp, slot), (u / p.n_slots) & 1)) { ok = false; break; }
            const uint32_t base = ring + slot * p.slot_bytes;     // rows are 16-byte aligned here
            int r = 0;
            for (; r + 2 <= un.nrows; r += 2) {                   // two weight rows at a time: independent chains
                float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
                if (has_item) {
                    Q4KWts w0, w1;
                    q4k_load_wts(base + r * p.rb, lane, w0);
                    q4k_load_wts(base + (r + 1) * p.rb, lane, w1);
                    a = q4k_dot2(w0, x0, x1);
                    b = q4k_dot2(w1, x0, x1);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    a.x += __shfl_xor_sync(0xffffffffu, a.x, o);
                    a.y += __shfl_xor_sync(0xffffffffu, a.y, o);
                    b.x += __shfl_xor_sync(0xffffffffu, b.x, o);
                    b.y += __shfl_xor_sync(0xffffffffu, b.y, o);
                }
                if (lane == 0) {
                    store_result<PEERS, EXT>(p, smem, g0, m0, un.j + r, a.x, un.mat);
                    store_result<PEERS, EXT>(p, smem, g0, m0, un.j + r + 1, b.x, un.mat);
                    if (m1 != m0) {
                        store_result<PEERS, EXT>(p, smem, g0, m1, un.j + r, a.y, un.mat);
                        store_result<PEERS, EXT>(p, smem, g0, m1, un.j + r + 1, b.y, un.mat);
                    }
                }
            }
            if (r < un.nrows) {
                float2 a = make_float2(0.f, 0.f);
                if (has_item) {
                    Q4KWts w0;
                    q4k_load_wts(base + r * p.rb, lane, w0);
                    a = q4k_dot2(w0, x0, x1);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    a.x += __shfl_xor_sync(0xffffffffu, a.x, o);
                    a.y += __shfl_xor_sync(0xffffffffu, a.y, o);
                }
                if (lane == 0) {
                    store_result<PEERS, EXT>(p, smem, g0, m0, un.j + r, a.x, un.mat);
                    if (m1 != m0) store_result<PEERS, EXT>(p, smem, g0, m1, un.j + r, a.y, un.mat);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(grp, slot));                   // one of the group's G releases
        }
    } else if constexpr (RESIDENT) {
        Q4KAct xr;
        const bool has_item = lane < n_items;
        if (has_item) q4k_load_act(act0 + lane * REC_BYTES, xr);
        for (; wk.template next<EXT>(p, un); ++u) {
            const int slot = u % p.n_slots;
            if (!mbar_wait_bounded(bar_full(grp, slot), (u / p.n_slots) & 1)) { ok = false; break; }
            const uint32_t base = ring + slot * p.slot_bytes;     // rows are 16-byte aligned here
            int r = 0;
            for (; r + 2 <= un.nrows; r += 2) {                   // two rows at a time: independent chains
                float a0 = 0.f, a1 = 0.f;
                if (has_item) {
                    Q4KWts w0, w1;
                    q4k_load_wts(base + r * p.rb, lane, w0);
                    q4k_load_wts(base + (r + 1) * p.rb, lane, w1);
                    a0 = q4k_dot(w0, xr);
                    a1 = q4k_dot(w1, xr);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                    a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                }
                if (lane == 0) { store_result<PEERS, EXT>(p, smem, g0, 0, un.j + r, a0, un.mat); store_result<PEERS, EXT>(p, smem, g0, 0, un.j + r + 1, a1, un.mat); }
            }
            if (r < un.nrows) {
                float a0 = 0.f;
                if (has_item) {
                    Q4KWts w0;
                    q4k_load_wts(base + r * p.rb, lane, w0);
                    a0 = q4k_dot(w0, xr);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                if (lane == 0) store_result<PEERS, EXT>(p, smem, g0, 0, un.j + r, a0, un.mat);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(grp, slot));                  // slot may be refilled
        }
    } else if (ACT_REGS && p.act_regs) {
        // One activation row, whole rows of at most 128 blocks of 32 values (K <= 4096): lane l keeps the activation
        // blocks l, l + 32, l + 64, l + 96 in registers, so the row loop reads only weights from shared memory.
        if constexpr (ACT_REGS) {
            uint4 xa[4][2];
            float xd[4], xs[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = lane + 32 * k;
                if (i < n_items) {
                    const uint32_t q = act_q(act0, i), ds = act_d(act0, i);
                    xa[k][0] = lds128(q); xa[k][1] = lds128(q + 16);
                    xd[k] = __uint_as_float(lds32(ds)); xs[k] = __uint_as_float(lds32(ds + 16));
                } else {
                    xa[k][0] = xa[k][1] = make_uint4(0u, 0u, 0u, 0u);
                    xd[k] = xs[k] = 0.f;
                }
            }
            for (; wk.template next<EXT>(p, un); ++u) {
                const int slot = u % p.n_slots;
                if (!mbar_wait_bounded(bar_full(grp, slot), (u / p.n_slots) & 1)) { ok = false; break; }
                const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(un.src) & 15u);
                for (int r = 0; r < un.nrows; ++r) {
                    const uint32_t row = ring + slot * p.slot_bytes + mis + r * p.rb;
                    float a = 0.f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int i = lane + 32 * k;
                        if (i < n_items) {
                            typename Traits<TYPE>::W w;
                            Traits<TYPE>::load_w(row, i, w);
                            a = Traits<TYPE>::dot(w, xa[k][0], xa[k][1], xd[k], xs[k], a);
                        }
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                    if (lane == 0) store_result<PEERS, EXT>(p, smem, g0, static_cast<size_t>(un.seg), un.j + r, a, un.mat);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty(grp, slot));
            }
        }
    } else {
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        for (; wk.template next<EXT>(p, un); ++u) {
            const int slot = u % p.n_slots;
            if (!mbar_wait_bounded(bar_full(grp, slot), (u / p.n_slots) & 1)) { ok = false; break; }
            const uint32_t mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(un.src) & 15u);
            const int arow = p.per_seg_x ? un.seg : 0;
            const uint32_t act = act0 + arow * p.act_row_stride, isum = isum0 + arow * p.isum_row_stride;
            const int i0 = un.slice * p.slice_items;
            const int i1 = (i0 + p.slice_items) < n_items ? (i0 + p.slice_items) : n_items;
            for (int r = 0; r < un.nrows; ++r) {
                // shared address where byte 0 of this weight row would sit
                const uint32_t row = ring + slot * p.slot_bytes + mis + r * p.rb - static_cast<uint32_t>(un.slice) * p.slice_bytes;
                for (int i = i0 + lane; i < i1; i += 32)
                    Traits<TYPE>::template item<M>(row, i, act, p.act_row_stride, isum, p.isum_row_stride, acc);
                if (un.slice == p.n_slices - 1) {
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        float a = acc[m];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                        if (lane == 0) store_result<PEERS, EXT>(p, smem, g0, static_cast<size_t>(un.seg) * M + m, un.j + r, a, un.mat);
                        acc[m] = 0.f;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(grp, slot));                  // slot may be refilled
        }
    }
    if (!ok && lane == 0) report_status(p.err, DEV_TIMEOUT_FULL);   // the producer drains the copies
    // Fused all-gather: the results are staged in shared memory; the all-gather warp sends them.
    if (PEERS && p.peers.world) asm volatile("bar.arrive 3, %0;" :: "r"((WARPS + 1) * 32) : "memory");
    // Let the next kernel in the stream start launching as this grid's SMs free up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Closes a chain of fused all-gather steps: announces this GPU's slices of the current step (complete,
// since this kernel runs after the GEMV that stored them) to every GPU, then waits (bounded) until every
// source's flag has reached this GPU's step: all slices of the step are in this GPU's buffer.
// One warp; lane r talks to GPU r.
// advance = 1: the step being closed is a NEW one whose slices were stored by kernels that do not run the step protocol
// themselves (the prefill GEMM with peer stores): the counter is advanced here first.
__global__ void allgather_wait_kernel(PeerOut po, int* err, int advance) {
    const int r = threadIdx.x;
    int step = 0;
    if (r == 0) {
        step = *reinterpret_cast<volatile const int*>(po.step_ctr) + advance;
        if (advance) *reinterpret_cast<volatile int*>(po.step_ctr) = step;
    }
    step = __shfl_sync(0xffffffffu, step, 0);
    if (r >= po.world) return;
    __threadfence_system();
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" :: "l"(po.flags[r] + po.rank), "r"(step) : "memory");
    for (uint32_t it = 0; it < (1u << 21); ++it) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(po.flags[po.rank] + r) : "memory");
        if (v - step >= 0) return;
        if (it > 64) __nanosleep(100);
    }
    report_status(err, DEV_TIMEOUT_PEER);
}

template <uint32_t TYPE, int M, int WARPS, bool RESIDENT = false, int PW = PRODUCER_WARPS, bool PEERS = true, bool EXT = false>
cudaError_t launch_one(const KParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    // The opt-in shared-memory size is raised once per instantiation (not on
    // every launch, so launches stay legal inside a stream capture).
    static bool configured = false;
    auto k = gemv_stream_kernel<TYPE, M, WARPS, RESIDENT, PW, PEERS, EXT>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(ctx().smem_optin));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    // Programmatic dependent launch: this grid may start (and prefetch weights,
    // which no earlier kernel writes) while the previous kernel in the stream
    // is still draining; griddepcontrol.wait in the kernel orders the reads of
    // x and the writes of y after that kernel's completion.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((WARPS + PW + (PEERS ? 1 : 0)) * 32);      // the fused all-gather has a warp of its own
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k, p);
}

constexpr int RESIDENT_PRODUCER_WARPS = 2;  // 448 threads per CTA leave 146 registers per thread: two weight rows in flight
constexpr int RESIDENT_WARPS = 12;      // consumer warps of the register-resident path with M > 1: splits into groups of 1, 2, 3 or 4

template <uint32_t TYPE, bool EXT>
cudaError_t launch_typed(int M, bool resident, bool long_rows, const KParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    // EXT (several matrices / RMSNorm prologue) never meets the fused all-gather, so it is built without that code
    constexpr bool PE = !EXT;
    switch (M) {
        case 1:
            if constexpr (TYPE == LAPLACE_TYPE_Q4_K) {
                // the common case (results to y) gets a kernel without the fused all-gather's code
                if (resident) return (PE && p.peers.world) ? launch_one<TYPE, 1, 16, true, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st)
                                                           : launch_one<TYPE, 1, 16, true, PRODUCER_WARPS, false, EXT>(p, grid, smem, st);
            }
            if constexpr (TYPE == LAPLACE_TYPE_Q4_0 || TYPE == LAPLACE_TYPE_Q5_0 || TYPE == LAPLACE_TYPE_Q8_0) {
                if (p.act_regs) return launch_one<TYPE, 1, 20, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
            }
            if (long_rows) return launch_one<TYPE, 1, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
            if constexpr (TYPE == LAPLACE_TYPE_Q6_K) return launch_one<TYPE, 1, 20, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
            return launch_one<TYPE, 1, 24, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
#define LP_RESIDENT_CASE(m) \
        if constexpr (TYPE == LAPLACE_TYPE_Q4_K) { if (resident) return launch_one<TYPE, m, RESIDENT_WARPS, true, RESIDENT_PRODUCER_WARPS, PE, EXT>(p, grid, smem, st); }
        case 2: LP_RESIDENT_CASE(2) return launch_one<TYPE, 2, 24, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
        case 3: LP_RESIDENT_CASE(3) return launch_one<TYPE, 3, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
        case 4: LP_RESIDENT_CASE(4) return launch_one<TYPE, 4, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
        case 5: LP_RESIDENT_CASE(5) return launch_one<TYPE, 5, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
        case 6: LP_RESIDENT_CASE(6) return launch_one<TYPE, 6, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
        case 7: LP_RESIDENT_CASE(7) return launch_one<TYPE, 7, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
        case 8: LP_RESIDENT_CASE(8) return launch_one<TYPE, 8, 16, false, PRODUCER_WARPS, PE, EXT>(p, grid, smem, st);
#undef LP_RESIDENT_CASE
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

int launch_gemv_stream(const GemvArgs& a, cudaStream_t st) {
    Context& c = ctx();
    if (a.M < 1 || a.M > 8) return fail(LAPLACE_ERR_ARG, "gemv: M=%d outside 1..8", a.M);
    const int epb = block_elems(a.type);
    if (!epb) return LAPLACE_UNSUPPORTED;
    if (a.K <= 0 || a.K % epb) return fail(LAPLACE_ERR_ARG, "gemv: K=%d is not a multiple of %d", a.K, epb);
    if (a.n_mats < 0 || a.n_mats > MAX_MATS) return fail(LAPLACE_ERR_ARG, "gemv: %d matrices (at most %d share one launch)", a.n_mats, MAX_MATS);
    if (a.n_mats && (a.expert_idx || a.peers || a.n_seg != 1)) return fail(LAPLACE_ERR_ARG, "gemv: several matrices take neither expert indices nor the fused all-gather");
    if (!a.n_mats && (a.N <= 0 || a.n_seg <= 0)) return fail(LAPLACE_ERR_ARG, "gemv: N=%d n_seg=%d", a.N, a.n_seg);
    if (reinterpret_cast<uintptr_t>(a.x) & 15) return fail(LAPLACE_ERR_ARG, "gemv: x not 16-byte aligned");
    if (a.norm_w && ((reinterpret_cast<uintptr_t>(a.norm_w) & 15) || (a.x_norm_out && (reinterpret_cast<uintptr_t>(a.x_norm_out) & 15)) || a.per_seg_x))
        return fail(LAPLACE_ERR_ARG, "gemv: the norm weights (and the optional output) must be 16-byte aligned, one shared x");
    uintptr_t w_bits = reinterpret_cast<uintptr_t>(a.w);
    long long total_rows_in = static_cast<long long>(a.n_seg) * a.N;
    if (a.n_mats) {
        w_bits = 0;
        total_rows_in = 0;
        for (int i = 0; i < a.n_mats; ++i) {
            if (!a.mat_w[i] || !a.mat_y[i] || a.mat_n[i] <= 0) return fail(LAPLACE_ERR_ARG, "gemv: matrix %d: null pointer or no rows", i);
            w_bits |= reinterpret_cast<uintptr_t>(a.mat_w[i]);
            total_rows_in += a.mat_n[i];
        }
    }
    if (w_bits & 1) return fail(LAPLACE_ERR_ARG, "gemv: weight pointer not 2-byte aligned");
    if (a.type == LAPLACE_TYPE_Q4_K && (w_bits & 15))
        return fail(LAPLACE_ERR_ARG, "gemv: Q4_K weights must be 16-byte aligned on the device");

    // 3..8 activation rows against a plain Q4_K matrix: the integer block sums on mma.sync (lp_gemv_mma.cu; measured
    // 15.1 us whatever the row count against 16.7 / 18.2 / 31.5 us of the dp4a kernel at 3 / 4 / 8 rows, 4096 x 14336; with
    // two rows the dp4a kernel's 11.4 us win)
    if (a.type == LAPLACE_TYPE_Q4_K && a.M >= 3 && !a.expert_idx && !a.peers && !a.n_mats && !a.norm_w && a.n_seg == 1 && a.K % 256 == 0) {
        const int rc = launch_gemv_mma_q4k(a.x, a.w, a.y, a.M, a.K, a.N, st);
        if (rc != LAPLACE_UNSUPPORTED) return rc;
    }
    // Register-resident activations (see the kernel): Q4_K, one activation row,
    // a plain matrix whose 16-byte-aligned rows hold at most 32 items.
    const bool resident = a.type == LAPLACE_TYPE_Q4_K && !a.expert_idx && a.K <= 4096 && (w_bits & 15) == 0;
    // consumer warps, and how many of them share one ring (resident path with M > 1: ceil(M / 2))
    // one activation row, rows of 8 KB and more (K = 14336): fewer consumer warps, so that a warp's ring slot
    // holds a K-slice of a few KB (small bulk copies are issue-bound)
    const bool long_rows = !resident && a.M == 1 && row_bytes(a.type, a.K) >= 8192;
    // one activation row against blocks of 32 values, at most four blocks per lane: activations in registers (16 warps)
    const bool act_regs = a.M == 1 && !a.per_seg_x && !a.peers && a.K <= 4096 &&
                          (a.type == LAPLACE_TYPE_Q4_0 || a.type == LAPLACE_TYPE_Q5_0 || a.type == LAPLACE_TYPE_Q8_0);
    const int cwarps = resident ? (a.M == 1 ? 16 : RESIDENT_WARPS) : (act_regs || (a.type == LAPLACE_TYPE_Q6_K && a.M == 1 && !long_rows)) ? 20 : (a.M <= 2 && !long_rows ? 24 : 16);
    const int warps = (resident && a.M > 1) ? cwarps / ((a.M + 1) / 2) : cwarps;      // ring groups
    KParams p{};
    p.x = a.x; p.w = a.w; p.y = a.y; p.expert_idx = a.expert_idx; p.err = c.d_err;
    if (a.peers) {
        if (a.peers->world < 1 || a.peers->world > MAX_PEERS) return fail(LAPLACE_ERR_ARG, "gemv: %d peers", a.peers->world);
        p.peers = *a.peers;
    }
    p.K = a.K; p.N = a.N; p.n_seg = a.n_seg; p.per_seg_x = a.per_seg_x;
    p.act_regs = act_regs ? 1 : 0;
    p.n_mats = a.n_mats;
    for (int i = 0, end = 0; i < a.n_mats; ++i) {
        end += a.mat_n[i];
        p.mat_w[i] = a.mat_w[i]; p.mat_y[i] = a.mat_y[i]; p.mat_n[i] = a.mat_n[i]; p.mat_end[i] = end;
    }
    if (a.n_mats) p.N = static_cast<int>(total_rows_in);      // for the planning below: rows of all matrices
    p.norm_w = a.norm_w; p.norm_eps = a.norm_eps; p.x_norm_out = a.x_norm_out;
    p.act_rows = a.per_seg_x ? a.n_seg : a.M;
    p.rb = static_cast<uint32_t>(row_bytes(a.type, a.K));
    p.act_row_stride = static_cast<uint32_t>((a.K + 127) / 128) * REC_BYTES;
    p.isum_row_stride = a.type == LAPLACE_TYPE_Q6_K ? static_cast<uint32_t>(a.K / 32) * 4 : 0;   // only Q6_K reads them
    const size_t act_bytes = static_cast<size_t>(p.act_rows) * p.act_row_stride;
    const size_t isum_bytes = (static_cast<size_t>(p.act_rows) * p.isum_row_stride + 15) & ~size_t(15);
    p.off_isum = static_cast<uint32_t>(OFF_ACT + act_bytes);
    p.off_ring = static_cast<uint32_t>((p.off_isum + isum_bytes + 127) & ~size_t(127));

    // Ring planning. Each warp gets an equal share of what the activations
    // leave; a slot holds one K-slice of one row plus slack for a source that
    // is not 16-byte aligned (<= 15 bytes in front) and the 4-byte read-ahead
    // of the unaligned loads. Slice boundaries sit on multiples of 8 blocks
    // (any super-block for Q4_K) so they are 16-byte aligned within the row.
    const int unit_blocks = a.type == LAPLACE_TYPE_Q4_K ? 1 : 8;   // 8 x 210, 8 x 18, 8 x 22, 8 x 34 are multiples of 16
    const int items_per_block = a.type == LAPLACE_TYPE_Q4_K ? 2 : (a.type == LAPLACE_TYPE_Q6_K ? 4 : 1);
    const uint32_t bpb = static_cast<uint32_t>(block_bytes(a.type));
    const int n_blocks = a.K / epb;
    // fused all-gather: room for this CTA's results ([M][rows per CTA] floats) at the end of shared memory
    size_t stage_bytes = 0;
    if (a.peers) {
        if (a.n_seg != 1) return fail(LAPLACE_ERR_ARG, "gemv: the fused all-gather takes a plain matrix");
        const int cta_rows_max = (a.N + c.sm_count - 1) / c.sm_count + warps * 8;     // grid may be smaller than the SM count
        p.stage_ld = (cta_rows_max + 3) & ~3;
        stage_bytes = (static_cast<size_t>(a.M) * p.stage_ld * sizeof(float) + 127) & ~size_t(127);
        if (stage_bytes > 48 * 1024) return fail(LAPLACE_ERR_LIMIT, "gemv: N=%d is too wide for the fused all-gather", a.N);
    }
    const size_t budget = c.smem_optin - stage_bytes;
    if (p.off_ring + static_cast<size_t>(warps) * 2 * 256 > budget)
        return fail(LAPLACE_ERR_LIMIT, "gemv: M=%d K=%d: the quantized activations do not fit shared memory", a.M, a.K);
    const size_t per_warp = ((budget - p.off_ring) / warps) & ~size_t(15);
    const bool aligned_rows = (p.rb % 16 == 0) && ((w_bits & 15) == 0) &&
                              (a.type == LAPLACE_TYPE_Q4_K);          // the others read 4 bytes ahead
    const uint32_t slack = aligned_rows ? 0u : 32u;
    const uint32_t unit_bytes = bpb * unit_blocks;
    const int units_total = (n_blocks + unit_blocks - 1) / unit_blocks;
    auto slot_cap = [&](int n_slots) { return (per_warp / n_slots) & ~size_t(15); };
    p.rows_per_unit = 1;
    if (p.rb + slack <= slot_cap(2)) {
        // whole rows; as many per copy as give ~4.6 KB copies and still leave two slots (three if possible)
        // (a group of G warps drains a unit G times as fast as one warp: proportionally larger copies)
        int R = static_cast<int>((4608 * static_cast<size_t>(cwarps / warps) + p.rb / 2) / p.rb);
        if (R < 1) R = 1;
        if (R > 8) R = 8;
        while (R > 1 && static_cast<size_t>(R) * p.rb + slack > slot_cap(3)) --R;
        if (static_cast<size_t>(R) * p.rb + slack > slot_cap(3)) p.n_slots = 2; else p.n_slots = 3;
        p.rows_per_unit = R;
        p.n_slices = 1; p.slice_bytes = p.rb; p.slice_items = n_blocks * items_per_block;
        p.slot_bytes = (static_cast<uint32_t>(R) * p.rb + slack + 15u) & ~15u;
    } else {
        // long rows: equal K-slices, three slots
        const size_t cap = slot_cap(3);
        if (cap < unit_bytes + slack)
            return fail(LAPLACE_ERR_LIMIT, "gemv: M=%d K=%d needs more shared memory than one SM has", a.M, a.K);
        const int max_units = static_cast<int>((cap - slack) / unit_bytes);
        p.n_slices = (units_total + max_units - 1) / max_units;
        const int slice_blocks = ((units_total + p.n_slices - 1) / p.n_slices) * unit_blocks;
        p.n_slices = (n_blocks + slice_blocks - 1) / slice_blocks;
        p.slice_bytes = static_cast<uint32_t>(slice_blocks) * bpb;
        p.slice_items = slice_blocks * items_per_block;
        p.n_slots = 3;
        p.slot_bytes = (p.slice_bytes + slack + 15u) & ~15u;
    }
    if (p.n_slices != 1 && p.act_regs) return fail(LAPLACE_ERR_STATE, "gemv: internal planning error (register-held activations need whole rows)");
    // spare room: a deeper ring
    while (p.n_slots < MAX_SLOTS && static_cast<size_t>(p.n_slots + 1) * p.slot_bytes <= per_warp) p.n_slots++;
    size_t smem = p.off_ring + static_cast<size_t>(warps) * p.n_slots * p.slot_bytes;
    if (stage_bytes) { smem = (smem + 127) & ~size_t(127); p.off_stage = static_cast<uint32_t>(smem); smem += stage_bytes; }
    if (resident && (p.n_slices != 1 || slack != 0))
        return fail(LAPLACE_ERR_STATE, "gemv: internal planning error (resident path needs whole aligned rows)");

    const long long total_rows = total_rows_in;
    if (total_rows >= (1LL << 31)) return fail(LAPLACE_ERR_LIMIT, "gemv: more than 2^31 weight rows");
    // every SM takes part as soon as there are four rows for it: a small matrix is launch-bound, and 32 CTAs of 32 rows
    // (one unit per warp, the earlier rule) took 3.75 us for 4096 x 1024 where 148 CTAs of 7 rows take 3.3 us
    const long long want = (total_rows + 3) / 4;
    int grid = c.sm_count;
    if (want < grid) grid = static_cast<int>(want);
    p.rows_q = static_cast<int>(total_rows / grid);
    p.rows_r = static_cast<int>(total_rows % grid);
    if (a.peers && p.rows_q + 1 > p.stage_ld) return fail(LAPLACE_ERR_STATE, "gemv: internal planning error (staging area too small)");

    cudaError_t e;
    const bool ext = a.n_mats > 0 || a.norm_w != nullptr;
    switch (a.type) {
        case LAPLACE_TYPE_Q4_K:
            e = ext ? launch_typed<LAPLACE_TYPE_Q4_K, true>(a.M, resident, long_rows, p, dim3(grid), smem, st)
                    : launch_typed<LAPLACE_TYPE_Q4_K, false>(a.M, resident, long_rows, p, dim3(grid), smem, st);
            break;
        case LAPLACE_TYPE_Q6_K: e = ext ? launch_typed<LAPLACE_TYPE_Q6_K, true>(a.M, false, long_rows, p, dim3(grid), smem, st)
                                        : launch_typed<LAPLACE_TYPE_Q6_K, false>(a.M, false, long_rows, p, dim3(grid), smem, st); break;
        case LAPLACE_TYPE_Q4_0: e = ext ? launch_typed<LAPLACE_TYPE_Q4_0, true>(a.M, false, long_rows, p, dim3(grid), smem, st)
                                        : launch_typed<LAPLACE_TYPE_Q4_0, false>(a.M, false, long_rows, p, dim3(grid), smem, st); break;
        case LAPLACE_TYPE_Q5_0: e = ext ? launch_typed<LAPLACE_TYPE_Q5_0, true>(a.M, false, long_rows, p, dim3(grid), smem, st)
                                        : launch_typed<LAPLACE_TYPE_Q5_0, false>(a.M, false, long_rows, p, dim3(grid), smem, st); break;
        case LAPLACE_TYPE_Q8_0: e = ext ? launch_typed<LAPLACE_TYPE_Q8_0, true>(a.M, false, long_rows, p, dim3(grid), smem, st)
                                        : launch_typed<LAPLACE_TYPE_Q8_0, false>(a.M, false, long_rows, p, dim3(grid), smem, st); break;
        default: return LAPLACE_UNSUPPORTED;
    }
    c.launches++;
    c.last_path = 1;
    return cuda_check(e, "gemv_stream launch");
}

int launch_allgather_wait(const PeerOut& po, cudaStream_t st, bool advance) {
    Context& c = ctx();
    if (po.world < 1 || po.world > MAX_PEERS) return fail(LAPLACE_ERR_ARG, "allgather_wait: %d peers", po.world);
    allgather_wait_kernel<<<1, 32, 0, st>>>(po, c.d_err, advance ? 1 : 0);
    c.launches++;
    return cuda_check(cudaGetLastError(), "allgather_wait launch");
}

}  // namespace lp
