/*
 * oracle_q8.c - CPU restatement of Laplace's int8-activation quantized matmul.
 * TEST INFRASTRUCTURE ONLY; see oracle_q8.h for scope, citations and the
 * parity pin. Build with -ffp-contract=off so that every fused multiply-add
 * below is one that the reference's intrinsics fuse, and none is added.
 */
#include "oracle_q8.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ fp16 */

/* src/fp16.h:9-38 - exact widening, subnormals normalised by shifting. */
float lpo_fp16_to_fp32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    int      e    = (h >> 10) & 0x1f;
    uint32_t man  = h & 0x3ffu;
    uint32_t bits;
    if (e == 0x1f) {
        bits = sign | 0x7f800000u | (man << 13);
    } else if (e != 0) {
        bits = sign | ((uint32_t)(e + 112) << 23) | (man << 13);
    } else if (man == 0) {
        bits = sign;
    } else {
        int shift = 0;
        while (!(man & 0x400u)) { man <<= 1; shift++; }
        bits = sign | ((uint32_t)(113 - shift) << 23) | ((man & 0x3ffu) << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* src/fp16.h:40-69 - narrowing with round-half-up on the dropped bits (this is
 * what the reference does; it is not IEEE round-to-nearest-even on ties). */
uint16_t lpo_fp32_to_fp16(float val) {
    uint32_t bits;
    memcpy(&bits, &val, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t  e    = (int32_t)((bits >> 23) & 0xffu) - 112;
    uint32_t man  = bits & 0x7fffffu;
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man = (man | 0x800000u) >> (1 - e);
        if (man & 0x1000u) man += 0x2000u;
        return (uint16_t)(sign | (man >> 13));
    }
    if (e == 0xff - 112) {
        return (uint16_t)(sign | 0x7c00u | (man ? (man >> 13) : 0));
    }
    if (e > 30) return (uint16_t)(sign | 0x7c00u);
    if (man & 0x1000u) {
        man += 0x2000u;
        if (man & 0x800000u) {
            man = 0;
            if (++e > 30) return (uint16_t)(sign | 0x7c00u);
        }
    }
    return (uint16_t)(sign | ((uint32_t)e << 10) | (man >> 13));
}

/* -------------------------------------------------------------- layouts */

/* src/kernels.h:21-54 (sizes), src/tensor.h:41-100 */
enum { Q4_0_BYTES = 18, Q5_0_BYTES = 22, Q8_0_BYTES = 34, Q4_K_BYTES = 144, Q6_K_BYTES = 210 };

int lpo_block_elems(uint32_t type) {
    switch (type) {
        case LPO_Q4_0: case LPO_Q5_0: case LPO_Q8_0: return 32;
        case LPO_Q4_K: case LPO_Q6_K: return 256;
        default: return 0;
    }
}

static size_t block_bytes(uint32_t type) {
    switch (type) {
        case LPO_Q4_0: return Q4_0_BYTES;
        case LPO_Q5_0: return Q5_0_BYTES;
        case LPO_Q8_0: return Q8_0_BYTES;
        case LPO_Q4_K: return Q4_K_BYTES;
        case LPO_Q6_K: return Q6_K_BYTES;
        default: return 0;
    }
}

size_t lpo_row_bytes(uint32_t type, int K) {
    int epb = lpo_block_elems(type);
    return epb ? (size_t)(K / epb) * block_bytes(type) : 0;
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* src/kernels.h:82-90 - sub-block j's 6-bit scale and min from the 12 packed bytes. */
static inline void k4_scale_min(int j, const uint8_t* s, int* sc, int* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4);
        *mn = (s[j + 4] >> 4)   | ((s[j]     >> 6) << 4);
    }
}

/* Q6_K: the 32 signed weights that meet activation block half*4+g
 * (src/matmul_simd.cpp:300-323): low nibbles of ql[0..31] (g=0) or ql[32..63]
 * (g=1), high nibbles of the same (g=2,3), two bits of qh at shift 2g, minus 32. */
static inline void q6k_group(const uint8_t* ql_half, const uint8_t* qh_half, int g, int8_t w[32]) {
    const uint8_t* lo = ql_half + ((g & 1) ? 32 : 0);
    for (int l = 0; l < 32; l++) {
        int nib = (g >= 2) ? (lo[l] >> 4) : (lo[l] & 0x0f);
        int top = (qh_half[l] >> (2 * g)) & 3;
        w[l] = (int8_t)((nib | (top << 4)) - 32);
    }
}

/* ------------------------------------------------------------ quantizer */

/* NEON FMAX propagates NaN; C's fmaxf does not. */
static inline float max_nan(float a, float b) {
    if (isnan(a) || isnan(b)) return NAN;
    return a > b ? a : b;
}

/* FCVTNS: nearest, ties to even, NaN -> 0, saturating at the int32 range. */
static inline int32_t cvt_rne_s32(float v) {
    if (isnan(v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)nearbyintf(v); /* default rounding mode = to nearest even */
}

static inline int8_t sat_s8(int32_t v) {
    /* vqmovn_s32 then vqmovn_s16: two saturating narrows = clamp to int8 */
    return (int8_t)(v > 127 ? 127 : (v < -128 ? -128 : v));
}

/* src/matmul_simd.cpp:348-410 */
void lpo_quantize_row(const float* x, int K, lpo_actq8* out) {
    for (int b = 0; b < K / 32; b++) {
        const float* xb = x + (size_t)b * 32;
        lpo_actq8*   a  = out + b;
        float amax = fabsf(xb[0]);
        for (int l = 1; l < 32; l++) amax = max_nan(amax, fabsf(xb[l]));
        float d  = amax / 127.0f;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        a->d = d;
        int32_t lo = 0, hi = 0;
        for (int l = 0; l < 32; l++) {
            int32_t q = cvt_rne_s32(xb[l] * id);   /* separate multiply, then convert */
            if (l < 16) lo += q; else hi += q;     /* sums use the values before narrowing */
            a->qs[l] = sat_s8(q);
        }
        a->sum_lo = (int16_t)lo;
        a->sum_hi = (int16_t)hi;
        a->sum    = d * (float)((int)a->sum_lo + (int)a->sum_hi);
    }
}

/* src/matmul_simd.cpp:418-427 */
void lpo_quantize_rows(const float* x, int M, int K, lpo_actq8* out) {
    for (int m = 0; m < M; m++)
        lpo_quantize_row(x + (size_t)m * K, K, out + (size_t)m * (K / 32));
}

/* ------------------------------------------------ 16-element int8 dots */

/* vdotq_s32 / vusdotq_s32 on a zero accumulator: lane i = sum of products 4i..4i+3. */
static inline void dot16_ss(const int8_t* a, const int8_t* b, int32_t p[4]) {
    for (int i = 0; i < 4; i++) {
        int32_t s = 0;
        for (int t = 0; t < 4; t++) s += (int32_t)a[4 * i + t] * (int32_t)b[4 * i + t];
        p[i] = s;
    }
}
static inline void dot16_us(const uint8_t* a, const int8_t* b, int32_t p[4]) {
    for (int i = 0; i < 4; i++) {
        int32_t s = 0;
        for (int t = 0; t < 4; t++) s += (int32_t)a[4 * i + t] * (int32_t)b[4 * i + t];
        p[i] = s;
    }
}
static inline int32_t sum4(const int32_t p[4]) { return p[0] + p[1] + p[2] + p[3]; }

/* vfmaq_f32(acc, dup(scale), cvt(p)) */
static inline void fma_lanes(float acc[4], float scale, const int32_t p[4]) {
    for (int i = 0; i < 4; i++) acc[i] = fmaf(scale, (float)p[i], acc[i]);
}
/* vaddvq_f32 = FADDP twice: (l0+l1)+(l2+l3) */
static inline float hsum4(const float v[4]) { return (v[0] + v[1]) + (v[2] + v[3]); }
static inline float hsum_pair(const float a[4], const float b[4]) {
    float s[4];
    for (int i = 0; i < 4; i++) s[i] = a[i] + b[i];
    return hsum4(s);
}

/* ----------------------------------------------------------------- Q8_0 */

/* src/matmul_simd.cpp:143-160 */
static double dot_q8_0(const lpo_actq8* xa, const uint8_t* row, int K, int mode, int32_t* sums) {
    float  acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    double acc64 = 0.0, mass = 0.0;
    for (int b = 0; b < K / 32; b++) {
        const uint8_t* blk = row + (size_t)b * Q8_0_BYTES;
        const int8_t*  wq  = (const int8_t*)(blk + 2);
        float dw = lpo_fp16_to_fp32(rd16(blk));
        int32_t p0[4], p1[4];
        dot16_ss(wq, xa[b].qs, p0);
        dot16_ss(wq + 16, xa[b].qs + 16, p1);
        if (sums) sums[b] = sum4(p0) + sum4(p1);
        float scale = dw * xa[b].d;
        fma_lanes(acc0, scale, p0);
        fma_lanes(acc1, scale, p1);
        double term = (double)dw * (double)xa[b].d * (double)(sum4(p0) + sum4(p1));
        acc64 += term;
        mass += fabs(term);
    }
    if (mode == LPO_MODE_MASS) return mass;
    return mode == LPO_MODE_F64 ? acc64 : (double)hsum_pair(acc0, acc1);
}

/* ----------------------------------------------------------------- Q4_0 */

/* src/matmul_simd.cpp:162-182 - nibbles stay unsigned; the -8 is a second
 * accumulator d_w * 8 * sum_x subtracted at the end. */
static double dot_q4_0(const lpo_actq8* xa, const uint8_t* row, int K, int mode, int32_t* sums) {
    float  acc[4] = {0, 0, 0, 0};
    float  acc_offset = 0.0f;
    double acc64 = 0.0, mass = 0.0;
    for (int b = 0; b < K / 32; b++) {
        const uint8_t* blk = row + (size_t)b * Q4_0_BYTES;
        float dw = lpo_fp16_to_fp32(rd16(blk));
        uint8_t lo[16], hi[16];
        for (int l = 0; l < 16; l++) { lo[l] = blk[2 + l] & 0x0f; hi[l] = blk[2 + l] >> 4; }
        int32_t p0[4], p1[4];
        dot16_us(lo, xa[b].qs, p0);
        dot16_us(hi, xa[b].qs + 16, p1);
        if (sums) sums[b] = sum4(p0) + sum4(p1);
        float scale = dw * xa[b].d;
        fma_lanes(acc, scale, p0);
        fma_lanes(acc, scale, p1);
        acc_offset += dw * 8.0f * xa[b].sum;
        double t1 = (double)dw * (double)xa[b].d * (double)(sum4(p0) + sum4(p1));
        double t2 = (double)dw * 8.0 * (double)xa[b].sum;
        acc64 += t1 - t2;
        mass += fabs(t1) + fabs(t2);
    }
    if (mode == LPO_MODE_MASS) return mass;
    return mode == LPO_MODE_F64 ? acc64 : (double)(hsum4(acc) - acc_offset);
}

/* ----------------------------------------------------------------- Q5_0 */

/* The 32 signed weights of one 22-byte block: nibble | fifth bit << 4, minus 16
 * (src/matmul_simd.cpp:196-214; qh bit l belongs to element l). */
static inline void q5_0_weights(const uint8_t* blk, int8_t w[32]) {
    uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
    for (int l = 0; l < 16; l++) {
        w[l]      = (int8_t)((int)((blk[6 + l] & 0x0f) | (((qh >> l) & 1u) << 4)) - 16);
        w[l + 16] = (int8_t)((int)((blk[6 + l] >> 4)   | (((qh >> (l + 16)) & 1u) << 4)) - 16);
    }
}

/* src/matmul_simd.cpp:184-224 - one accumulator, the two halves fma'd in turn. */
static double dot_q5_0(const lpo_actq8* xa, const uint8_t* row, int K, int mode, int32_t* sums) {
    float  acc[4] = {0, 0, 0, 0};
    double acc64 = 0.0, mass = 0.0;
    for (int b = 0; b < K / 32; b++) {
        const uint8_t* blk = row + (size_t)b * Q5_0_BYTES;
        float dw = lpo_fp16_to_fp32(rd16(blk));
        int8_t w[32];
        q5_0_weights(blk, w);
        int32_t p0[4], p1[4];
        dot16_ss(w, xa[b].qs, p0);
        dot16_ss(w + 16, xa[b].qs + 16, p1);
        if (sums) sums[b] = sum4(p0) + sum4(p1);
        float scale = dw * xa[b].d;
        fma_lanes(acc, scale, p0);
        fma_lanes(acc, scale, p1);
        double term = (double)dw * (double)xa[b].d * (double)(sum4(p0) + sum4(p1));
        acc64 += term;
        mass += fabs(term);
    }
    if (mode == LPO_MODE_MASS) return mass;
    return mode == LPO_MODE_F64 ? acc64 : (double)hsum4(acc);
}

/* ----------------------------------------------------------------- Q4_K */

/* src/matmul_simd.cpp:226-283 */
static double dot_q4_k(const lpo_actq8* xa, const uint8_t* row, int K, int mode, int32_t* sums) {
    float  acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    float  acc_min = 0.0f;
    double acc64 = 0.0, mass = 0.0;
    for (int sb = 0; sb < K / 256; sb++) {
        const uint8_t*   blk = row + (size_t)sb * Q4_K_BYTES;
        const lpo_actq8* xs  = xa + (size_t)sb * 8;
        float d    = lpo_fp16_to_fp32(rd16(blk));
        float dmin = lpo_fp16_to_fp32(rd16(blk + 2));
        const uint8_t* scales = blk + 4;
        const uint8_t* q      = blk + 16;
        for (int c = 0; c < 4; c++, q += 32) {      /* 64 elements: low nibbles then high */
            int sc1, mn1, sc2, mn2;
            k4_scale_min(2 * c,     scales, &sc1, &mn1);
            k4_scale_min(2 * c + 1, scales, &sc2, &mn2);
            float d1 = d * (float)sc1, m1 = dmin * (float)mn1;
            float d2 = d * (float)sc2, m2 = dmin * (float)mn2;
            const lpo_actq8* a1 = xs + 2 * c;
            const lpo_actq8* a2 = a1 + 1;
            uint8_t lo[32], hi[32];
            for (int l = 0; l < 32; l++) { lo[l] = q[l] & 0x0f; hi[l] = q[l] >> 4; }
            int32_t p1a[4], p1b[4], p2a[4], p2b[4];
            dot16_us(lo,      a1->qs,      p1a);
            dot16_us(lo + 16, a1->qs + 16, p1b);
            dot16_us(hi,      a2->qs,      p2a);
            dot16_us(hi + 16, a2->qs + 16, p2b);
            int32_t u1 = sum4(p1a) + sum4(p1b), u2 = sum4(p2a) + sum4(p2b);
            if (sums) { sums[sb * 8 + 2 * c] = u1; sums[sb * 8 + 2 * c + 1] = u2; }
            float s1 = d1 * a1->d, s2 = d2 * a2->d;
            fma_lanes(acc0, s1, p1a);
            fma_lanes(acc1, s1, p1b);
            fma_lanes(acc0, s2, p2a);
            fma_lanes(acc1, s2, p2b);
            acc_min += m1 * a1->sum + m2 * a2->sum;
            double t1 = (double)d * sc1 * (double)a1->d * u1, t2 = (double)d * sc2 * (double)a2->d * u2;
            double t3 = (double)dmin * mn1 * (double)a1->sum, t4 = (double)dmin * mn2 * (double)a2->sum;
            acc64 += t1 + t2 - t3 - t4;
            mass += fabs(t1) + fabs(t2) + fabs(t3) + fabs(t4);
        }
    }
    if (mode == LPO_MODE_MASS) return mass;
    return mode == LPO_MODE_F64 ? acc64 : (double)(hsum_pair(acc0, acc1) - acc_min);
}

/* ----------------------------------------------------------------- Q6_K */

/* src/matmul_simd.cpp:285-342 - the -32 is applied to the weights before the
 * dot, and each 32-weight group carries two int8 sub-scales (one per 16). */
static double dot_q6_k(const lpo_actq8* xa, const uint8_t* row, int K, int mode, int32_t* sums) {
    float  acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    double acc64 = 0.0, mass = 0.0;
    for (int sb = 0; sb < K / 256; sb++) {
        const uint8_t* blk = row + (size_t)sb * Q6_K_BYTES;
        const int8_t*  sc  = (const int8_t*)(blk + 192);
        float d = lpo_fp16_to_fp32(rd16(blk + 208));
        for (int half = 0; half < 2; half++) {
            const uint8_t* ql = blk + 64 * half;
            const uint8_t* qh = blk + 128 + 32 * half;
            for (int g = 0; g < 4; g++) {
                int8_t w[32];
                q6k_group(ql, qh, g, w);
                const lpo_actq8* a = xa + (size_t)sb * 8 + half * 4 + g;
                int32_t p0[4], p1[4];
                dot16_ss(w, a->qs, p0);
                dot16_ss(w + 16, a->qs + 16, p1);
                int s0 = sc[8 * half + 2 * g], s1 = sc[8 * half + 2 * g + 1];
                if (sums) {
                    sums[sb * 16 + (half * 4 + g) * 2]     = sum4(p0);
                    sums[sb * 16 + (half * 4 + g) * 2 + 1] = sum4(p1);
                }
                float scale0 = d * a->d * (float)s0;
                float scale1 = d * a->d * (float)s1;
                fma_lanes(acc0, scale0, p0);
                fma_lanes(acc1, scale1, p1);
                double t0 = (double)d * (double)a->d * (double)s0 * sum4(p0);
                double t1 = (double)d * (double)a->d * (double)s1 * sum4(p1);
                acc64 += t0 + t1;
                mass += fabs(t0) + fabs(t1);
            }
        }
    }
    if (mode == LPO_MODE_MASS) return mass;
    return mode == LPO_MODE_F64 ? acc64 : (double)hsum_pair(acc0, acc1);
}

static double dot_any(uint32_t type, const lpo_actq8* xa, const uint8_t* row, int K, int mode,
                      int32_t* sums) {
    switch (type) {
        case LPO_Q8_0: return dot_q8_0(xa, row, K, mode, sums);
        case LPO_Q4_0: return dot_q4_0(xa, row, K, mode, sums);
        case LPO_Q5_0: return dot_q5_0(xa, row, K, mode, sums);
        case LPO_Q4_K: return dot_q4_k(xa, row, K, mode, sums);
        case LPO_Q6_K: return dot_q6_k(xa, row, K, mode, sums);
        default: return 0.0;
    }
}

double lpo_dot(uint32_t type, const lpo_actq8* xa, const uint8_t* row, int K, int mode) {
    return dot_any(type, xa, row, K, mode, NULL);
}

int lpo_row_blocksums(uint32_t type, const lpo_actq8* xa, const uint8_t* row, int K, int32_t* out) {
    if (!lpo_block_elems(type)) return 0;
    dot_any(type, xa, row, K, LPO_MODE_F64, out);
    return type == LPO_Q6_K ? K / 16 : K / 32;
}

/* ------------------------------------------------ static-chunk threading */

/* The reference's parallel_for hands thread t the contiguous range
 * [t*ceil(n/T), (t+1)*ceil(n/T)) (src/threadpool.h:310-320). */
typedef void (*item_fn)(void* ctx, int i);
typedef struct { item_fn fn; void* ctx; int begin, end; } span_t;

static void* span_main(void* p) {
    span_t* s = (span_t*)p;
    for (int i = s->begin; i < s->end; i++) s->fn(s->ctx, i);
    return NULL;
}

static void parallel_for(int n, int threads, item_fn fn, void* ctx) {
    if (threads > 256) threads = 256;
    if (threads <= 1 || n <= 1) {
        for (int i = 0; i < n; i++) fn(ctx, i);
        return;
    }
    pthread_t tid[256];
    span_t    sp[256];
    int chunk = (n + threads - 1) / threads;
    int used = 0;
    for (int t = 0; t < threads && t * chunk < n; t++, used++) {
        sp[t].fn = fn;
        sp[t].ctx = ctx;
        sp[t].begin = t * chunk;
        sp[t].end = sp[t].begin + chunk > n ? n : sp[t].begin + chunk;
    }
    /* the caller runs span 0, like the reference's tid 0 */
    for (int t = 1; t < used; t++) pthread_create(&tid[t], NULL, span_main, &sp[t]);
    span_main(&sp[0]);
    for (int t = 1; t < used; t++) pthread_join(tid[t], NULL);
}

/* --------------------------------------------------------------- gemm */

typedef struct {
    const lpo_actq8* xa;
    const uint8_t*   w;
    const int*       expert_idx;
    float*           y;
    uint32_t         type;
    int              M, K, N, mode;
    size_t           rb, bpr, x_stride_blocks;
} job_t;

/* src/matmul_simd.cpp:438-448 - one item = two adjacent weight rows, all m. */
static void gemm_item(void* p, int b) {
    const job_t* j = (const job_t*)p;
    int j0 = 2 * b, j1 = j0 + 2 < j->N ? j0 + 2 : j->N;
    for (int col = j0; col < j1; col++) {
        const uint8_t* row = j->w + (size_t)col * j->rb;
        for (int m = 0; m < j->M; m++)
            j->y[(size_t)m * j->N + col] =
                (float)dot_any(j->type, j->xa + (size_t)m * j->bpr, row, j->K, j->mode, NULL);
    }
}

int lpo_gemm(const float* x, const uint8_t* w, uint32_t type, float* y,
             int M, int K, int N, int mode, int threads) {
    if (!lpo_block_elems(type)) return 1;
    job_t j;
    memset(&j, 0, sizeof j);
    j.bpr = (size_t)(K / 32);
    lpo_actq8* xa = (lpo_actq8*)malloc(sizeof(lpo_actq8) * j.bpr * (size_t)(M > 0 ? M : 1));
    lpo_quantize_rows(x, M, K, xa);
    j.xa = xa; j.w = w; j.y = y; j.type = type; j.M = M; j.K = K; j.N = N; j.mode = mode;
    j.rb = lpo_row_bytes(type, K);
    int items = (N + 1) / 2;
    /* src/matmul_simd.cpp:450-454: threaded only when M > 1 or N >= 128 */
    parallel_for(items, (M > 1 || N >= 128) ? threads : 1, gemm_item, &j);
    free(xa);
    return 0;
}

/* src/matmul_simd.cpp:506-544 - one item = one (expert slot k, column). */
static void moe_item(void* p, int idx) {
    const job_t* j = (const job_t*)p;
    int k = idx / j->N, col = idx % j->N;
    const uint8_t* row = j->w + (size_t)j->expert_idx[k] * ((size_t)j->N * j->rb) + (size_t)col * j->rb;
    j->y[(size_t)k * j->N + col] =
        (float)dot_any(j->type, j->xa + (size_t)k * j->x_stride_blocks, row, j->K, j->mode, NULL);
}

static int moe_common(const float* x, int x_rows, const uint8_t* w, uint32_t type,
                      const int* expert_idx, int n_experts, float* y, int K, int N,
                      int mode, int threads) {
    if (!lpo_block_elems(type)) return 1;
    job_t j;
    memset(&j, 0, sizeof j);
    j.bpr = (size_t)(K / 32);
    lpo_actq8* xa = (lpo_actq8*)malloc(sizeof(lpo_actq8) * j.bpr * (size_t)(x_rows > 0 ? x_rows : 1));
    lpo_quantize_rows(x, x_rows, K, xa);
    j.xa = xa; j.w = w; j.expert_idx = expert_idx; j.y = y; j.type = type;
    j.K = K; j.N = N; j.mode = mode; j.rb = lpo_row_bytes(type, K);
    j.x_stride_blocks = x_rows == 1 ? 0 : j.bpr;   /* shared x: every slot reads row 0 */
    parallel_for(n_experts * N, threads, moe_item, &j);
    free(xa);
    return 0;
}

int lpo_moe_gemv(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                 int n_experts, float* y, int K, int N, int mode, int threads) {
    return moe_common(x, 1, w, type, expert_idx, n_experts, y, K, N, mode, threads);
}

int lpo_moe_gemv_multi(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                       int n_experts, float* y, int K, int N, int mode, int threads) {
    return moe_common(x, n_experts, w, type, expert_idx, n_experts, y, K, N, mode, threads);
}

int lpo_gemm_blocksums(const float* x, const uint8_t* w, uint32_t type, int32_t* out,
                       int M, int K, int N) {
    if (!lpo_block_elems(type)) return 1;
    size_t bpr = (size_t)(K / 32), rb = lpo_row_bytes(type, K);
    size_t per = type == LPO_Q6_K ? (size_t)(K / 16) : (size_t)(K / 32);
    lpo_actq8* xa = (lpo_actq8*)malloc(sizeof(lpo_actq8) * bpr * (size_t)(M > 0 ? M : 1));
    lpo_quantize_rows(x, M, K, xa);
    for (int m = 0; m < M; m++)
        for (int col = 0; col < N; col++)
            dot_any(type, xa + (size_t)m * bpr, w + (size_t)col * rb, K, LPO_MODE_F64,
                    out + ((size_t)m * N + col) * per);
    free(xa);
    return 0;
}

/* ---------------------------------- scalar fp32-activation cross-check */

/* src/matmul.cpp:84-100,123-198 - same loop order and float expressions. */
float lpo_dot_scalar(uint32_t type, const float* x, const uint8_t* row, int K) {
    float acc = 0.0f;
    if (type == LPO_Q4_0) {
        for (int b = 0; b < K / 32; b++) {
            const uint8_t* blk = row + (size_t)b * Q4_0_BYTES;
            const float*   xb  = x + b * 32;
            float sum = 0.0f;
            for (int l = 0; l < 16; l++) {
                sum += xb[l]      * (float)((blk[2 + l] & 0x0f) - 8);
                sum += xb[l + 16] * (float)((blk[2 + l] >> 4) - 8);
            }
            acc += lpo_fp16_to_fp32(rd16(blk)) * sum;
        }
    } else if (type == LPO_Q5_0) {                    /* src/matmul.cpp:102-121 */
        for (int b = 0; b < K / 32; b++) {
            const uint8_t* blk = row + (size_t)b * Q5_0_BYTES;
            const float*   xb  = x + b * 32;
            int8_t w[32];
            q5_0_weights(blk, w);
            float sum = 0.0f;
            for (int l = 0; l < 16; l++) {
                sum += xb[l]      * (float)w[l];
                sum += xb[l + 16] * (float)w[l + 16];
            }
            acc += lpo_fp16_to_fp32(rd16(blk)) * sum;
        }
    } else if (type == LPO_Q8_0) {
        for (int b = 0; b < K / 32; b++) {
            const uint8_t* blk = row + (size_t)b * Q8_0_BYTES;
            const int8_t*  q   = (const int8_t*)(blk + 2);
            float sum = 0.0f;
            for (int l = 0; l < 32; l++) sum += x[b * 32 + l] * q[l];
            acc += lpo_fp16_to_fp32(rd16(blk)) * sum;
        }
    } else if (type == LPO_Q4_K) {
        for (int sb = 0; sb < K / 256; sb++) {
            const uint8_t* blk = row + (size_t)sb * Q4_K_BYTES;
            const float*   xb  = x + sb * 256;
            float d = lpo_fp16_to_fp32(rd16(blk)), dmin = lpo_fp16_to_fp32(rd16(blk + 2));
            const uint8_t* q = blk + 16;
            for (int c = 0; c < 4; c++, q += 32) {
                int sc1, mn1, sc2, mn2;
                k4_scale_min(2 * c,     blk + 4, &sc1, &mn1);
                k4_scale_min(2 * c + 1, blk + 4, &sc2, &mn2);
                float d1 = d * sc1, m1 = dmin * mn1, d2 = d * sc2, m2 = dmin * mn2;
                float s1 = 0, s2 = 0, x1 = 0, x2 = 0;
                for (int l = 0; l < 32; l++) {
                    s1 += xb[64 * c + l]      * (float)(q[l] & 0x0f);
                    x1 += xb[64 * c + l];
                    s2 += xb[64 * c + 32 + l] * (float)(q[l] >> 4);
                    x2 += xb[64 * c + 32 + l];
                }
                acc += d1 * s1 - m1 * x1 + d2 * s2 - m2 * x2;
            }
        }
    } else if (type == LPO_Q6_K) {
        for (int sb = 0; sb < K / 256; sb++) {
            const uint8_t* blk = row + (size_t)sb * Q6_K_BYTES;
            const int8_t*  sc  = (const int8_t*)(blk + 192);
            float d = lpo_fp16_to_fp32(rd16(blk + 208));
            for (int half = 0; half < 2; half++) {
                const uint8_t* ql = blk + 64 * half;
                const uint8_t* qh = blk + 128 + 32 * half;
                const float*   xb = x + sb * 256 + half * 128;
                const int8_t*  s  = sc + 8 * half;
                for (int l = 0; l < 32; l++) {
                    int is = l / 16;
                    int q1 = (int)((ql[l]      & 0x0f) | (((qh[l] >> 0) & 3) << 4)) - 32;
                    int q2 = (int)((ql[l + 32] & 0x0f) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    int q3 = (int)((ql[l]      >> 4)   | (((qh[l] >> 4) & 3) << 4)) - 32;
                    int q4 = (int)((ql[l + 32] >> 4)   | (((qh[l] >> 6) & 3) << 4)) - 32;
                    acc += xb[l]      * (d * s[is]     * q1);
                    acc += xb[l + 32] * (d * s[is + 2] * q2);
                    acc += xb[l + 64] * (d * s[is + 4] * q3);
                    acc += xb[l + 96] * (d * s[is + 6] * q4);
                }
            }
        }
    }
    return acc;
}

typedef struct { const float* x; const uint8_t* w; float* y; uint32_t type; int M, K, N; size_t rb; } sjob_t;

/* src/matmul.cpp:320-334 - one item = one weight row, all m. */
static void scalar_item(void* p, int col) {
    const sjob_t* j = (const sjob_t*)p;
    for (int m = 0; m < j->M; m++)
        j->y[(size_t)m * j->N + col] =
            lpo_dot_scalar(j->type, j->x + (size_t)m * j->K, j->w + (size_t)col * j->rb, j->K);
}

int lpo_gemm_scalar(const float* x, const uint8_t* w, uint32_t type, float* y,
                    int M, int K, int N, int threads) {
    if (!lpo_block_elems(type)) return 1;
    sjob_t j = { x, w, y, type, M, K, N, lpo_row_bytes(type, K) };
    parallel_for(N, (M > 1 || N >= 128) ? threads : 1, scalar_item, &j);
    return 0;
}

/* src/matmul.cpp:504-603 (the four types of this path) */
int lpo_dequantize(uint32_t type, const uint8_t* w, float* dst, size_t n) {
    if (type == LPO_Q4_0) {
        for (size_t i = 0; i < n; i += 32) {
            const uint8_t* blk = w + (i / 32) * Q4_0_BYTES;
            float d = lpo_fp16_to_fp32(rd16(blk));
            for (int l = 0; l < 16; l++) {
                dst[i + l]      = d * ((blk[2 + l] & 0x0f) - 8);
                dst[i + l + 16] = d * ((blk[2 + l] >> 4) - 8);
            }
        }
    } else if (type == LPO_Q5_0) {                    /* src/matmul.cpp:532-545 */
        for (size_t i = 0; i < n; i += 32) {
            const uint8_t* blk = w + (i / 32) * Q5_0_BYTES;
            float d = lpo_fp16_to_fp32(rd16(blk));
            int8_t q[32];
            q5_0_weights(blk, q);
            for (int l = 0; l < 32; l++) dst[i + l] = d * (float)q[l];
        }
    } else if (type == LPO_Q8_0) {
        for (size_t i = 0; i < n; i += 32) {
            const uint8_t* blk = w + (i / 32) * Q8_0_BYTES;
            float d = lpo_fp16_to_fp32(rd16(blk));
            for (int l = 0; l < 32; l++) dst[i + l] = d * ((const int8_t*)blk)[2 + l];
        }
    } else if (type == LPO_Q4_K) {
        for (size_t i = 0; i < n; i += 256) {
            const uint8_t* blk = w + (i / 256) * Q4_K_BYTES;
            float d = lpo_fp16_to_fp32(rd16(blk)), dmin = lpo_fp16_to_fp32(rd16(blk + 2));
            const uint8_t* q = blk + 16;
            for (int c = 0; c < 4; c++, q += 32) {
                int sc1, mn1, sc2, mn2;
                k4_scale_min(2 * c,     blk + 4, &sc1, &mn1);
                k4_scale_min(2 * c + 1, blk + 4, &sc2, &mn2);
                float d1 = d * sc1, m1 = dmin * mn1, d2 = d * sc2, m2 = dmin * mn2;
                for (int l = 0; l < 32; l++) dst[i + 64 * c + l]      = d1 * (q[l] & 0x0f) - m1;
                for (int l = 0; l < 32; l++) dst[i + 64 * c + 32 + l] = d2 * (q[l] >> 4)   - m2;
            }
        }
    } else if (type == LPO_Q6_K) {
        for (size_t i = 0; i < n; i += 256) {
            const uint8_t* blk = w + (i / 256) * Q6_K_BYTES;
            const int8_t*  sc  = (const int8_t*)(blk + 192);
            float d = lpo_fp16_to_fp32(rd16(blk + 208));
            for (int half = 0; half < 2; half++) {
                const uint8_t* ql = blk + 64 * half;
                const uint8_t* qh = blk + 128 + 32 * half;
                const int8_t*  s  = sc + 8 * half;
                float*         y  = dst + i + 128 * half;
                for (int l = 0; l < 32; l++) {
                    int is = l / 16;
                    int q1 = (int)((ql[l]      & 0x0f) | (((qh[l] >> 0) & 3) << 4)) - 32;
                    int q2 = (int)((ql[l + 32] & 0x0f) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    int q3 = (int)((ql[l]      >> 4)   | (((qh[l] >> 4) & 3) << 4)) - 32;
                    int q4 = (int)((ql[l + 32] >> 4)   | (((qh[l] >> 6) & 3) << 4)) - 32;
                    y[l]      = d * s[is]     * q1;
                    y[l + 32] = d * s[is + 2] * q2;
                    y[l + 64] = d * s[is + 4] * q3;
                    y[l + 96] = d * s[is + 6] * q4;
                }
            }
        }
    } else {
        return 1;
    }
    return 0;
}

/* ------------------------------- the reference test's own seeded inputs */

/* tests/test_util.h:47-61 */
typedef struct { uint32_t s; } xs32;
static inline uint32_t xs_next(xs32* r) {
    r->s ^= r->s << 13; r->s ^= r->s >> 17; r->s ^= r->s << 5;
    return r->s;
}
static inline float xs_float(xs32* r) { return (float)(xs_next(r) >> 8) * (2.0f / 16777216.0f) - 1.0f; }
static inline uint8_t xs_byte(xs32* r) { return (uint8_t)(xs_next(r) & 0xff); }
/* tests/test_matmul.cpp:51-55 */
static inline uint16_t xs_small_fp16(xs32* r) {
    float d = 0.005f + 0.065f * (xs_float(r) * 0.5f + 0.5f);
    return lpo_fp32_to_fp16(d);
}
static inline void put16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)(v & 0xff); p[1] = (uint8_t)(v >> 8); }

/* tests/test_matmul.cpp:60-61: x for check_against_ref is XorShift32(7 + type). */
void lpo_testgen_x(uint32_t type, int K, float* x) {
    xs32 r = { 7u + type };
    for (int k = 0; k < K; k++) x[k] = xs_float(&r);
}

/* tests/test_matmul.cpp:142-212: weight blocks of test_q4_0 / q8_0 / q4_k / q6_k
 * (seeds 17 / 19 / 23 / 29), N * K / block_elems blocks in memory order. */
int lpo_testgen_weights(uint32_t type, int K, int N, uint8_t* out) {
    int epb = lpo_block_elems(type);
    if (!epb || type == LPO_Q5_0) return 1;          /* that test has no Q5_0 case */
    size_t nblk = (size_t)N * (size_t)(K / epb);
    xs32 r;
    switch (type) {
        case LPO_Q4_0:
            r.s = 17;
            for (size_t b = 0; b < nblk; b++, out += Q4_0_BYTES) {
                put16(out, xs_small_fp16(&r));
                for (int i = 0; i < 16; i++) out[2 + i] = xs_byte(&r);
            }
            break;
        case LPO_Q8_0:
            r.s = 19;
            for (size_t b = 0; b < nblk; b++, out += Q8_0_BYTES) {
                put16(out, xs_small_fp16(&r));
                for (int i = 0; i < 32; i++) out[2 + i] = xs_byte(&r);
            }
            break;
        case LPO_Q4_K:
            r.s = 23;
            for (size_t b = 0; b < nblk; b++, out += Q4_K_BYTES) {
                put16(out, xs_small_fp16(&r));
                put16(out + 2, xs_small_fp16(&r));
                for (int i = 0; i < 12; i++) out[4 + i] = xs_byte(&r);
                for (int i = 0; i < 128; i++) out[16 + i] = xs_byte(&r);
            }
            break;
        default: /* Q6_K */
            r.s = 29;
            for (size_t b = 0; b < nblk; b++, out += Q6_K_BYTES) {
                for (int i = 0; i < 128; i++) out[i] = xs_byte(&r);
                for (int i = 0; i < 64; i++) out[128 + i] = xs_byte(&r);
                for (int i = 0; i < 16; i++) out[192 + i] = (uint8_t)(int8_t)((int)(xs_next(&r) % 17) - 8);
                put16(out + 208, xs_small_fp16(&r));
            }
            break;
    }
    return 0;
}
