// lp_gemm_sa.cu - prefill GEMM (M >= 9 activation rows) and expert-grouped matmul for Q4_K weights on the
// 5th-generation tensor cores, "scaled activation" formulation. Replaces gemm_int<dot_row_q4_k_int_neon> of
// Laplace's NEON back-end (src/matmul_simd.cpp:226-283, 432-455) for large M.
//
// The reference's result for one (token m, weight row n) is
//   y[m,n] = sum_sb ( d[n,sb] * sum_{j<8} sc[n,sb,j] * d_x[m,b] * U[m,n,b]  -  dmin[n,sb] * sum_{j<8} mn[n,sb,j] * sum_x[m,b] ),
//   b = 8 sb + j,  U = integer dot of a 32-value block,  sum_x = d_x * (integer sum of the block's int8 activations).
// Every 32-value block carries its own fp32 activation scale d_x, so a tensor-core kernel that keeps the block sums
// as integers has to take each block's 128x128 partial result out of TMEM and scale it on CUDA cores: one
// multiply-add per element per block, as much work as the MMA itself, plus a hand-off per block. Here the scale
// goes INTO the activation operand instead: a[m,k] = 2^e_m * d_x[m,b] * q_x[m,k] (fp32, e_m a per-row exponent that
// brings the row's largest value to 2^13), split into two fp16 pieces a = hi + lo that carry 22 bits of it. The
// weight operand is sc * nibble <= 945, exact in fp16. Two MMAs per 16-value step then accumulate, in fp32, a whole
// super-block (256 values) per drain:
//   F[n,m]  = sum_{k in sb} (sc*nibble)[n,k] * (hi + lo)[m,k]                    (tcgen05.mma kind::f16, 2 x 16 steps)
//   G[n,m]  = sum_{j<8} mn[n,sb,j] * (ghi + glo)[m,8sb+j],  g = 2^e_m / 64 * sum_x   (one more K = 16 step)
//   y[m,n] += 2^-e_m * ( d[n,sb] * F - 64 dmin[n,sb] * G )                          (CUDA cores, once per super-block)
// Products are exact; what is rounded is the split of a (2^-22 relative) and the fp32 accumulation, which the
// reference also does in fp32 in another order. Integer block sums are still exact whenever the activations are:
// a block whose scale is a power of two gives lo = 0 and an exact hi, hence an exact integer times the scale.
//
// Roles of the operands: WEIGHT rows sit on the MMA's M side (128 TMEM lanes), TOKENS on its N side (16 .. 128
// columns), so a tile with few tokens - an expert of a mixture-of-experts layer with 16 tokens - costs a
// proportionally short MMA, and the per-super-block weight scales are per-lane scalars in the drain.
//
// One 512-thread CTA per SM, persistent over tiles of 128 weight rows x up to 128 tokens:
//   warp 0      TMA: activation operand tiles (hi and lo piece, 64 k x tokens, 128-byte swizzle)
//   warp 1      MMA issue (one lane); owns the TMEM allocation
//   warp 3      TMA: packed Q4_K super-blocks (128 rows x 144 bytes) and the g operand (4 super-blocks per tile)
//   warps 4-7   converters: packed super-block -> fp16 weight operand tile (thread = weight row), the row's
//               d / dmin into a table, its mins into the G operand
//   warps 8-15  drain: tcgen05.ld of F and G (double buffered in TMEM) once per super-block, running y in registers
// All mbarrier waits are bounded; a wait that gives up raises the status word and every role leaves its loop.
#include <cuda_fp16.h>

#include <vector>

#include "lp_tc.cuh"

namespace lp {

namespace {

using namespace tc;

constexpr int TW = 128;                            // weight rows per tile (MMA M)
constexpr int TT = 128;                            // most tokens per tile (MMA N)
constexpr int BKC = 64;                            // k per pipeline stage
constexpr int STAGES = 3;
constexpr int RAW_STAGES = 2;
constexpr int RAW_TILE = TW * Q4_K_BYTES;          // 18 KB
constexpr int OP_TILE = 128 * BKC * 2;             // 16 KB: 128 rows of 64 fp16
constexpr int TABN = 4;                            // ring of per-super-block (d, -64 dmin) tables
constexpr int THREADS = 512;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_F = 0, TM_G = 256;           // two buffers of 128 columns each

constexpr uint32_t OFF_W = 0;
constexpr uint32_t OFF_AH = OFF_W + STAGES * OP_TILE;
constexpr uint32_t OFF_AL = OFF_AH + STAGES * OP_TILE;
constexpr uint32_t OFF_GM = OFF_AL + STAGES * OP_TILE;      // mins operand: 128 weight rows x (4 super-blocks x 16 k)
constexpr uint32_t OFF_GS = OFF_GM + OP_TILE;               // g operand: tokens x (4 super-blocks x 16 k)
constexpr uint32_t OFF_RAW = OFF_GS + OP_TILE;
constexpr uint32_t OFF_TAB = OFF_RAW + RAW_STAGES * RAW_TILE;
constexpr uint32_t OFF_BAR = OFF_TAB + TABN * TW * 8;
constexpr uint32_t BAR_FULL_A = OFF_BAR, BAR_FULL_W = BAR_FULL_A + 8 * STAGES, BAR_EMPTY = BAR_FULL_W + 8 * STAGES,
                   BAR_RAW_FULL = BAR_EMPTY + 8 * STAGES, BAR_RAW_EMPTY = BAR_RAW_FULL + 8 * RAW_STAGES,
                   BAR_TMEM_FULL = BAR_RAW_EMPTY + 8 * RAW_STAGES, BAR_TMEM_EMPTY = BAR_TMEM_FULL + 16,
                   BAR_G_FULL_S = BAR_TMEM_EMPTY + 16, BAR_G_FULL_M = BAR_G_FULL_S + 8, BAR_G_EMPTY = BAR_G_FULL_M + 32,
                   BAR_TAB_EMPTY = BAR_G_EMPTY + 8, OFF_TMEM_PTR = BAR_TAB_EMPTY + 8 * TABN, OFF_ABORT = OFF_TMEM_PTR + 8;
constexpr uint32_t SMEM_BYTES = OFF_ABORT + 8 + 1024;       // + slack for the 1024-byte alignment
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(OFF_RAW % 128 == 0 && RAW_TILE % 128 == 0, "TMA destinations are 128-byte aligned");

struct SaParams {
    float*       y;            // [rows of y][N]
    const float* inv_s;        // [operand rows] 2^-e_m
    int*         err;
    int          M, N, K;
    int          m_pad;        // operand rows per piece: the lo piece of operand row r is row m_pad + r of the tensor map
    int          tiles_m, tiles_n;
    // expert-grouped calls: tiles come from a table built on the device; operand row r is written to row out_row[r]
    // of y (-1: a padding row)
    const int4*  tile_tab;     // {first operand row, first weight row within the expert, first weight row of the expert, tokens}
    const int*   n_tiles_dev;
    const int*   out_row;
    int          out_identity; // 1: a live operand row r is written to row r of y
    // split-K (dense tiling with few output tiles): ksplit CTAs share an output tile, each takes sb_per super-blocks
    // and writes its partial result to y_part[slice][M][N]; a second kernel adds the slices in a fixed order
    int          ksplit, sb_per;
    float*       y_part;
};

struct TileRef { int m0, n0, wrow0, nt, sb0, sb1, ks; };     // nt = tokens of the tile (the MMA's N is nt rounded up to 16)
__device__ __forceinline__ TileRef tile_ref(const SaParams& p, int tile) {
    const int nsb = p.K / 256;
    if (p.tile_tab) {
        const int4 t = __ldg(p.tile_tab + tile);
        return {t.x, t.y, t.z, t.w, 0, nsb, 0};
    }
    const int out_tiles = p.tiles_m * p.tiles_n;
    const int ks = tile / out_tiles, t = tile - ks * out_tiles;
    const int sb0 = ks * p.sb_per;
    const int sb1 = sb0 + p.sb_per < nsb ? sb0 + p.sb_per : nsb;
    const int m0 = (t % p.tiles_m) * TT;
    return {m0, (t / p.tiles_m) * TW, 0, p.M - m0 < TT ? p.M - m0 : TT, sb0, sb1, ks};
}
__device__ __forceinline__ int tile_count(const SaParams& p) {
    return p.tile_tab ? __ldg(p.n_tiles_dev) : p.tiles_m * p.tiles_n * p.ksplit;
}
// Activation boxes come in four heights; a tile uses the smallest that holds its tokens.
__device__ __forceinline__ int box_bucket(int nt) { return nt <= 16 ? 0 : nt <= 32 ? 1 : nt <= 64 ? 2 : 3; }

struct SaMaps {
    CUtensorMap a[4];      // activation pieces, [2 * m_pad][K] fp16, boxes of 64 k x {16, 32, 64, 128} rows, 128-byte swizzle
    CUtensorMap g[4];      // g pieces, [m_pad][K/256 * 16] fp16, same boxes
    CUtensorMap w;         // packed weights as bytes, rows of K/256 * 144 bytes, boxes of 144 bytes x 128 rows
};

__global__ void __launch_bounds__(THREADS, 1)
gemm_q4k_sa_kernel(const __grid_constant__ SaMaps maps, const SaParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_ABORT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sbase + BAR_FULL_A + 8 * s, 1);
            mbar_init(sbase + BAR_FULL_W + 8 * s, 4);        // one arrive per converter warp
            mbar_init(sbase + BAR_EMPTY + 8 * s, 1);         // tcgen05.commit
        }
        for (int q = 0; q < RAW_STAGES; ++q) {
            mbar_init(sbase + BAR_RAW_FULL + 8 * q, 1);
            mbar_init(sbase + BAR_RAW_EMPTY + 8 * q, 4);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(sbase + BAR_TMEM_FULL + 8 * t, 1);     // tcgen05.commit
            mbar_init(sbase + BAR_TMEM_EMPTY + 8 * t, 8);    // one arrive per drain warp
        }
        mbar_init(sbase + BAR_G_FULL_S, 1);
        for (int j = 0; j < 4; ++j) mbar_init(sbase + BAR_G_FULL_M + 8 * j, 4);
        mbar_init(sbase + BAR_G_EMPTY, 1);                   // tcgen05.commit
        for (int t = 0; t < TABN; ++t) mbar_init(sbase + BAR_TAB_EMPTY + 8 * t, 8);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(sbase + OFF_TMEM_PTR), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + OFF_TMEM_PTR);
    const int n_tiles = tile_count(p);

    // Counters every role advances in the same order:
    //   it   64-k chunk counter, main-ring stage = it % STAGES
    //   sbc  super-block counter: TMEM buffer = sbc & 1, raw slot = sbc % RAW_STAGES, table slot = sbc % TABN
    //   gg   group counter: a group is up to four consecutive super-blocks of one tile, sharing one G operand tile;
    //        super-block j of its group uses the j-th 32-byte slice of the tile's 128-byte rows
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer: activation pieces ----------------
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                const int bk = box_bucket(tr.nt);
                const uint32_t bytes = static_cast<uint32_t>(16 << bk) * 128u * 2u;
                for (int kc = tr.sb0 * 4; kc < tr.sb1 * 4; ++kc, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort<false>(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_FULL_A + 8 * s, bytes);
                    tma_load_2d(sbase + OFF_AH + s * OP_TILE, &maps.a[bk], kc * BKC, tr.m0, sbase + BAR_FULL_A + 8 * s);
                    tma_load_2d(sbase + OFF_AL + s * OP_TILE, &maps.a[bk], kc * BKC, p.m_pad + tr.m0, sbase + BAR_FULL_A + 8 * s);
                }
            }
            if (!ok) {
                // tiles in flight must land before shared memory is released
                for (int k = 0; k < STAGES; ++k) {
                    const int v = it - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_FULL_A + 8 * (v % STAGES), (v / STAGES) & 1);
                }
            }
        } else if (warp == 3 && lane == 0) {
            // ---------------- TMA producer: packed weights (rows past N are zero-filled: d = 0, every scale 0),
            // and per group the g operand tile. The latter is asked for after the raw tile of the group's second
            // super-block, so that waiting for the previous group's G products never delays a weight copy.
            int sbc = 0, gg = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                const int bk = box_bucket(tr.nt);
                for (int sb = tr.sb0; sb < tr.sb1; ++sb, ++sbc) {
                    const int q = sbc % RAW_STAGES;
                    if (!wait_or_abort<false>(sbase + BAR_RAW_EMPTY + 8 * q, ((sbc / RAW_STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_RAW_FULL + 8 * q, RAW_TILE);
                    tma_load_2d(sbase + OFF_RAW + q * RAW_TILE, &maps.w, sb * Q4_K_BYTES, tr.wrow0 + tr.n0, sbase + BAR_RAW_FULL + 8 * q);
                    const int j = (sb - tr.sb0) & 3;
                    const int group_size = tr.sb1 - (sb - j) < 4 ? tr.sb1 - (sb - j) : 4;
                    if (j == (group_size > 1 ? 1 : 0)) {
                        if (!wait_or_abort<false>(sbase + BAR_G_EMPTY, (gg & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                        mbar_expect_tx(sbase + BAR_G_FULL_S, static_cast<uint32_t>(16 << bk) * 128u);
                        tma_load_2d(sbase + OFF_GS, &maps.g[bk], (sb - j) * 16, tr.m0, sbase + BAR_G_FULL_S);
                        ++gg;
                    }
                }
            }
            if (!ok) {
                for (int k = 0; k < RAW_STAGES; ++k) {
                    const int v = sbc - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_RAW_FULL + 8 * (v % RAW_STAGES), (v / RAW_STAGES) & 1);
                }
                if (gg > 0) mbar_wait_bounded(sbase + BAR_G_FULL_S, (gg - 1) & 1);
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issue ----------------
            int it = 0, sbc = 0, gg = 0;
            uint32_t gpar = 0;                     // bit j: parity of the next completion of the j-th "mins written" barrier
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                const uint32_t idesc = idesc_f16_m128((tr.nt + 15) & ~15);
                for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                    const int b = sbc & 1, j = (sb - tr.sb0) & 3;
                    if (!wait_or_abort<true>(sbase + BAR_TMEM_EMPTY + 8 * b, ((sbc >> 1) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_TMEM)) { ok = false; break; }
                    fence_after();
                    const uint32_t f_tmem = tmem_base + TM_F + b * TT, g_tmem = tmem_base + TM_G + b * TT;
                    for (int c = 0; c < 4; ++c, ++it) {
                        const int s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!wait_or_abort<true>(sbase + BAR_FULL_A + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                            !wait_or_abort<true>(sbase + BAR_FULL_W + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                        fence_after();
                        const uint64_t wdesc = smem_desc_sw128(sbase + OFF_W + s * OP_TILE);
                        const uint64_t hdesc = smem_desc_sw128(sbase + OFF_AH + s * OP_TILE);
                        const uint64_t ldesc = smem_desc_sw128(sbase + OFF_AL + s * OP_TILE);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t off = static_cast<uint64_t>(ks * 2);      // 32 bytes >> 4 inside the swizzle row
                            mma_f16(f_tmem, wdesc + off, hdesc + off, idesc, (c | ks) != 0);
                            mma_f16(f_tmem, wdesc + off, ldesc + off, idesc, 1);
                        }
                        commit(sbase + BAR_EMPTY + 8 * s);                  // operands consumed -> producers
                    }
                    if (!ok) break;
                    // G of this super-block: one K = 16 step on the j-th slice of the group's operand tiles
                    if ((j == 0 && !wait_or_abort<true>(sbase + BAR_G_FULL_S, gg & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) ||
                        !wait_or_abort<true>(sbase + BAR_G_FULL_M + 8 * j, (gpar >> j) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                    gpar ^= 1u << j;
                    fence_after();
                    mma_f16(g_tmem, smem_desc_sw128(sbase + OFF_GM) + static_cast<uint64_t>(j * 2),
                            smem_desc_sw128(sbase + OFF_GS) + static_cast<uint64_t>(j * 2), idesc, 0);
                    commit(sbase + BAR_TMEM_FULL + 8 * b);                  // F and G of the super-block complete -> drain
                    if (j == 3 || sb == tr.sb1 - 1) { commit(sbase + BAR_G_EMPTY); ++gg; }      // the group's G operands are consumed
                }
            }
        }
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
        // ---------------- converters: thread r owns weight row n0 + r ----------------
        const int r = threadIdx.x - 128;
        int it = 0, sbc = 0, gg = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const TileRef tr = tile_ref(p, tile);
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                const int q = sbc % RAW_STAGES, slot = sbc % TABN, j = (sb - tr.sb0) & 3;
                const uint32_t raw = sbase + OFF_RAW + q * RAW_TILE + r * Q4_K_BYTES;      // this row's 144 bytes
                if (!wait_or_abort<false>(sbase + BAR_RAW_FULL + 8 * q, (sbc / RAW_STAGES) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                const uint4 hdr = lds128(raw);
                // 6-bit scales / mins, eight of each (Laplace src/kernels.h:82-90), one per byte
                const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, mn_lo = hdr.z & 0x3f3f3f3fu;
                const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
                const uint32_t mn_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
                if (!wait_or_abort<false>(sbase + BAR_TAB_EMPTY + 8 * slot, ((sbc / TABN) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                reinterpret_cast<float2*>(smem + OFF_TAB)[slot * TW + r] =
                    make_float2(half_bits_to_float(hdr.x), -64.0f * half_bits_to_float(hdr.x >> 16));
#pragma unroll
                for (int c = 0; c < 4; ++c, ++it) {
                    const uint4 qa = lds128(raw + 16 + 32 * c), qb = lds128(raw + 32 + 32 * c);
                    const int s = it % STAGES;
                    if (!wait_or_abort<false>(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    const uint32_t scw = c < 2 ? sc_lo : sc_hi;
                    const uint32_t sc1 = (scw >> (16 * (c & 1))) & 0xff, sc2 = (scw >> (16 * (c & 1) + 8)) & 0xff;
                    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    // fp16 operand row: 32 low-nibble values * sc1, then 32 high-nibble values * sc2.
                    // Within every 4 values the order is (0, 2, 1, 3); the activation operand uses the same order.
                    // (v | 0x6400) is fp16(1024 + v); one fused multiply-add turns it into v * sc exactly:
                    // (1024 + v) * sc - 1024 * sc. High nibbles stay in place as 16 v and use sc / 16.
                    const __half2 s1 = __half2half2(__ushort2half_rn(static_cast<unsigned short>(sc1)));
                    const __half2 s2 = __half2half2(__hmul(__ushort2half_rn(static_cast<unsigned short>(sc2)), __float2half_rn(0.0625f)));
                    const __half2 o1 = __hmul2(s1, __half2half2(__float2half_rn(-1024.f)));
                    const __half2 o2 = __hmul2(s2, __half2half2(__float2half_rn(-1024.f)));
                    uint32_t h[32];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t w = qw[i], t = w >> 8;
                        const uint32_t a0 = (w & 0x000f000fu) | 0x64006400u, a1 = (t & 0x000f000fu) | 0x64006400u;
                        const uint32_t b0 = (w & 0x00f000f0u) | 0x64006400u, b1 = (t & 0x00f000f0u) | 0x64006400u;
                        __half2 x;
                        x = __hfma2(*reinterpret_cast<const __half2*>(&a0), s1, o1); h[2 * i] = *reinterpret_cast<uint32_t*>(&x);
                        x = __hfma2(*reinterpret_cast<const __half2*>(&a1), s1, o1); h[2 * i + 1] = *reinterpret_cast<uint32_t*>(&x);
                        x = __hfma2(*reinterpret_cast<const __half2*>(&b0), s2, o2); h[16 + 2 * i] = *reinterpret_cast<uint32_t*>(&x);
                        x = __hfma2(*reinterpret_cast<const __half2*>(&b1), s2, o2); h[16 + 2 * i + 1] = *reinterpret_cast<uint32_t*>(&x);
                    }
                    uint8_t* wrow = smem + OFF_W + s * OP_TILE + r * 128;
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj)
                        *reinterpret_cast<uint4*>(wrow + ((jj ^ (r & 7)) << 4)) = make_uint4(h[4 * jj], h[4 * jj + 1], h[4 * jj + 2], h[4 * jj + 3]);
                    fence_proxy_async();          // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + BAR_FULL_W + 8 * s);
                }
                if (!ok) break;
                // the packed super-block has been read: its slot may be refilled
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + BAR_RAW_EMPTY + 8 * q);
                // G operand, written last so that the wait for the previous group's products is short: k = 2 jj + piece
                // -> mn_jj as fp16 (exact), 16 values = the j-th 32-byte slice of this row
                if (j == 0) {
                    if (!wait_or_abort<false>(sbase + BAR_G_EMPTY, (gg & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                }
                {
                    uint32_t gw[8];
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                        const uint32_t mw = jj < 4 ? mn_lo : mn_hi;
                        const __half hv = __ushort2half_rn(static_cast<unsigned short>((mw >> (8 * (jj & 3))) & 0xff));
                        const uint32_t hb = __half_as_ushort(hv);
                        gw[jj] = hb | (hb << 16);
                    }
                    uint8_t* grow = smem + OFF_GM + r * 128;
                    *reinterpret_cast<uint4*>(grow + (((2 * j) ^ (r & 7)) << 4)) = make_uint4(gw[0], gw[1], gw[2], gw[3]);
                    *reinterpret_cast<uint4*>(grow + (((2 * j + 1) ^ (r & 7)) << 4)) = make_uint4(gw[4], gw[5], gw[6], gw[7]);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + BAR_G_FULL_M + 8 * j);
                }
                if (j == 3 || sb == tr.sb1 - 1) ++gg;
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        // ---------------- drain: lane = weight row (output column), 64 token columns per warp ----------------
        const int e8 = warp - 8;
        const int quad = e8 & 3, half = e8 >> 2;
        const uint32_t t_lane = static_cast<uint32_t>(quad * 32) << 16;
        const int wr = quad * 32 + lane;                 // weight row inside the tile
        int sbc = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const TileRef tr = tile_ref(p, tile);
            float acc[64];
#pragma unroll
            for (int c = 0; c < 64; ++c) acc[c] = 0.f;
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                const int b = sbc & 1, slot = sbc % TABN;
                if (!wait_or_abort<false>(sbase + BAR_TMEM_FULL + 8 * b, (sbc >> 1) & 1, abort_flag, p.err, DEV_TIMEOUT_MMA)) { ok = false; break; }
                fence_after();
                const float2 dm = reinterpret_cast<const float2*>(smem + OFF_TAB)[slot * TW + wr];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (half * 64 + h * 32 < tr.nt) {                  // warp-uniform: columns past the tile's tokens hold nothing
                        float f[32], g[32];
                        ld32(tmem_base + t_lane + TM_F + b * TT + half * 64 + h * 32, f);
                        ld32(tmem_base + t_lane + TM_G + b * TT + half * 64 + h * 32, g);
                        wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) acc[h * 32 + c] = fmaf(dm.y, g[c], fmaf(dm.x, f[c], acc[h * 32 + c]));
                    }
                }
                // F, G and the table entry are in registers: the MMA and the converters may reuse them
                fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(sbase + BAR_TMEM_EMPTY + 8 * b);
                    mbar_arrive(sbase + BAR_TAB_EMPTY + 8 * slot);
                }
            }
            if (!ok) break;
            // y[token][n] = 2^-e_token * acc: for a fixed token the warp's 32 lanes write 32 consecutive floats
            const int n = tr.n0 + wr;
            float* ybase = p.ksplit > 1 ? p.y_part + static_cast<size_t>(tr.ks) * p.M * p.N : p.y;
            if (n < p.N) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int col = half * 64 + c;
                    if (col < tr.nt) {
                        const int row = tr.m0 + col;
                        int orow = p.out_row ? __ldg(p.out_row + row) : row;
                        if (p.out_identity && orow >= 0) orow = row;
                        if (orow >= 0) ybase[static_cast<size_t>(orow) * p.N + n] = acc[c] * __ldg(p.inv_s + row);
                    }
                }
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- activation quantizer ------------------------------------------------------------------
// One CTA per activation row. The int8 values q and the block scales d are the reference's (Laplace
// src/matmul_simd.cpp:348-410: d = amax / 127, q = rne(x * (1 / d)), sums from the unclamped integers); what is
// written is the tensor-core operand built from them:
//   hi, lo [k]      fp16 pieces of 2^e * (d * q[k]), e chosen so that the row's largest |x| lands in [2^13, 2^14);
//                   within every four consecutive k the order is (0, 2, 1, 3), like the weight operand
//   g [16 sb + 2 j + piece]   fp16 pieces of 2^e / 64 * (d * integer sum) of block 8 sb + j
//   inv_s           2^-e
// `load(b, t8)` returns values 4 t8 .. 4 t8 + 3 of block b of the row. The row is read twice (maximum, then
// quantization); the second read hits L1 / L2.
template <class Load>
__device__ __forceinline__ void quantize_row_sa(Load load, int K, __half* __restrict__ hi_row, __half* __restrict__ lo_row,
                                                __half* __restrict__ g_row, float* __restrict__ inv_s) {
    __shared__ float red[8];
    const int bpr = K / 32, grp = threadIdx.x >> 3, t8 = threadIdx.x & 7, groups = blockDim.x >> 3;
    float amax = 0.f;
    for (int b = grp; b < bpr; b += groups) {
        const float4 v = load(b, t8);
        amax = max_nan(amax, max_nan(max_nan(fabsf(v.x), fabsf(v.y)), max_nan(fabsf(v.z), fabsf(v.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) amax = max_nan(amax, red[w]);
    // 2^e with e = 13 - floor(log2(amax)), as exponent-field arithmetic; rows of zeros, infinities or NaN use 1
    const int ex = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);
    int field = 267 - ex;
    if (ex == 0 || ex == 255) field = 127;
    field = field < 1 ? 1 : (field > 253 ? 253 : field);
    const float s = __uint_as_float(static_cast<uint32_t>(field) << 23);
    const float gs = s * 0.015625f;
    if (threadIdx.x == 0) *inv_s = __uint_as_float(static_cast<uint32_t>(254 - field) << 23);
    const int iters = (bpr + groups - 1) / groups;
    for (int itn = 0; itn < iters; ++itn) {                    // whole warps iterate together: the 8-lane shuffles stay converged
        const int b = grp + itn * groups;
        const bool live = b < bpr;
        const float4 v = live ? load(b, t8) : make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t packed; int hs;
        const float d = quantize_block_8lanes(v, packed, hs);
        const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
        if (!live) continue;
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            a[i] = __fmul_rn(__fmul_rn(d, static_cast<float>(static_cast<int8_t>((packed >> (8 * i)) & 0xff))), s);
        __half h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            h[i] = __float2half_rn(a[i]);
            l[i] = __float2half_rn(a[i] - __half2float(h[i]));
        }
        const __half2 h02 = __halves2half2(h[0], h[2]), h13 = __halves2half2(h[1], h[3]);
        const __half2 l02 = __halves2half2(l[0], l[2]), l13 = __halves2half2(l[1], l[3]);
        uint2 oh, ol;
        oh.x = *reinterpret_cast<const uint32_t*>(&h02); oh.y = *reinterpret_cast<const uint32_t*>(&h13);
        ol.x = *reinterpret_cast<const uint32_t*>(&l02); ol.y = *reinterpret_cast<const uint32_t*>(&l13);
        reinterpret_cast<uint2*>(hi_row + b * 32)[t8] = oh;
        reinterpret_cast<uint2*>(lo_row + b * 32)[t8] = ol;
        if (t8 == 0) {
            const short slo = static_cast<short>(hs), shi = static_cast<short>(hs_hi);
            const float sum = __fmul_rn(d, static_cast<float>(static_cast<int>(slo) + static_cast<int>(shi)));
            const float gv = __fmul_rn(sum, gs);
            const __half gh = __float2half_rn(gv);
            const __half gl = __float2half_rn(gv - __half2float(gh));
            reinterpret_cast<__half2*>(g_row)[b] = __halves2half2(gh, gl);        // element 16 (b / 8) + 2 (b % 8) + piece = 2 b + piece
        }
    }
}

struct SaOperand {          // operand buffers of one matmul
    __half* a;              // [2][m_pad][K]: hi rows, then lo rows
    __half* g;              // [m_pad][K / 16]
    float*  inv_s;          // [m_pad]
    int     m_pad;
};

__global__ void __launch_bounds__(256) quantize_sa_kernel(const float* __restrict__ x, int K, SaOperand op) {
    const int m = blockIdx.x;
    const float* xr = x + static_cast<size_t>(m) * K;
    quantize_row_sa([&](int b, int t8) { return __ldg(reinterpret_cast<const float4*>(xr + b * 32) + t8); }, K,
                    op.a + static_cast<size_t>(m) * K, op.a + (static_cast<size_t>(op.m_pad) + m) * K,
                    op.g + static_cast<size_t>(m) * (K / 16), op.inv_s + m);
}

// y = sum of the k-slices' partial results, slices added in index order.
__global__ void __launch_bounds__(256) splitk_reduce_sa_kernel(const float4* __restrict__ part, long long n4, int ksplit,
                                                               float4* __restrict__ y) {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float4 a = __ldg(part + i);
        for (int k = 1; k < ksplit; ++k) {
            const float4 b = __ldg(part + static_cast<long long>(k) * n4 + i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        y[i] = a;
    }
}

inline size_t align256(size_t n) { return (n + 255) & ~size_t(255); }

// Scratch owned by this translation unit. A buffer that has been handed to a launch may be baked into a captured
// CUDA graph (its address and the tensor maps built from it), so a buffer is never freed when a larger one is
// needed: superseded buffers are kept until laplace_cuda_shutdown. Growing calls the allocator, which is illegal
// while the call's stream is being captured: such a call is refused and the capture stays valid.
struct Scratch {
    void*  p = nullptr;
    size_t cap = 0;
    std::vector<void*> retired;
    int ensure(size_t n, cudaStream_t st) {
        if (n <= cap) return LAPLACE_OK;
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone)
            return fail(LAPLACE_ERR_STATE, "the call needs %zu bytes of scratch but only %zu are allocated, and its stream is being "
                                           "captured: make the same call once before the capture begins", n, cap);
        if (p) retired.push_back(p);
        p = nullptr; cap = 0;
        cudaError_t e = cudaMalloc(&p, n + n / 8);
        if (e != cudaSuccess) return cuda_check(e, "cudaMalloc scratch");
        cap = n + n / 8;
        return LAPLACE_OK;
    }
    void release() {
        if (p) cudaFree(p);
        for (void* q : retired) cudaFree(q);
        retired.clear();
        p = nullptr; cap = 0;
    }
};
Scratch g_scratch;

struct OperandBytes { size_t a, g, s; size_t total() const { return a + g + s; } };
OperandBytes operand_bytes(size_t m_pad, int K) {
    return {align256(2 * m_pad * K * sizeof(__half)), align256(m_pad * (K / 16) * sizeof(__half)), align256(m_pad * sizeof(float))};
}
SaOperand carve_operand(uint8_t*& s, size_t m_pad, int K) {
    const OperandBytes ob = operand_bytes(m_pad, K);
    SaOperand op;
    op.a = reinterpret_cast<__half*>(s);      s += ob.a;
    op.g = reinterpret_cast<__half*>(s);      s += ob.g;
    op.inv_s = reinterpret_cast<float*>(s);   s += ob.s;
    op.m_pad = static_cast<int>(m_pad);
    return op;
}

struct SaLaunch {
    const uint8_t* w; float* y; int M, K, N;
    long long w_rows;            // rows of the (stacked) weight matrix
    SaOperand op;
    const int4* tile_tab; const int* n_tiles_dev; const int* out_row; int out_identity;
    int tiles_m, tiles_n, grid;
    int ksplit, sb_per; float* y_part;
};

int run_sa_kernel(const SaLaunch& L, cudaStream_t st) {
    Context& c = ctx();
    const int K = L.K;
    SaMaps maps;
    for (int bk = 0; bk < 4; ++bk) {
        if (!make_map_2d(&maps.a[bk], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, L.op.a, static_cast<uint64_t>(K), 2ull * L.op.m_pad,
                         static_cast<uint64_t>(K) * 2, BKC, 16u << bk, CU_TENSOR_MAP_SWIZZLE_128B, "activations") ||
            !make_map_2d(&maps.g[bk], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, L.op.g, static_cast<uint64_t>(K / 16), static_cast<uint64_t>(L.op.m_pad),
                         static_cast<uint64_t>(K / 16) * 2, 64, 16u << bk, CU_TENSOR_MAP_SWIZZLE_128B, "g operand"))
            return LAPLACE_ERR_CUDA;
    }
    const uint64_t rb = row_bytes(LAPLACE_TYPE_Q4_K, K);
    if (!make_map_2d(&maps.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, L.w, rb, static_cast<uint64_t>(L.w_rows), rb, Q4_K_BYTES, TW,
                     CU_TENSOR_MAP_SWIZZLE_NONE, "weights"))
        return LAPLACE_ERR_CUDA;
    SaParams p{};
    p.y = L.y; p.inv_s = L.op.inv_s; p.err = c.d_err;
    p.M = L.M; p.N = L.N; p.K = K; p.m_pad = L.op.m_pad;
    p.tiles_m = L.tiles_m; p.tiles_n = L.tiles_n;
    p.tile_tab = L.tile_tab; p.n_tiles_dev = L.n_tiles_dev; p.out_row = L.out_row; p.out_identity = L.out_identity;
    p.ksplit = L.ksplit > 1 ? L.ksplit : 1; p.sb_per = L.ksplit > 1 ? L.sb_per : K / 256; p.y_part = L.y_part;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_q4k_sa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
        if (e != cudaSuccess) return cuda_check(e, "cudaFuncSetAttribute gemm_sa");
        configured = true;
    }
    gemm_q4k_sa_kernel<<<L.grid, THREADS, SMEM_BYTES, st>>>(maps, p);
    c.launches++;
    c.last_path = 2;
    return cuda_check(cudaGetLastError(), "gemm_sa launch");
}

// Split-K plan for a dense call with few output tiles: up to four CTAs share a tile, each over a multiple of four
// super-blocks (one G operand group).
struct SplitPlan { int ksplit, sb_per; };
SplitPlan plan_split(int M, int K, int N, bool allow) {
    const int nsb = K / 256, tiles = ((M + TT - 1) / TT) * ((N + TW - 1) / TW), sms = ctx().sm_count;
    SplitPlan s{1, nsb};
    if (!allow || nsb < 8 || tiles * 2 > sms) return s;
    double best = static_cast<double>((tiles + sms - 1) / sms) * nsb;
    for (int want = 2; want <= 4; ++want) {
        int per = (nsb + want - 1) / want;
        per = (per + 3) & ~3;
        const int ks = (nsb + per - 1) / per;
        if (ks < 2) continue;
        const double waves = static_cast<double>((static_cast<long long>(tiles) * ks + sms - 1) / sms);
        // cost in super-blocks of one tile (~1.2 us each); the reduction moves (slices + 1) x M x N floats
        const double cost = waves * per + static_cast<double>(ks + 1) * M * N * 4.0 / 6.0e6 / 1.2 + 0.5;
        if (cost < best * 0.97) { best = cost; s.ksplit = ks; s.sb_per = per; }
    }
    return s;
}

}  // namespace

void release_gemm_sa_scratch() { g_scratch.release(); }

bool gemm_sa_supports(uint32_t type, int M, int K, int N) {
    return type == LAPLACE_TYPE_Q4_K && M > 8 && N > 0 && K > 0 && K % 256 == 0;
}

namespace {

struct SaPlan {
    int tiles_m, tiles_n;
    size_t m_pad;
    SplitPlan sp;
    size_t op_bytes, part_bytes;
    size_t total() const { return op_bytes + part_bytes; }
};
SaPlan plan_sa(int M, int K, int N, bool allow_split) {
    SaPlan pl;
    pl.tiles_m = (M + TT - 1) / TT;
    pl.tiles_n = (N + TW - 1) / TW;
    pl.m_pad = static_cast<size_t>(pl.tiles_m) * TT;
    pl.sp = plan_split(M, K, N, allow_split);
    pl.op_bytes = operand_bytes(pl.m_pad, K).total();
    pl.part_bytes = pl.sp.ksplit > 1 ? align256(static_cast<size_t>(pl.sp.ksplit) * M * N * sizeof(float)) : 0;
    return pl;
}

int check_args(const float* x, const uint8_t* w, uint32_t type, int M, int K, int N) {
    if (!gemm_sa_supports(type, M, K, N)) return LAPLACE_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(w) & 15) return fail(LAPLACE_ERR_ARG, "gemm: weights must be 16-byte aligned on the device");
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(LAPLACE_ERR_ARG, "gemm: x not 16-byte aligned");
    return LAPLACE_OK;
}

// Quantizes x into `scratch` (device memory of at least pl.total() bytes, 256-byte aligned) and runs the kernel.
int gemm_sa_on_scratch(uint8_t* scratch, const SaPlan& pl, const float* x, const uint8_t* w, float* y, int M, int K, int N,
                       cudaStream_t st) {
    Context& c = ctx();
    int rc;
    uint8_t* s = scratch;
    const SaOperand op = carve_operand(s, pl.m_pad, K);
    quantize_sa_kernel<<<M, 256, 0, st>>>(x, K, op);
    c.launches++;
    if ((rc = cuda_check(cudaGetLastError(), "quantize_sa launch"))) return rc;
    SaLaunch L{};
    L.w = w; L.y = y; L.M = M; L.K = K; L.N = N; L.w_rows = N; L.op = op;
    L.tiles_m = pl.tiles_m; L.tiles_n = pl.tiles_n;
    L.ksplit = pl.sp.ksplit; L.sb_per = pl.sp.sb_per;
    L.y_part = pl.sp.ksplit > 1 ? reinterpret_cast<float*>(s) : nullptr;
    const int n_tiles = pl.tiles_m * pl.tiles_n * pl.sp.ksplit;
    L.grid = n_tiles < c.sm_count ? n_tiles : c.sm_count;
    if ((rc = run_sa_kernel(L, st))) return rc;
    if (pl.sp.ksplit > 1) {
        const long long n4 = static_cast<long long>(M) * N / 4;
        long long blocks = (n4 + 255) / 256;
        if (blocks > static_cast<long long>(c.sm_count) * 8) blocks = static_cast<long long>(c.sm_count) * 8;
        splitk_reduce_sa_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(reinterpret_cast<const float4*>(L.y_part), n4, pl.sp.ksplit,
                                                                        reinterpret_cast<float4*>(y));
        c.launches++;
        return cuda_check(cudaGetLastError(), "splitk_reduce launch");
    }
    return LAPLACE_OK;
}

// split-K only when its partial results can be added up with vector loads
bool can_split(const float* y, int M, int N) {
    return (static_cast<long long>(M) * N) % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
}

}  // namespace

int launch_gemm_sa(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, cudaStream_t st) {
    int rc = check_args(x, w, type, M, K, N);
    if (rc) return rc;
    const SaPlan pl = plan_sa(M, K, N, can_split(y, M, N));
    if ((rc = g_scratch.ensure(pl.total(), st))) return rc;
    return gemm_sa_on_scratch(static_cast<uint8_t*>(g_scratch.p), pl, x, w, y, M, K, N, st);
}

// The same call on scratch memory the caller owns (`cap` bytes at `scratch`, 256-byte aligned); nothing is
// allocated. The K-split of launch_gemm_sa is kept when its partial results fit too (the result is then
// bit-identical to launch_gemm_sa's), otherwise the call runs unsplit.
int launch_gemm_sa_prealloc(uint8_t* scratch, size_t cap, const float* x, const uint8_t* w, uint32_t type, float* y,
                            int M, int K, int N, cudaStream_t st) {
    int rc = check_args(x, w, type, M, K, N);
    if (rc) return rc;
    SaPlan pl = plan_sa(M, K, N, can_split(y, M, N));
    if (pl.total() > cap) pl = plan_sa(M, K, N, false);
    if (pl.total() > cap)
        return fail(LAPLACE_ERR_LIMIT, "gemm: M=%d K=%d needs %zu bytes of scratch, the caller's area holds %zu", M, K, pl.total(), cap);
    return gemm_sa_on_scratch(scratch, pl, x, w, y, M, K, N, st);
}

}  // namespace lp
