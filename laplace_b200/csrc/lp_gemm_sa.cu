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
// weight operand is sc * nibble <= 945, exact in fp16. The tensor core accumulates, in fp32, a whole super-block
// (256 values) per drain:
//   F_hi[n,m], F_lo[n,m] = sum_{k in sb} (sc*nibble)[n,k] * hi[m,k], ... * lo[m,k]        (tcgen05.mma kind::f16)
//   y[m,n] += 2^-e_m * ( d[n,sb] * (F_hi + F_lo) - sum_{j<8} (dmin * mn_j)[n,sb] * g[m,8sb+j] ),   g = 2^e_m * sum_x
// on CUDA cores once per super-block; the min term is the reference's own fp32 arithmetic. Products are exact;
// what is rounded is the split of a (2^-22 relative) and the fp32 accumulation, which the reference also does in fp32
// in another order. Integer block sums are still exact whenever the activations are: a block whose scale is a power
// of two gives lo = 0 and an exact hi, hence an exact integer times the scale.
//
// Roles of the operands: WEIGHT rows sit on the MMA's M side (128 TMEM lanes), TOKENS on its N side, the lo piece
// stacked behind the hi piece (up to 2 x 128 columns), so a tile with few tokens - an expert of a mixture-of-experts
// layer with 16 tokens - costs a proportionally short MMA, the per-super-block weight scales are per-lane scalars in
// the drain, and each 16-value step is ONE instruction: a single thread issues a tcgen05.mma about every 115 cycles
// however small it is, so few wide instructions beat many narrow ones.
//
// One 512-thread CTA per SM, persistent over tiles of 128 weight rows x up to 128 tokens:
//   warp 0      TMA: activation operand tiles (hi and lo piece, 64 k x tokens, 128-byte swizzle)
//   warp 1      MMA issue (one lane); owns the TMEM allocation
//   warp 3      TMA: packed Q4_K super-blocks (128 rows x 144 bytes) and the tiles of activation block sums
//   warps 4-7   converters: packed super-block -> fp16 weight operand tile (thread = weight row), and the row's
//               d and dmin * mn_j into a table for the drain
//   warps 8-15  drain: tcgen05.ld of the accumulator (double buffered in TMEM) once per super-block, running y in
//               registers
// All mbarrier waits are bounded; a wait that gives up raises the status word and every role leaves its loop.
#include <cuda_fp16.h>

#include <vector>

#include "lp_tc.cuh"

namespace lp {

namespace {

using namespace tc;

constexpr int TW = 128;                            // weight rows per tile (MMA M)
constexpr int TT = 128;                            // most tokens per tile
constexpr int BKC = 64;                            // k per pipeline stage
constexpr int STAGES = 3;
constexpr int RAW_STAGES = 2;
constexpr int RAW_TILE = TW * Q4_K_BYTES;          // 18 KB
constexpr int W_TILE = TW * BKC * 2;               // 16 KB: 128 rows of 64 fp16
constexpr int A_TILE = 2 * TT * BKC * 2;           // 32 KB: the hi rows, then the lo rows
constexpr int TABN = 4;                            // ring of per-super-block weight-scale tables and g tiles
constexpr int TAB_ROW = 12;                        // floats per weight row: d, -dmin*mn[0..7], 3 unused
constexpr int G_TILE = (TT / 2) * 16 * 4;          // 4 KB: per token pair 8 x (g[even token], g[odd token])
constexpr int THREADS = 512;
constexpr uint32_t TMEM_COLS = 512;                // two accumulators of 256 columns (hi | lo)

constexpr uint32_t OFF_W = 0;
constexpr uint32_t OFF_A = OFF_W + STAGES * W_TILE;
constexpr uint32_t OFF_RAW = OFF_A + STAGES * A_TILE;
constexpr uint32_t OFF_TAB = OFF_RAW + RAW_STAGES * RAW_TILE;
constexpr uint32_t OFF_G = OFF_TAB + TABN * TW * TAB_ROW * 4;
constexpr uint32_t OFF_BAR = OFF_G + TABN * G_TILE;
constexpr uint32_t BAR_FULL_A = OFF_BAR, BAR_FULL_W = BAR_FULL_A + 8 * STAGES, BAR_EMPTY = BAR_FULL_W + 8 * STAGES,
                   BAR_RAW_FULL = BAR_EMPTY + 8 * STAGES, BAR_RAW_EMPTY = BAR_RAW_FULL + 8 * RAW_STAGES,
                   BAR_TMEM_FULL = BAR_RAW_EMPTY + 8 * RAW_STAGES, BAR_TMEM_EMPTY = BAR_TMEM_FULL + 16,
                   BAR_G_FULL = BAR_TMEM_EMPTY + 16, BAR_TAB_EMPTY = BAR_G_FULL + 8 * TABN,
                   OFF_TMEM_PTR = BAR_TAB_EMPTY + 8 * TABN, OFF_ABORT = OFF_TMEM_PTR + 8;
constexpr uint32_t SMEM_BYTES = OFF_ABORT + 8 + 1024;       // + slack for the 1024-byte alignment
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(OFF_RAW % 128 == 0 && RAW_TILE % 128 == 0 && OFF_G % 128 == 0, "TMA destinations are 128-byte aligned");
static_assert(OFF_A % 1024 == 0 && A_TILE % 1024 == 0 && W_TILE % 1024 == 0, "swizzled tiles are 1024-byte aligned");

struct SaParams {
    const uint8_t* w;          // packed weights (the two-piece weight types copy rows by address)
    uint32_t     rb;           // bytes per weight row
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
    // Balanced split of a dense call: the work is the list of (output tile, super-block) units in tile order, and CTA c
    // takes units [c * units / grid, (c + 1) * units / grid). A tile whose units fall to more than one CTA is written as
    // partial results (slot 2c for the piece that continues a tile, 2c + 1 for the piece that begins one; a slot holds
    // [TT tokens][TW rows] floats) which a second kernel adds up in k order. 0 units: whole tiles, dealt round-robin.
    long long    sk_units;
    float*       y_part;
};

// Row-split over several GPUs: the tile goes to row-major [M][ld] buffers of EVERY GPU at column col0 + n (plain stores
// to peer-mapped memory; complete when the grid is) instead of to SaParams::y. A kernel parameter of its own that only
// the PEERS instantiations carry, so that the one-GPU kernels keep their parameter block and code as they were.
template <bool PEERS> struct SaPeers {};
template <> struct SaPeers<true> { float* y[MAX_PEERS]; int n, ld, col0; };

struct TileRef { int m0, n0, wrow0, nt, sb0, sb1, part; };     // nt = tokens of the tile; part = slot of a partial result or -1
// The pieces of work of one CTA, in the order every role of the CTA walks them.
struct Segments { int n; long long u0, u1; };
__host__ __device__ __forceinline__ long long sk_start(long long units, int grid, int c) { return units * c / grid; }
__device__ __forceinline__ Segments segments(const SaParams& p) {
    if (p.tile_tab || p.sk_units == 0) {
        const int n_tiles = p.tile_tab ? __ldg(p.n_tiles_dev) : p.tiles_m * p.tiles_n;
        const int b = static_cast<int>(blockIdx.x), g = static_cast<int>(gridDim.x);
        return {b < n_tiles ? (n_tiles - b + g - 1) / g : 0, 0, 0};
    }
    const int nsb = p.K / 256;
    const long long u0 = sk_start(p.sk_units, gridDim.x, blockIdx.x), u1 = sk_start(p.sk_units, gridDim.x, blockIdx.x + 1);
    return {u1 > u0 ? static_cast<int>((u1 - 1) / nsb - u0 / nsb) + 1 : 0, u0, u1};
}
__device__ __forceinline__ TileRef seg_ref(const SaParams& p, const Segments& sg, int i) {
    const int nsb = p.K / 256;
    if (p.tile_tab) {
        const int4 t = __ldg(p.tile_tab + blockIdx.x + i * gridDim.x);
        return {t.x, t.y, t.z, t.w, 0, nsb, -1};
    }
    int t, sb0 = 0, sb1 = nsb;
    if (p.sk_units == 0) {
        t = blockIdx.x + i * gridDim.x;
    } else {
        const int t_first = static_cast<int>(sg.u0 / nsb), t_last = static_cast<int>((sg.u1 - 1) / nsb);
        t = t_first + i;
        if (i == 0) sb0 = static_cast<int>(sg.u0 - static_cast<long long>(t_first) * nsb);
        if (t == t_last) sb1 = static_cast<int>(sg.u1 - 1 - static_cast<long long>(t_last) * nsb) + 1;
    }
    const int m0 = (t % p.tiles_m) * TT;
    const int part = (sb0 > 0 || sb1 < nsb) ? 2 * static_cast<int>(blockIdx.x) + (sb0 == 0 ? 1 : 0) : -1;
    return {m0, (t / p.tiles_m) * TW, 0, p.M - m0 < TT ? p.M - m0 : TT, sb0, sb1, part};
}
// Activation boxes come in four heights (16, 32, 64, 128 rows); a tile uses the smallest that holds its tokens.
// In shared memory and in TMEM the lo piece follows the hi piece at a distance of one box height.
__device__ __forceinline__ int box_bucket(int nt) { return nt <= 16 ? 0 : nt <= 32 ? 1 : nt <= 64 ? 2 : 3; }

struct SaMaps {
    CUtensorMap a[4];      // activation pieces, [2 * m_pad][K] fp16, boxes of 64 k x {16, 32, 64, 128} rows, 128-byte swizzle
    CUtensorMap g[4];      // block sums, [m_pad / 2][K/256 * 16] fp32, boxes of 16 x {8, 16, 32, 64} token pairs
    CUtensorMap w;         // packed weights as bytes, rows of K/256 * 144 bytes, boxes of 144 bytes x 128 rows
};

// PEERS: the result tile goes to every GPU's buffer (SaPeers) instead of y. A template parameter, not a run-time
// branch: these kernels are sensitive to their code size and layout (the peer stores as a branch inside the one-GPU kernel
// cost it 14 to 37 %).
template <bool PEERS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_q4k_sa_kernel(const __grid_constant__ SaMaps maps, const SaParams p, const SaPeers<PEERS> pe) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_ABORT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sbase + BAR_FULL_A + 8 * s, 2);        // one arrive per activation piece
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
        for (int t = 0; t < TABN; ++t) {
            mbar_init(sbase + BAR_G_FULL + 8 * t, 1);
            mbar_init(sbase + BAR_TAB_EMPTY + 8 * t, 8);
        }
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
    const Segments sg = segments(p);

    // Counters every role advances in the same order:
    //   it   64-k chunk counter, main-ring stage = it % STAGES
    //   sbc  super-block counter: accumulator = sbc & 1, raw slot = sbc % RAW_STAGES, table / g slot = sbc % TABN
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if ((warp == 0 || warp == 2) && lane == 0) {
            // ---------------- TMA producers: warp 0 copies the hi piece of the activations, warp 2 the lo piece.
            // (The copies one thread issues are served one after the other at some 20 bytes per clock; the copies of
            // two threads run side by side.) ----------------
            const int pc = warp >> 1;
            int it = 0;
            bool ok = true;
            for (int seg = 0; ok && seg < sg.n; ++seg) {
                const TileRef tr = seg_ref(p, sg, seg);
                const int bk = box_bucket(tr.nt);
                const uint32_t piece = static_cast<uint32_t>(16 << bk) * 128u;
                for (int kc = tr.sb0 * 4; kc < tr.sb1 * 4; ++kc, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort<false>(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_FULL_A + 8 * s, piece);
                    tma_load_2d(sbase + OFF_A + s * A_TILE + pc * piece, &maps.a[bk], kc * BKC, pc * p.m_pad + tr.m0, sbase + BAR_FULL_A + 8 * s);
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
            // ---------------- TMA producer: packed weights (rows past N are zero-filled: d = 0, every scale 0)
            // and, per super-block, the tile of activation block sums ----------------
            int sbc = 0;
            bool ok = true;
            for (int seg = 0; ok && seg < sg.n; ++seg) {
                const TileRef tr = seg_ref(p, sg, seg);
                const int bk = box_bucket(tr.nt);
                for (int sb = tr.sb0; sb < tr.sb1; ++sb, ++sbc) {
                    const int q = sbc % RAW_STAGES, slot = sbc % TABN;
                    if (!wait_or_abort<false>(sbase + BAR_RAW_EMPTY + 8 * q, ((sbc / RAW_STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_RAW_FULL + 8 * q, RAW_TILE);
                    tma_load_2d(sbase + OFF_RAW + q * RAW_TILE, &maps.w, sb * Q4_K_BYTES, tr.wrow0 + tr.n0, sbase + BAR_RAW_FULL + 8 * q);
                    if (!wait_or_abort<false>(sbase + BAR_TAB_EMPTY + 8 * slot, ((sbc / TABN) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_G_FULL + 8 * slot, static_cast<uint32_t>(8 << bk) * 64u);
                    tma_load_2d(sbase + OFF_G + slot * G_TILE, &maps.g[bk], sb * 16, tr.m0 >> 1, sbase + BAR_G_FULL + 8 * slot);
                }
            }
            if (!ok) {
                for (int k = 0; k < RAW_STAGES; ++k) {
                    const int v = sbc - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_RAW_FULL + 8 * (v % RAW_STAGES), (v / RAW_STAGES) & 1);
                }
                for (int k = 0; k < TABN; ++k) {
                    const int v = sbc - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_G_FULL + 8 * (v % TABN), (v / TABN) & 1);
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issue: per 16-value step one instruction over the stacked pieces, D columns
            // [0, nt) = weights x hi, [box, box + nt) = weights x lo. (One thread issues an instruction roughly every
            // 115 cycles however small it is, so one wide instruction beats two narrow ones.) ----------------
            int it = 0, sbc = 0;
            bool ok = true;
            for (int seg = 0; ok && seg < sg.n; ++seg) {
                const TileRef tr = seg_ref(p, sg, seg);
                const uint32_t idesc = idesc_f16_m128((16 << box_bucket(tr.nt)) + ((tr.nt + 15) & ~15));
                for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                    const int b = sbc & 1;
                    if (!wait_or_abort<true>(sbase + BAR_TMEM_EMPTY + 8 * b, ((sbc >> 1) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_TMEM)) { ok = false; break; }
                    fence_after();
                    const uint32_t f_tmem = tmem_base + b * 256;
                    for (int c = 0; c < 4; ++c, ++it) {
                        const int s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!wait_or_abort<true>(sbase + BAR_FULL_A + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                            !wait_or_abort<true>(sbase + BAR_FULL_W + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                        fence_after();
                        const uint64_t wdesc = smem_desc_sw128(sbase + OFF_W + s * W_TILE);
                        const uint64_t adesc = smem_desc_sw128(sbase + OFF_A + s * A_TILE);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t off = static_cast<uint64_t>(ks * 2);      // 32 bytes >> 4 inside the swizzle row
                            mma_f16(f_tmem, wdesc + off, adesc + off, idesc, (c | ks) != 0);
                        }
                        commit(sbase + BAR_EMPTY + 8 * s);                  // operands consumed -> producers
                    }
                    if (!ok) break;
                    commit(sbase + BAR_TMEM_FULL + 8 * b);                  // the super-block's products are complete -> drain
                }
            }
        }
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
        // ---------------- converters: thread r owns weight row n0 + r ----------------
        const int r = threadIdx.x - 128;
        int it = 0, sbc = 0;
        bool ok = true;
        for (int seg = 0; ok && seg < sg.n; ++seg) {
            const TileRef tr = seg_ref(p, sg, seg);
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                const int q = sbc % RAW_STAGES, slot = sbc % TABN;
                const uint32_t raw = sbase + OFF_RAW + q * RAW_TILE + r * Q4_K_BYTES;      // this row's 144 bytes
                if (!wait_or_abort<false>(sbase + BAR_RAW_FULL + 8 * q, (sbc / RAW_STAGES) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                const uint4 hdr = lds128(raw);
                // 6-bit scales / mins, eight of each (Laplace src/kernels.h:82-90), one per byte
                const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, mn_lo = hdr.z & 0x3f3f3f3fu;
                const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
                const uint32_t mn_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
                if (!wait_or_abort<false>(sbase + BAR_TAB_EMPTY + 8 * slot, ((sbc / TABN) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                {
                    // the row's scales for the drain: d, and -dmin * mn_j (exact in fp32, as the reference forms them)
                    const float d = half_bits_to_float(hdr.x), ndmin = -half_bits_to_float(hdr.x >> 16);
                    float4* trow = reinterpret_cast<float4*>(smem + OFF_TAB + (slot * TW + r) * (TAB_ROW * 4));
                    trow[0] = make_float4(d, ndmin * static_cast<float>(mn_lo & 0xff), ndmin * static_cast<float>((mn_lo >> 8) & 0xff),
                                          ndmin * static_cast<float>((mn_lo >> 16) & 0xff));
                    trow[1] = make_float4(ndmin * static_cast<float>(mn_lo >> 24), ndmin * static_cast<float>(mn_hi & 0xff),
                                          ndmin * static_cast<float>((mn_hi >> 8) & 0xff), ndmin * static_cast<float>((mn_hi >> 16) & 0xff));
                    trow[2] = make_float4(ndmin * static_cast<float>(mn_hi >> 24), 0.f, 0.f, 0.f);
                }
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
                    uint8_t* wrow = smem + OFF_W + s * W_TILE + r * 128;
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
            }
        }
    } else {
        // (register budget of the CTA: 4 x 40 + 4 x 104 + 8 x 184 <= 16 x 128 per lane; a sum above what the CTA was
        // launched with would leave setmaxnreg.inc waiting for registers that never come)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        // ---------------- drain: lane = weight row (output column), 64 token columns per warp ----------------
        // Once per super-block: y += d * (F_hi + F_lo) + sum_j (-dmin mn_j) * g_j, two token columns per packed
        // instruction. The min term is the reference's own fp32 arithmetic (src/matmul_simd.cpp:263-279:
        // acc_min += (dmin * m) * sum_x), not a tensor-core product.
        const int e8 = warp - 8;
        const int quad = e8 & 3, half = e8 >> 2;
        const uint32_t t_lane = static_cast<uint32_t>(quad * 32) << 16;
        const int wr = quad * 32 + lane;                 // weight row inside the tile
        int sbc = 0;
        bool ok = true;
        for (int seg = 0; ok && seg < sg.n; ++seg) {
            const TileRef tr = seg_ref(p, sg, seg);
            const int box = 16 << box_bucket(tr.nt);
            float2 acc[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = make_float2(0.f, 0.f);
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                const int b = sbc & 1, slot = sbc % TABN;
                if (!wait_or_abort<false>(sbase + BAR_TMEM_FULL + 8 * b, (sbc >> 1) & 1, abort_flag, p.err, DEV_TIMEOUT_MMA) ||
                    !wait_or_abort<false>(sbase + BAR_G_FULL + 8 * slot, (sbc / TABN) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                fence_after();
                const uint32_t trow = sbase + OFF_TAB + (slot * TW + wr) * (TAB_ROW * 4);
                const uint4 t0 = lds128(trow), t1 = lds128(trow + 16);
                const float dm8 = __uint_as_float(lds32(trow + 32));
                const float2 dd = make_float2(__uint_as_float(t0.x), __uint_as_float(t0.x));
                const float dm[8] = {__uint_as_float(t0.y), __uint_as_float(t0.z), __uint_as_float(t0.w), __uint_as_float(t1.x),
                                     __uint_as_float(t1.y), __uint_as_float(t1.z), __uint_as_float(t1.w), dm8};
                const uint32_t gbase = sbase + OFF_G + slot * G_TILE + half * 32 * 64;      // this warp's 32 token pairs
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (half * 64 + h * 32 < tr.nt) {                  // warp-uniform: columns past the tile's tokens hold nothing
                        float fh[32], fl[32];
                        ld32(tmem_base + t_lane + b * 256 + half * 64 + h * 32, fh);
                        ld32(tmem_base + t_lane + b * 256 + box + half * 64 + h * 32, fl);
                        wait_ld();
                        if (h == 1 || half * 64 + 32 >= tr.nt) {
                            // the accumulator is in registers: the MMA may overwrite it
                            fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(sbase + BAR_TMEM_EMPTY + 8 * b);
                        }
#pragma unroll
                        for (int c2 = 0; c2 < 16; ++c2) {
                            const int cp = h * 16 + c2;                // token pair of this warp
                            float2 a = acc[cp];
                            a = __ffma2_rn(dd, __fadd2_rn(make_float2(fh[2 * c2], fh[2 * c2 + 1]), make_float2(fl[2 * c2], fl[2 * c2 + 1])), a);
#pragma unroll
                            for (int jq = 0; jq < 4; ++jq) {
                                const uint4 gv = lds128(gbase + cp * 64 + jq * 16);      // (g_j[even], g_j[odd], g_j+1[even], g_j+1[odd])
                                a = __ffma2_rn(make_float2(dm[2 * jq], dm[2 * jq]), make_float2(__uint_as_float(gv.x), __uint_as_float(gv.y)), a);
                                a = __ffma2_rn(make_float2(dm[2 * jq + 1], dm[2 * jq + 1]), make_float2(__uint_as_float(gv.z), __uint_as_float(gv.w)), a);
                            }
                            acc[cp] = a;
                        }
                    } else if (h == 0) {
                        // nothing to read for this warp: release the accumulator at once
                        fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sbase + BAR_TMEM_EMPTY + 8 * b);
                    }
                }
                // the table entry and the g tile have been read: the converters and the copy engine may reuse them
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + BAR_TAB_EMPTY + 8 * slot);
            }
            if (!ok) break;
            // y[token][n] = 2^-e_token * acc: for a fixed token the warp's 32 lanes write 32 consecutive floats
            const int n = tr.n0 + wr;
            if (tr.part >= 0) {
                // a piece of a tile: [token][weight row] into the piece's slot
                float* part = p.y_part + static_cast<size_t>(tr.part) * (TT * TW);
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int col = half * 64 + c;
                    const float v = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                    if (col < tr.nt) part[col * TW + wr] = v * __ldg(p.inv_s + tr.m0 + col);
                }
            } else if (n < p.N) {
                if constexpr (PEERS) {
                    // one copy of the 64 unrolled stores, walked once per destination buffer
#pragma unroll 1
                    for (int r = 0; r < pe.n; ++r) {
                        float* dst = pe.y[r] + pe.col0;
#pragma unroll
                        for (int c = 0; c < 64; ++c) {
                            const int col = half * 64 + c;
                            if (col < tr.nt) {
                                const int row = tr.m0 + col;
                                const float v = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                                dst[static_cast<size_t>(row) * pe.ld + n] = v * __ldg(p.inv_s + row);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int col = half * 64 + c;
                        if (col < tr.nt) {
                            const int row = tr.m0 + col;
                            int orow = p.out_row ? __ldg(p.out_row + row) : row;
                            if (p.out_identity && orow >= 0) orow = row;
                            const float v = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                            if (orow >= 0) p.y[static_cast<size_t>(orow) * p.N + n] = v * __ldg(p.inv_s + row);
                        }
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

// ---- the same kernel for weight types whose operand needs two fp16 pieces: Q4_0, Q8_0, Q6_K ----------------------
// (replaces gemm_int<dot_row_q4_0_int_neon / q8_0 / q6_k> of Laplace src/matmul_simd.cpp:143-182, 285-342 for large M.)
// A drain group is 256 values: a Q6_K super-block, or eight consecutive 32-value blocks of Q4_0 / Q8_0 (K % 256 == 0).
//   Q6_K        weight value sc * (q6 - 32), up to +-4096: split exactly into H = 32 * ((u >> 5) - 128) and L = u & 31 with
//               u = value + 4096 (both exact in fp16); group scale t = d of the super-block.
//   Q8_0, Q4_0  every block has its own fp16 scale d_b, so the operand carries (d_b / t) * q with t = max |d_b| of the
//               group: ratio = d_b / t in fp32, cut into fp16 pieces r1 + r2 (22 bits), and per value
//               hi = rn(r1 * q), lo = rn(r2 * q + (r1 * q - hi)) - the inner difference is exact (one fused
//               multiply-add). A group whose blocks share one scale has ratio 1: the operand is the integer q itself.
// Both weight pieces meet the stacked activation pieces: two MMA instructions per 16-value step, D += Wh . [hi | lo] and
// D += Wl . [hi | lo]; the drain adds y += t * (F_hi + F_lo) once per group. No min term in these types (Q4_0's offset
// -8 is part of the operand value nibble - 8). Weight rows are only 2-byte aligned in general (34-byte and 210-byte
// blocks), so the packed rows arrive by one plain bulk copy per row from the 16-byte boundary below the group's first
// byte, and the converters skip the difference.
namespace w2 {

constexpr int STAGES = 2;
constexpr int RAW_TILE_MAX = TW * 288;             // 36 KB: Q8_0 rows of 272 bytes + alignment slop
constexpr int TABN2 = 4;
template <uint32_t TYPE> struct Geo;
template <> struct Geo<LAPLACE_TYPE_Q4_0> { static constexpr int GROUP_BYTES = 8 * Q4_0_BYTES, PITCH = 160; };
template <> struct Geo<LAPLACE_TYPE_Q8_0> { static constexpr int GROUP_BYTES = 8 * Q8_0_BYTES, PITCH = 288; };
template <> struct Geo<LAPLACE_TYPE_Q6_K> { static constexpr int GROUP_BYTES = Q6_K_BYTES, PITCH = 224; };

constexpr uint32_t OFF_WH = 0;
constexpr uint32_t OFF_WL = OFF_WH + STAGES * W_TILE;
constexpr uint32_t OFF_A = OFF_WL + STAGES * W_TILE;
constexpr uint32_t OFF_RAW = OFF_A + STAGES * A_TILE;
constexpr uint32_t OFF_TAB = OFF_RAW + RAW_STAGES * RAW_TILE_MAX;
constexpr uint32_t OFF_BAR = OFF_TAB + TABN2 * TW * 4;
constexpr uint32_t BAR_FULL_A = OFF_BAR, BAR_FULL_W = BAR_FULL_A + 8 * STAGES, BAR_EMPTY = BAR_FULL_W + 8 * STAGES,
                   BAR_RAW_FULL = BAR_EMPTY + 8 * STAGES, BAR_RAW_EMPTY = BAR_RAW_FULL + 8 * RAW_STAGES,
                   BAR_TMEM_FULL = BAR_RAW_EMPTY + 8 * RAW_STAGES, BAR_TMEM_EMPTY = BAR_TMEM_FULL + 16,
                   BAR_TAB_EMPTY = BAR_TMEM_EMPTY + 16, OFF_TMEM_PTR = BAR_TAB_EMPTY + 8 * TABN2, OFF_ABORT = OFF_TMEM_PTR + 8;
constexpr uint32_t SMEM_BYTES = OFF_ABORT + 8 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(OFF_A % 1024 == 0 && OFF_RAW % 128 == 0, "tile alignment");

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
// hi / lo pieces of (r1 + r2) * x for a pair of exact small integers x
__device__ __forceinline__ void two_piece(__half2 r1, __half2 r2, __half2 x, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __hmul2(r1, x);
    hi = h2_bits(h);
    lo = h2_bits(__hfma2(r2, x, __hfma2(r1, x, __hneg2(h))));
}
// fp16 pieces of a ratio in [-1, 1]
__device__ __forceinline__ void ratio_pieces(float d, float t, __half2& r1, __half2& r2) {
    const float ratio = t > 0.0f ? __fdiv_rn(d, t) : 0.0f;
    const __half a = __float2half_rn(ratio);
    r1 = __half2half2(a);
    r2 = __half2half2(__float2half_rn(ratio - __half2float(a)));
}

// Where group `sb` of weight row `grow` starts, and how far that is above the 16-byte boundary the row's copy starts at.
template <uint32_t TYPE>
__device__ __forceinline__ const uint8_t* group_src(const SaParams& p, long long grow, int sb, uint32_t& mis) {
    const uint8_t* src = p.w + grow * static_cast<long long>(p.rb) + static_cast<long long>(sb) * Geo<TYPE>::GROUP_BYTES;
    mis = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & 15u);
    return src - mis;
}

template <uint32_t TYPE, bool PEERS>
__global__ void __launch_bounds__(THREADS, 1)
gemm_w2_sa_kernel(const __grid_constant__ SaMaps maps, const SaParams p, const SaPeers<PEERS> pe) {
    using G = Geo<TYPE>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_ABORT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sbase + BAR_FULL_A + 8 * s, 2);
            mbar_init(sbase + BAR_FULL_W + 8 * s, 4);
            mbar_init(sbase + BAR_EMPTY + 8 * s, 1);
        }
        for (int q = 0; q < RAW_STAGES; ++q) {
            mbar_init(sbase + BAR_RAW_FULL + 8 * q, 1);
            mbar_init(sbase + BAR_RAW_EMPTY + 8 * q, 4);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(sbase + BAR_TMEM_FULL + 8 * t, 1);
            mbar_init(sbase + BAR_TMEM_EMPTY + 8 * t, 8);
        }
        for (int t = 0; t < TABN2; ++t) mbar_init(sbase + BAR_TAB_EMPTY + 8 * t, 8);
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
    const Segments sg = segments(p);

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if ((warp == 0 || warp == 2) && lane == 0) {
            // ---------------- TMA producers: warp 0 copies the hi piece of the activations, warp 2 the lo piece ----------------
            const int pc = warp >> 1;
            int it = 0;
            bool ok = true;
            for (int seg = 0; ok && seg < sg.n; ++seg) {
                const TileRef tr = seg_ref(p, sg, seg);
                const int bk = box_bucket(tr.nt);
                const uint32_t piece = static_cast<uint32_t>(16 << bk) * 128u;
                for (int kc = tr.sb0 * 4; kc < tr.sb1 * 4; ++kc, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort<false>(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_FULL_A + 8 * s, piece);
                    tma_load_2d(sbase + OFF_A + s * A_TILE + pc * piece, &maps.a[bk], kc * BKC, pc * p.m_pad + tr.m0, sbase + BAR_FULL_A + 8 * s);
                }
            }
            if (!ok) {
                for (int k = 0; k < STAGES; ++k) {
                    const int v = it - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_FULL_A + 8 * (v % STAGES), (v / STAGES) & 1);
                }
            }
        } else if (warp == 3) {
            // ---------------- packed weights: one bulk copy per row and group, four rows per lane ----------------
            int sbc = 0;
            bool ok = true;
            for (int seg = 0; ok && seg < sg.n; ++seg) {
                const TileRef tr = seg_ref(p, sg, seg);
                for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                    const int q = sbc % RAW_STAGES;
                    bool w_ok = true;
                    if (lane == 0) w_ok = wait_or_abort<false>(sbase + BAR_RAW_EMPTY + 8 * q, ((sbc / RAW_STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY);
                    if (!__shfl_sync(0xffffffffu, w_ok, 0)) { ok = false; break; }
                    const uint8_t* src[4];
                    uint32_t bytes[4], total = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = 4 * lane + i;
                        uint32_t mis = 0;
                        src[i] = group_src<TYPE>(p, static_cast<long long>(tr.wrow0) + tr.n0 + r, sb, mis);
                        bytes[i] = tr.n0 + r < p.N ? ((mis + G::GROUP_BYTES + 15u) & ~15u) : 0u;       // rows past N: nothing to copy
                        total += bytes[i];
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                    if (lane == 0) mbar_expect_tx(sbase + BAR_RAW_FULL + 8 * q, total);
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (bytes[i]) bulk_g2s(sbase + OFF_RAW + q * RAW_TILE_MAX + (4 * lane + i) * G::PITCH, src[i], bytes[i], sbase + BAR_RAW_FULL + 8 * q);
                }
            }
            if (!ok && lane == 0) {
                for (int k = 0; k < RAW_STAGES; ++k) {
                    const int v = sbc - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_RAW_FULL + 8 * (v % RAW_STAGES), (v / RAW_STAGES) & 1);
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issue: two instructions per 16-value step (weight pieces Wh, Wl) ----------------
            int it = 0, sbc = 0;
            bool ok = true;
            for (int seg = 0; ok && seg < sg.n; ++seg) {
                const TileRef tr = seg_ref(p, sg, seg);
                const uint32_t idesc = idesc_f16_m128((16 << box_bucket(tr.nt)) + ((tr.nt + 15) & ~15));
                for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                    const int b = sbc & 1;
                    if (!wait_or_abort<true>(sbase + BAR_TMEM_EMPTY + 8 * b, ((sbc >> 1) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_TMEM)) { ok = false; break; }
                    fence_after();
                    const uint32_t f_tmem = tmem_base + b * 256;
                    for (int c = 0; c < 4; ++c, ++it) {
                        const int s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!wait_or_abort<true>(sbase + BAR_FULL_A + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                            !wait_or_abort<true>(sbase + BAR_FULL_W + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                        fence_after();
                        const uint64_t hdesc = smem_desc_sw128(sbase + OFF_WH + s * W_TILE);
                        const uint64_t ldesc = smem_desc_sw128(sbase + OFF_WL + s * W_TILE);
                        const uint64_t adesc = smem_desc_sw128(sbase + OFF_A + s * A_TILE);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t off = static_cast<uint64_t>(ks * 2);
                            mma_f16(f_tmem, hdesc + off, adesc + off, idesc, (c | ks) != 0);
                            mma_f16(f_tmem, ldesc + off, adesc + off, idesc, 1);
                        }
                        commit(sbase + BAR_EMPTY + 8 * s);
                    }
                    if (!ok) break;
                    commit(sbase + BAR_TMEM_FULL + 8 * b);
                }
            }
        }
    } else if (warp < 8) {
        // ---------------- converters: thread r owns weight row n0 + r (they keep the 128 registers of the launch) ----------------
        const int r = threadIdx.x - 128;
        const __half2 k1152 = __half2half2(__float2half_rn(1152.f));
        int it = 0, sbc = 0;
        bool ok = true;
        // A finished operand chunk is handed to the MMA thread one chunk late: the fence that makes the stores visible
        // to the tensor core waits for them to land, which takes about as long as converting the next chunk.
        int pend = -1;
        auto publish = [&]() {
            if (pend < 0) return;
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + BAR_FULL_W + 8 * pend);
            pend = -1;
        };
        for (int seg = 0; ok && seg < sg.n; ++seg) {
            const TileRef tr = seg_ref(p, sg, seg);
            const bool live = tr.n0 + r < p.N;
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                const int q = sbc % RAW_STAGES, slot = sbc % TABN2;
                uint32_t mis = 0;
                group_src<TYPE>(p, static_cast<long long>(tr.wrow0) + tr.n0 + r, sb, mis);
                const uint32_t raw = sbase + OFF_RAW + q * RAW_TILE_MAX + r * G::PITCH + mis;      // byte 0 of this row's group (2-byte aligned)
                if (!wait_or_abort<false>(sbase + BAR_RAW_FULL + 8 * q, (sbc / RAW_STAGES) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                    !wait_or_abort<false>(sbase + BAR_TAB_EMPTY + 8 * slot, ((sbc / TABN2) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                // group scale t and (Q4_0 / Q8_0) the blocks' own scales
                float t = 0.0f, dblk[8];
                if constexpr (TYPE == LAPLACE_TYPE_Q6_K) {
                    t = live ? half_bits_to_float(lds16(raw + 208)) : 0.0f;
                } else {
                    constexpr int BB = TYPE == LAPLACE_TYPE_Q8_0 ? Q8_0_BYTES : Q4_0_BYTES;
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        dblk[b] = live ? half_bits_to_float(lds16(raw + b * BB)) : 0.0f;
                        t = fmaxf(t, fabsf(dblk[b]));
                    }
                }
                reinterpret_cast<float*>(smem + OFF_TAB)[slot * TW + r] = t;
#pragma unroll 1
                for (int c = 0; c < 4; ++c, ++it) {
                    const int s = it % STAGES;
                    uint32_t hw[32], lw[32];                 // the row's 64 operand values of this chunk, two pieces
                    if (!live) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) hw[i] = lw[i] = 0u;
                    } else if constexpr (TYPE == LAPLACE_TYPE_Q8_0) {
#pragma unroll
                        for (int bb = 0; bb < 2; ++bb) {
                            __half2 r1, r2;
                            ratio_pieces(dblk[2 * c + bb], t, r1, r2);
                            uint32_t w8[8];
                            {
                                uint32_t a4[4], b4[4];
                                lds16B_align2(raw + (2 * c + bb) * Q8_0_BYTES + 2, a4);
                                lds16B_align2(raw + (2 * c + bb) * Q8_0_BYTES + 18, b4);
#pragma unroll
                                for (int i = 0; i < 4; ++i) { w8[i] = a4[i]; w8[4 + i] = b4[i]; }
                            }
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                // bytes + 128 under an fp16 exponent of 2^10: (1024 + 128 + q) - 1152 = q, exactly
                                const uint32_t u = w8[i] ^ 0x80808080u;
                                const __half2 x02 = __hsub2(bits_h2(prmt(u, 0x64646464u, 0x4240u)), k1152);
                                const __half2 x13 = __hsub2(bits_h2(prmt(u, 0x64646464u, 0x4341u)), k1152);
                                two_piece(r1, r2, x02, hw[16 * bb + 2 * i], lw[16 * bb + 2 * i]);
                                two_piece(r1, r2, x13, hw[16 * bb + 2 * i + 1], lw[16 * bb + 2 * i + 1]);
                            }
                        }
                    } else if constexpr (TYPE == LAPLACE_TYPE_Q4_0) {
                        const __half2 k1032 = __half2half2(__float2half_rn(1032.f)), k16th = __half2half2(__float2half_rn(0.0625f)),
                                      km72 = __half2half2(__float2half_rn(-72.f));
#pragma unroll
                        for (int bb = 0; bb < 2; ++bb) {
                            __half2 r1, r2;
                            ratio_pieces(dblk[2 * c + bb], t, r1, r2);
                            uint32_t w4[4];
                            lds16B_align2(raw + (2 * c + bb) * Q4_0_BYTES + 2, w4);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                // element l = low nibble of byte l, element l + 16 = high nibble; value = nibble - 8
                                const uint32_t w = w4[i], sh = w >> 8;
                                const __half2 l02 = __hsub2(bits_h2((w & 0x000f000fu) | 0x64006400u), k1032);
                                const __half2 l13 = __hsub2(bits_h2((sh & 0x000f000fu) | 0x64006400u), k1032);
                                const __half2 h02 = __hfma2(bits_h2((w & 0x00f000f0u) | 0x64006400u), k16th, km72);      // (1024 + 16 n) / 16 - 72
                                const __half2 h13 = __hfma2(bits_h2((sh & 0x00f000f0u) | 0x64006400u), k16th, km72);
                                two_piece(r1, r2, l02, hw[16 * bb + 2 * i], lw[16 * bb + 2 * i]);
                                two_piece(r1, r2, l13, hw[16 * bb + 2 * i + 1], lw[16 * bb + 2 * i + 1]);
                                two_piece(r1, r2, h02, hw[16 * bb + 8 + 2 * i], lw[16 * bb + 8 + 2 * i]);
                                two_piece(r1, r2, h13, hw[16 * bb + 8 + 2 * i + 1], lw[16 * bb + 8 + 2 * i + 1]);
                            }
                        }
                    } else {
                        // Q6_K (Laplace src/kernels.h:46-54, src/matmul.cpp:180-195): chunk c = half h, nibble side nib;
                        // value v of the chunk: 4 bits from ql[64 h + v] (low or high nibble), 2 bits from
                        // qh[32 h + (v & 31)] at shift 2 * (2 nib + (v >> 5)), scale sc[8 h + 4 nib + (v >> 4)]
                        const int h = c >> 1, nib = c & 1;
                        const __half2 hoff = __half2half2(__float2half_rn(-36864.f)), loff = __half2half2(__float2half_rn(-1024.f));
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {                 // 16 values share a scale
                            uint32_t ql4[4], qh4[4];
                            lds16B_align2(raw + 64 * h + 16 * j4, ql4);
                            lds16B_align2(raw + 128 + 32 * h + 16 * (j4 & 1), qh4);
                            const int sc = lds_s8(raw + 192 + 8 * h + 4 * nib + j4);
                            const int hshift = 2 * (2 * nib + (j4 >> 1));
                            const uint32_t cc = static_cast<uint32_t>(4096 - 32 * sc) * 0x00010001u;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t q6 = ((ql4[i] >> (4 * nib)) & 0x0f0f0f0fu) | (((qh4[i] >> hshift) << 4) & 0x30303030u);
                                const uint32_t e02 = q6 & 0x00ff00ffu, e13 = (q6 >> 8) & 0x00ff00ffu;
                                // both 16-bit lanes: u = sc * (q6 - 32) + 4096 in [0, 8192]; the 32-bit product cannot borrow
                                const uint32_t u02 = e02 * static_cast<uint32_t>(sc) + cc, u13 = e13 * static_cast<uint32_t>(sc) + cc;
                                // (v | 0x7800) is fp16(32768 + 32 v), (v | 0x6400) is fp16(1024 + v)
                                hw[8 * j4 + 2 * i] = h2_bits(__hadd2(bits_h2(((u02 >> 5) & 0x01ff01ffu) | 0x78007800u), hoff));
                                hw[8 * j4 + 2 * i + 1] = h2_bits(__hadd2(bits_h2(((u13 >> 5) & 0x01ff01ffu) | 0x78007800u), hoff));
                                lw[8 * j4 + 2 * i] = h2_bits(__hadd2(bits_h2((u02 & 0x001f001fu) | 0x64006400u), loff));
                                lw[8 * j4 + 2 * i + 1] = h2_bits(__hadd2(bits_h2((u13 & 0x001f001fu) | 0x64006400u), loff));
                            }
                        }
                    }
                    if (!wait_or_abort<false>(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    publish();                    // the previous chunk
                    uint8_t* hrow = smem + OFF_WH + s * W_TILE + r * 128;
                    uint8_t* lrow = smem + OFF_WL + s * W_TILE + r * 128;
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                        const uint32_t off = static_cast<uint32_t>(jj ^ (r & 7)) << 4;
                        *reinterpret_cast<uint4*>(hrow + off) = make_uint4(hw[4 * jj], hw[4 * jj + 1], hw[4 * jj + 2], hw[4 * jj + 3]);
                        *reinterpret_cast<uint4*>(lrow + off) = make_uint4(lw[4 * jj], lw[4 * jj + 1], lw[4 * jj + 2], lw[4 * jj + 3]);
                    }
                    pend = s;
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + BAR_RAW_EMPTY + 8 * q);
            }
        }
        if (ok) publish();
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");       // 4 x 40 + 4 x 128 + 8 x 168 <= 16 x 128
        // ---------------- drain: y += t * (F_hi + F_lo) once per group ----------------
        const int e8 = warp - 8;
        const int quad = e8 & 3, half = e8 >> 2;
        const uint32_t t_lane = static_cast<uint32_t>(quad * 32) << 16;
        const int wr = quad * 32 + lane;
        int sbc = 0;
        bool ok = true;
        for (int seg = 0; ok && seg < sg.n; ++seg) {
            const TileRef tr = seg_ref(p, sg, seg);
            const int box = 16 << box_bucket(tr.nt);
            float2 acc[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = make_float2(0.f, 0.f);
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++sbc) {
                const int b = sbc & 1, slot = sbc % TABN2;
                if (!wait_or_abort<false>(sbase + BAR_TMEM_FULL + 8 * b, (sbc >> 1) & 1, abort_flag, p.err, DEV_TIMEOUT_MMA)) { ok = false; break; }
                fence_after();
                const float tt = reinterpret_cast<const float*>(smem + OFF_TAB)[slot * TW + wr];
                const float2 t2 = make_float2(tt, tt);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (half * 64 + h * 32 < tr.nt) {
                        float fh[32], fl[32];
                        ld32(tmem_base + t_lane + b * 256 + half * 64 + h * 32, fh);
                        ld32(tmem_base + t_lane + b * 256 + box + half * 64 + h * 32, fl);
                        wait_ld();
#pragma unroll
                        for (int c2 = 0; c2 < 16; ++c2)
                            acc[h * 16 + c2] = __ffma2_rn(t2, __fadd2_rn(make_float2(fh[2 * c2], fh[2 * c2 + 1]), make_float2(fl[2 * c2], fl[2 * c2 + 1])),
                                                          acc[h * 16 + c2]);
                    }
                }
                fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(sbase + BAR_TMEM_EMPTY + 8 * b);
                    mbar_arrive(sbase + BAR_TAB_EMPTY + 8 * slot);
                }
            }
            if (!ok) break;
            const int n = tr.n0 + wr;
            if (tr.part >= 0) {
                // a piece of a tile: [token][weight row] into the piece's slot
                float* part = p.y_part + static_cast<size_t>(tr.part) * (TT * TW);
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int col = half * 64 + c;
                    const float v = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                    if (col < tr.nt) part[col * TW + wr] = v * __ldg(p.inv_s + tr.m0 + col);
                }
            } else if (n < p.N) {
                if constexpr (PEERS) {
                    // one copy of the 64 unrolled stores, walked once per destination buffer
#pragma unroll 1
                    for (int r = 0; r < pe.n; ++r) {
                        float* dst = pe.y[r] + pe.col0;
#pragma unroll
                        for (int c = 0; c < 64; ++c) {
                            const int col = half * 64 + c;
                            if (col < tr.nt) {
                                const int row = tr.m0 + col;
                                const float v = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                                dst[static_cast<size_t>(row) * pe.ld + n] = v * __ldg(p.inv_s + row);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int col = half * 64 + c;
                        if (col < tr.nt) {
                            const int row = tr.m0 + col;
                            int orow = p.out_row ? __ldg(p.out_row + row) : row;
                            if (p.out_identity && orow >= 0) orow = row;
                            const float v = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                            if (orow >= 0) p.y[static_cast<size_t>(orow) * p.N + n] = v * __ldg(p.inv_s + row);
                        }
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

}  // namespace w2


// ---- activation quantizer ------------------------------------------------------------------
// One CTA per activation row. The int8 values q and the block scales d are the reference's (Laplace
// src/matmul_simd.cpp:348-410: d = amax / 127, q = rne(x * (1 / d)), sums from the unclamped integers); what is
// written is the tensor-core operand built from them:
//   hi, lo [k]      fp16 pieces of 2^e * (d * q[k]), e chosen so that the row's largest |x| lands in [2^13, 2^14);
//                   within every four consecutive k the order is (0, 2, 1, 3), like the weight operand
//   g               fp32 2^e * (d * integer sum) per block - the reference's ActQ8::sum, scaled like the row -
//                   stored per PAIR of rows: g_pair[16 sb + 2 j + (row & 1)] for block 8 sb + j
//   inv_s           2^-e
// `load(b, t8)` returns values 4 t8 .. 4 t8 + 3 of block b of the row. The row is read twice (maximum, then
// quantization); the second read hits L1 / L2.
template <class Load>
__device__ __forceinline__ void quantize_row_sa(Load load, int K, __half* __restrict__ hi_row, __half* __restrict__ lo_row,
                                                float* __restrict__ g_pair, int odd, float* __restrict__ inv_s) {
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
            g_pair[2 * b + odd] = __fmul_rn(sum, s);          // element 16 (b / 8) + 2 (b % 8) + odd
        }
    }
}

struct SaOperand {          // operand buffers of one matmul
    __half* a;              // [2][m_pad][K]: hi rows, then lo rows
    float*  g;              // [m_pad / 2][K / 16]: block sums of a pair of rows, interleaved
    float*  inv_s;          // [m_pad]
    int     m_pad;
};

__global__ void __launch_bounds__(256) quantize_sa_kernel(const float* __restrict__ x, int K, SaOperand op) {
    const int m = blockIdx.x;
    const float* xr = x + static_cast<size_t>(m) * K;
    quantize_row_sa([&](int b, int t8) { return __ldg(reinterpret_cast<const float4*>(xr + b * 32) + t8); }, K,
                    op.a + static_cast<size_t>(m) * K, op.a + (static_cast<size_t>(op.m_pad) + m) * K,
                    op.g + static_cast<size_t>(m >> 1) * (K / 16), m & 1, op.inv_s + m);
}

// The same with the RMSNorm of the row in front (Laplace src/ops.cpp:34-74: inv = 1 / sqrt(mean(x^2) + eps),
// x_norm = (x * inv) * w), for prefill calls whose matrices share one normalised input (src/arch_llama.cpp:475-499).
__global__ void __launch_bounds__(256) quantize_sa_norm_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                                               float* __restrict__ x_norm_out, int K, SaOperand op) {
    __shared__ float red[8];
    __shared__ float s_inv;
    const int m = blockIdx.x;
    const float* xr = x + static_cast<size_t>(m) * K;
    float ss = 0.f;
    for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(xr) + i);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
        s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, static_cast<float>(K)), eps)));
    }
    __syncthreads();
    const float inv = s_inv;
    auto load = [&](int b, int t8) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(xr + b * 32) + t8);
        const float4 w = __ldg(reinterpret_cast<const float4*>(norm_w + b * 32) + t8);
        return make_float4(__fmul_rn(__fmul_rn(v.x, inv), w.x), __fmul_rn(__fmul_rn(v.y, inv), w.y),
                           __fmul_rn(__fmul_rn(v.z, inv), w.z), __fmul_rn(__fmul_rn(v.w, inv), w.w));
    };
    if (x_norm_out)
        for (int i = threadIdx.x; i < K / 4; i += blockDim.x)
            reinterpret_cast<float4*>(x_norm_out + static_cast<size_t>(m) * K)[i] = load(i >> 3, i & 7);
    __syncthreads();                  // quantize_row_sa reuses a shared array of its own for the row maximum
    quantize_row_sa(load, K, op.a + static_cast<size_t>(m) * K, op.a + (static_cast<size_t>(op.m_pad) + m) * K,
                    op.g + static_cast<size_t>(m >> 1) * (K / 16), m & 1, op.inv_s + m);
}

// Adds up the pieces of every output tile that the balanced split cut, in k order, and writes the tile to y.
// Block (t, j) handles 16 tokens of output tile t; a tile one CTA computed whole is already in y.
template <bool PEERS>
__global__ void __launch_bounds__(256) sk_fixup_kernel(const float* __restrict__ part, long long units, int grid, int nsb, int tiles_m,
                                                       int M, int N, float* __restrict__ y, const SaPeers<PEERS> pe) {
    const int t = blockIdx.x;
    const long long ua = static_cast<long long>(t) * nsb, ub = ua + nsb - 1;
    // the CTA that holds unit u is the largest c with sk_start(c) <= u
    auto owner = [&](long long u) {
        int c = static_cast<int>(((u + 1) * grid + units - 1) / units) - 1;
        c = c < 0 ? 0 : c >= grid ? grid - 1 : c;
        while (c + 1 < grid && sk_start(units, grid, c + 1) <= u) ++c;
        while (c > 0 && sk_start(units, grid, c) > u) --c;
        return c;
    };
    const int ca = owner(ua), cb = owner(ub);
    if (ca == cb) return;
    const int m0 = (t % tiles_m) * TT, n0 = (t / tiles_m) * TW;
    const int nt = M - m0 < TT ? M - m0 : TT;
    const int wr = threadIdx.x & (TW - 1);
    const int col0 = blockIdx.y * 16 + (threadIdx.x >> 7);          // this thread: tokens col0, col0 + 2, ..., col0 + 14
    if (n0 + wr >= N || col0 >= nt) return;
    float a[8];
    for (int c = ca; c <= cb; ++c) {
        const int slot = 2 * c + (c == ca ? 1 : 0);        // CTA ca holds the tile's first unit: its piece begins the tile
        const float* src = part + static_cast<size_t>(slot) * (TT * TW) + wr;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = col0 + 2 * j;
            const float v = col < nt ? __ldg(src + col * TW) : 0.f;
            a[j] = c == ca ? v : a[j] + v;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int col = col0 + 2 * j;
        if (col < nt) {
            if constexpr (PEERS) {
                const size_t at = static_cast<size_t>(m0 + col) * pe.ld + pe.col0 + n0 + wr;
                for (int r = 0; r < pe.n; ++r) pe.y[r][at] = a[j];
            } else {
                y[static_cast<size_t>(m0 + col) * N + n0 + wr] = a[j];
            }
        }
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
    return {align256(2 * m_pad * K * sizeof(__half)), align256(m_pad / 2 * (K / 16) * sizeof(float)), align256(m_pad * sizeof(float))};
}
SaOperand carve_operand(uint8_t*& s, size_t m_pad, int K) {
    const OperandBytes ob = operand_bytes(m_pad, K);
    SaOperand op;
    op.a = reinterpret_cast<__half*>(s);      s += ob.a;
    op.g = reinterpret_cast<float*>(s);       s += ob.g;
    op.inv_s = reinterpret_cast<float*>(s);   s += ob.s;
    op.m_pad = static_cast<int>(m_pad);
    return op;
}

struct SaLaunch {
    const uint8_t* w; uint32_t type; float* y; int M, K, N;
    long long w_rows;            // rows of the (stacked) weight matrix
    SaOperand op;
    const int4* tile_tab; const int* n_tiles_dev; const int* out_row; int out_identity;
    int tiles_m, tiles_n, grid;
    long long sk_units; float* y_part;
    const PeerOut* peers;        // nullptr, or: the result goes to every GPU's buffer
};

int run_sa_kernel(const SaLaunch& L, cudaStream_t st) {
    Context& c = ctx();
    const int K = L.K;
    SaMaps maps;
    for (int bk = 0; bk < 4; ++bk) {
        if (!make_map_2d(&maps.a[bk], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, L.op.a, static_cast<uint64_t>(K), 2ull * L.op.m_pad,
                         static_cast<uint64_t>(K) * 2, BKC, 16u << bk, CU_TENSOR_MAP_SWIZZLE_128B, "activations") ||
            !make_map_2d(&maps.g[bk], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, L.op.g, static_cast<uint64_t>(K / 16), static_cast<uint64_t>(L.op.m_pad / 2),
                         static_cast<uint64_t>(K / 16) * 4, 16, 8u << bk, CU_TENSOR_MAP_SWIZZLE_NONE, "block sums"))
            return LAPLACE_ERR_CUDA;
    }
    const uint64_t rb = row_bytes(L.type, K);
    if (L.type == LAPLACE_TYPE_Q4_K) {
        if (!make_map_2d(&maps.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, L.w, rb, static_cast<uint64_t>(L.w_rows), rb, Q4_K_BYTES, TW,
                         CU_TENSOR_MAP_SWIZZLE_NONE, "weights"))
            return LAPLACE_ERR_CUDA;
    } else {
        maps.w = maps.a[0];      // not used by the two-piece kernels (they copy weight rows by address)
    }
    SaParams p{};
    p.w = L.w; p.rb = static_cast<uint32_t>(rb);
    p.y = L.y; p.inv_s = L.op.inv_s; p.err = c.d_err;
    p.M = L.M; p.N = L.N; p.K = K; p.m_pad = L.op.m_pad;
    p.tiles_m = L.tiles_m; p.tiles_n = L.tiles_n;
    p.tile_tab = L.tile_tab; p.n_tiles_dev = L.n_tiles_dev; p.out_row = L.out_row; p.out_identity = L.out_identity;
    p.sk_units = L.sk_units; p.y_part = L.y_part;
    SaPeers<true> pe{};
    if (L.peers) {
        for (int r = 0; r < L.peers->world; ++r) pe.y[r] = L.peers->y[r];
        pe.n = L.peers->world; pe.ld = L.peers->ld; pe.col0 = L.peers->col0;
    }
    const SaPeers<false> none{};
    static bool configured = false;
    if (!configured) {
        const int q = static_cast<int>(SMEM_BYTES), w = static_cast<int>(w2::SMEM_BYTES);
        const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
        cudaError_t e = cudaFuncSetAttribute(gemm_q4k_sa_kernel<false>, at, q);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_q4k_sa_kernel<true>, at, q);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q4_0, false>, at, w);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q8_0, false>, at, w);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q6_K, false>, at, w);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q4_0, true>, at, w);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q8_0, true>, at, w);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q6_K, true>, at, w);
        if (e != cudaSuccess) return cuda_check(e, "cudaFuncSetAttribute gemm_sa");
        configured = true;
    }
    if (L.peers && (L.out_row || L.tile_tab)) return fail(LAPLACE_ERR_STATE, "gemm_sa: the peer-store form takes a plain dense call");
    const bool peers = L.peers != nullptr;
    switch (L.type) {
        case LAPLACE_TYPE_Q4_K:
            if (peers) gemm_q4k_sa_kernel<true><<<L.grid, THREADS, SMEM_BYTES, st>>>(maps, p, pe);
            else gemm_q4k_sa_kernel<false><<<L.grid, THREADS, SMEM_BYTES, st>>>(maps, p, none);
            break;
        case LAPLACE_TYPE_Q4_0:
            if (peers) w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q4_0, true><<<L.grid, THREADS, w2::SMEM_BYTES, st>>>(maps, p, pe);
            else w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q4_0, false><<<L.grid, THREADS, w2::SMEM_BYTES, st>>>(maps, p, none);
            break;
        case LAPLACE_TYPE_Q8_0:
            if (peers) w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q8_0, true><<<L.grid, THREADS, w2::SMEM_BYTES, st>>>(maps, p, pe);
            else w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q8_0, false><<<L.grid, THREADS, w2::SMEM_BYTES, st>>>(maps, p, none);
            break;
        case LAPLACE_TYPE_Q6_K:
            if (peers) w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q6_K, true><<<L.grid, THREADS, w2::SMEM_BYTES, st>>>(maps, p, pe);
            else w2::gemm_w2_sa_kernel<LAPLACE_TYPE_Q6_K, false><<<L.grid, THREADS, w2::SMEM_BYTES, st>>>(maps, p, none);
            break;
        default: return LAPLACE_UNSUPPORTED;
    }
    c.launches++;
    c.last_path = 2;
    return cuda_check(cudaGetLastError(), "gemm_sa launch");
}

// Balanced split of a dense call (see SaParams::sk_units). With at least as many output tiles as SMs every SM gets the
// same number of super-blocks; with fewer tiles a CTA takes no less than three super-blocks (about 4 us of work), so
// that a small call is not cut into pieces that cost more to add up than they save.
struct SplitPlan { int grid; long long units; };
SplitPlan plan_split(int M, int K, int N, bool allow) {
    const int nsb = K / 256, tiles = ((M + TT - 1) / TT) * ((N + TW - 1) / TW), sms = ctx().sm_count;
    SplitPlan s{tiles < sms ? tiles : sms, 0};
    if (!allow || tiles % sms == 0) return s;
    const long long units = static_cast<long long>(tiles) * nsb;
    long long grid = tiles >= sms ? sms : units / 3;
    if (grid > sms) grid = sms;
    if (grid < 2) return s;
    // the longest CTA's work, in super-blocks, with whole tiles and with the split; adding up the pieces is one more
    // launch, worth about three super-blocks
    const long long whole = static_cast<long long>((tiles + sms - 1) / sms) * nsb, split = (units + grid - 1) / grid;
    if (whole - split < 3) return s;
    s.grid = static_cast<int>(grid);
    s.units = units;
    return s;
}

}  // namespace

void release_gemm_sa_scratch() { g_scratch.release(); }

bool gemm_sa_supports(uint32_t type, int M, int K, int N) {
    // drain groups are 256 values for every type (a super-block, or eight 32-value blocks)
    return (type == LAPLACE_TYPE_Q4_K || type == LAPLACE_TYPE_Q6_K || type == LAPLACE_TYPE_Q4_0 || type == LAPLACE_TYPE_Q8_0) &&
           M > 8 && N > 0 && K > 0 && K % 256 == 0;
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
    pl.part_bytes = pl.sp.units ? align256(static_cast<size_t>(2 * pl.sp.grid) * TT * TW * sizeof(float)) : 0;
    return pl;
}

int check_args(const float* x, const uint8_t* w, uint32_t type, int M, int K, int N) {
    if (!gemm_sa_supports(type, M, K, N)) return LAPLACE_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(w) & (type == LAPLACE_TYPE_Q4_K ? 15 : 1))
        return fail(LAPLACE_ERR_ARG, "gemm: weights must be 16-byte (Q4_K) / 2-byte aligned on the device");
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(LAPLACE_ERR_ARG, "gemm: x not 16-byte aligned");
    return LAPLACE_OK;
}

// Quantizes x into `scratch` (device memory of at least pl.total() bytes, 256-byte aligned) and runs the kernel.
int gemm_sa_on_scratch(uint8_t* scratch, const SaPlan& pl, const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N,
                       cudaStream_t st, const PeerOut* peers = nullptr) {
    Context& c = ctx();
    int rc;
    uint8_t* s = scratch;
    const SaOperand op = carve_operand(s, pl.m_pad, K);
    if (x) {                          // nullptr: the operand is in place already (several matrices share one input)
        quantize_sa_kernel<<<M, 256, 0, st>>>(x, K, op);
        c.launches++;
        if ((rc = cuda_check(cudaGetLastError(), "quantize_sa launch"))) return rc;
    }
    SaLaunch L{};
    L.w = w; L.type = type; L.y = y; L.M = M; L.K = K; L.N = N; L.w_rows = N; L.op = op;
    L.tiles_m = pl.tiles_m; L.tiles_n = pl.tiles_n;
    L.sk_units = pl.sp.units;
    L.peers = peers;
    L.y_part = pl.sp.units ? reinterpret_cast<float*>(s) : nullptr;
    L.grid = pl.sp.grid;
    if ((rc = run_sa_kernel(L, st))) return rc;
    if (pl.sp.units) {
        const dim3 fg(pl.tiles_m * pl.tiles_n, TT / 16);
        if (peers) {
            SaPeers<true> pe{};
            for (int r = 0; r < peers->world; ++r) pe.y[r] = peers->y[r];
            pe.n = peers->world; pe.ld = peers->ld; pe.col0 = peers->col0;
            sk_fixup_kernel<true><<<fg, 256, 0, st>>>(L.y_part, pl.sp.units, pl.sp.grid, K / 256, pl.tiles_m, M, N, nullptr, pe);
        } else {
            sk_fixup_kernel<false><<<fg, 256, 0, st>>>(L.y_part, pl.sp.units, pl.sp.grid, K / 256, pl.tiles_m, M, N, y, SaPeers<false>{});
        }
        c.launches++;
        return cuda_check(cudaGetLastError(), "sk_fixup launch");
    }
    return LAPLACE_OK;
}


}  // namespace

int launch_gemm_sa(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, cudaStream_t st) {
    int rc = check_args(x, w, type, M, K, N);
    if (rc) return rc;
    const SaPlan pl = plan_sa(M, K, N, true);
    if ((rc = g_scratch.ensure(pl.total(), st))) return rc;
    return gemm_sa_on_scratch(static_cast<uint8_t*>(g_scratch.p), pl, x, w, type, y, M, K, N, st);
}

// Several matrices of one type and K against the same input rows (q / k / v, gate / up of src/arch_llama.cpp:475-499): the
// input is normalised (optional) and quantized once, then every matrix runs on that operand.
int launch_gemm_sa_multi(const float* x, const float* norm_w, float eps, float* x_norm_out, const uint8_t* const* ws, float* const* ys,
                         const int* ns, int n_mats, uint32_t type, int M, int K, cudaStream_t st) {
    int rc;
    size_t need = 0;
    for (int i = 0; i < n_mats; ++i) {
        if ((rc = check_args(x, ws[i], type, M, K, ns[i]))) return rc;
        const size_t t = plan_sa(M, K, ns[i], true).total();
        need = t > need ? t : need;
    }
    if (norm_w && ((reinterpret_cast<uintptr_t>(norm_w) & 15) || (x_norm_out && (reinterpret_cast<uintptr_t>(x_norm_out) & 15))))
        return fail(LAPLACE_ERR_ARG, "gemm_multi: the norm weights (and the optional output) must be 16-byte aligned");
    if ((rc = g_scratch.ensure(need, st))) return rc;
    uint8_t* scratch = static_cast<uint8_t*>(g_scratch.p);
    {
        uint8_t* s = scratch;
        const SaOperand op = carve_operand(s, plan_sa(M, K, ns[0], true).m_pad, K);
        if (norm_w) quantize_sa_norm_kernel<<<M, 256, 0, st>>>(x, norm_w, eps, x_norm_out, K, op);
        else quantize_sa_kernel<<<M, 256, 0, st>>>(x, K, op);
        ctx().launches++;
        if ((rc = cuda_check(cudaGetLastError(), "quantize_sa launch"))) return rc;
    }
    for (int i = 0; i < n_mats; ++i)
        if ((rc = gemm_sa_on_scratch(scratch, plan_sa(M, K, ns[i], true), nullptr, ws[i], type, ys[i], M, K, ns[i], st))) return rc;
    return LAPLACE_OK;
}

// The same call for a row-split matrix: this GPU's N columns of the result go to every GPU's [M][ld] buffer at column col0
// (see SaPeers). The stores are complete when the launched kernels are; announcing them to the other GPUs is
// the caller's next step (laplace_cuda_allgather_step_wait_dev).
int launch_gemm_sa_peers(const float* x, const uint8_t* w, uint32_t type, const PeerOut& po, int M, int K, int N, cudaStream_t st) {
    int rc = check_args(x, w, type, M, K, N);
    if (rc) return rc;
    const SaPlan pl = plan_sa(M, K, N, true);
    if ((rc = g_scratch.ensure(pl.total(), st))) return rc;
    return gemm_sa_on_scratch(static_cast<uint8_t*>(g_scratch.p), pl, x, w, type, nullptr, M, K, N, st, &po);
}

// The same call on scratch memory the caller owns (`cap` bytes at `scratch`, 256-byte aligned); nothing is
// allocated. The balanced split of launch_gemm_sa is kept when its partial results fit too (the result is then
// bit-identical to launch_gemm_sa's), otherwise the call runs on whole tiles.
int launch_gemm_sa_prealloc(uint8_t* scratch, size_t cap, const float* x, const uint8_t* w, uint32_t type, float* y,
                            int M, int K, int N, cudaStream_t st) {
    int rc = check_args(x, w, type, M, K, N);
    if (rc) return rc;
    SaPlan pl = plan_sa(M, K, N, true);
    if (pl.total() > cap) pl = plan_sa(M, K, N, false);
    if (pl.total() > cap)
        return fail(LAPLACE_ERR_LIMIT, "gemm: M=%d K=%d needs %zu bytes of scratch, the caller's area holds %zu", M, K, pl.total(), cap);
    return gemm_sa_on_scratch(scratch, pl, x, w, type, y, M, K, N, st);
}


// ---- expert-grouped matmul and fused expert FFN ---------------------------------------------------------------
// Laplace runs a mixture-of-experts layer token by token: per token one fused_moe_gemm_idx call over its top-k
// experts (gate/up, src/matmul.cpp:467-482, src/arch_gemma4.cpp:604), the gated activation (src/ops.cpp:128-176),
// one fused_moe_gemm_multi call (down, src/matmul.cpp:484-500, src/arch_gemma4.cpp:626) and a weighted sum
// (:634-638). With a batch of tokens every such call streams the selected experts again. Here all (token, expert)
// pairs of the batch are grouped by expert on the device and every expert's weights meet all of its tokens in one
// pass of the kernel above: for every pair p, y[p] = W[pair_expert[p]] . quantize(x[pair_row[p]]), which is what the
// per-token calls compute (a pair's result does not depend on which other pairs share its tile). An expert's tokens
// sit on the MMA's N side, padded to a multiple of 16 only, so an expert with 16 tokens costs an eighth of a full tile.
namespace {

// One block plans the whole call: pairs per expert, every pair's slot inside its expert, the first operand row of
// every expert (counts padded to 16 rows), the operand row of every pair and the inverse map, and the tile tables
// {first operand row, first weight row inside the expert, first weight row of the expert, tokens}: for every expert,
// for every group of up to 128 of its tokens, one tile per 128 weight rows. A second table (another N over the same
// row groups) serves the second matmul of a fused FFN; tiles_n2 = 0 leaves it out. Which slot a pair gets depends on
// the order the atomics land in; results do not.
__global__ void __launch_bounds__(1024) moe_plan_sa_kernel(const int* __restrict__ pair_expert, int P, int E, int rows_max,
                                                           int* __restrict__ dst_row, int* __restrict__ out_row,
                                                           int N1, int tiles_n1, int4* __restrict__ tab1, int* __restrict__ n_tiles1,
                                                           int N2, int tiles_n2, int4* __restrict__ tab2, int* __restrict__ n_tiles2,
                                                           int* err) {
    extern __shared__ int sm[];
    int* cnt = sm;              // [E] pairs per expert
    int* base = sm + E;         // [E] first operand row
    int* grp0 = sm + 2 * E;     // [E] row groups before the expert
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    for (int r = threadIdx.x; r < rows_max; r += blockDim.x) out_row[r] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = pair_expert[p];
        int slot = -1;                     // the pair is skipped: negative = "not mine" (experts placed on another GPU),
        if (e >= 0 && e < E) slot = atomicAdd(cnt + e, 1);
        else if (e >= E) report_status(err, DEV_BAD_INDEX);      // too large = the host reports a bad argument
        dst_row[p] = slot;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, groups = 0;
        for (int e = 0; e < E; ++e) {
            base[e] = rows;
            grp0[e] = groups;
            rows += (cnt[e] + 15) & ~15;
            groups += (cnt[e] + TT - 1) / TT;
        }
        *n_tiles1 = groups * tiles_n1;
        if (tiles_n2) *n_tiles2 = groups * tiles_n2;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int groups = (cnt[e] + TT - 1) / TT;
        for (int g = 0; g < groups; ++g) {
            const int nt = cnt[e] - g * TT < TT ? cnt[e] - g * TT : TT;
            for (int t = 0; t < tiles_n1; ++t) tab1[(grp0[e] + g) * tiles_n1 + t] = make_int4(base[e] + g * TT, t * TW, e * N1, nt);
            for (int t = 0; t < tiles_n2; ++t) tab2[(grp0[e] + g) * tiles_n2 + t] = make_int4(base[e] + g * TT, t * TW, e * N2, nt);
        }
    }
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int slot = dst_row[p];
        if (slot < 0) continue;
        const int r = base[pair_expert[p]] + slot;
        dst_row[p] = r;
        out_row[r] = p;
    }
}

// quantize_sa_kernel with a row gather on the way in and a row scatter on the way out: pair p reads x row
// src_rows[p] (p / src_div when src_rows is null: the top-k pairs of a token are consecutive) and writes operand
// row dst_rows[p] (negative: a skipped pair).
__global__ void __launch_bounds__(256) quantize_sa_mapped_kernel(const float* __restrict__ x, int K, const int* __restrict__ src_rows,
                                                                 int src_div, const int* __restrict__ dst_rows, SaOperand op) {
    const int p = blockIdx.x;
    const int dr = __ldg(dst_rows + p);
    if (dr < 0) return;
    const float* xr = x + static_cast<size_t>(src_rows ? __ldg(src_rows + p) : p / src_div) * K;
    quantize_row_sa([&](int b, int t8) { return __ldg(reinterpret_cast<const float4*>(xr + b * 32) + t8); }, K,
                    op.a + static_cast<size_t>(dr) * K, op.a + (static_cast<size_t>(op.m_pad) + dr) * K,
                    op.g + static_cast<size_t>(dr >> 1) * (K / 16), dr & 1, op.inv_s + dr);
}

__device__ __forceinline__ float act_swiglu(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
__device__ __forceinline__ float act_geglu(float g, float u) {
    const float g3 = (g * g) * g;
    const float gelu = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g3)));
    return gelu * u;
}

// Operand rows of the down matmul from the gate/up result: operand row r of gu holds [gate(I) | up(I)];
// h = act(gate) * up (ops::swiglu / ops::geglu, Laplace src/ops.cpp:128-176) is quantized like any activation row.
// One CTA per pair; h_out (optional) receives h in pair order.
__global__ void __launch_bounds__(256) moe_act_quant_sa_kernel(const float* __restrict__ gu, int I, int activation,
                                                               const int* __restrict__ dst_rows, SaOperand op, float* __restrict__ h_out) {
    const int p = blockIdx.x;
    const int r = __ldg(dst_rows + p);
    if (r < 0) return;
    const float* row = gu + static_cast<size_t>(r) * (2 * I);
    auto load = [&](int b, int t8) {
        const float4 g = __ldg(reinterpret_cast<const float4*>(row + b * 32) + t8);
        const float4 u = __ldg(reinterpret_cast<const float4*>(row + I + b * 32) + t8);
        return activation == 1 ? make_float4(act_geglu(g.x, u.x), act_geglu(g.y, u.y), act_geglu(g.z, u.z), act_geglu(g.w, u.w))
                               : make_float4(act_swiglu(g.x, u.x), act_swiglu(g.y, u.y), act_swiglu(g.z, u.z), act_swiglu(g.w, u.w));
    };
    if (h_out)
        for (int i = threadIdx.x; i < I / 4; i += blockDim.x)
            reinterpret_cast<float4*>(h_out + static_cast<size_t>(p) * I)[i] = load(i >> 3, i & 7);
    quantize_row_sa(load, I, op.a + static_cast<size_t>(r) * I, op.a + (static_cast<size_t>(op.m_pad) + r) * I,
                    op.g + static_cast<size_t>(r >> 1) * (I / 16), r & 1, op.inv_s + r);
}

// out[t][:] = sum over the token's live pairs, in slot order, of top_w[t][j] * dn[row of pair][:]
// (the reference's weight of pair j is top_w[j] * down_scale[expert], src/arch_gemma4.cpp:634-638; down_scale may be null)
__global__ void __launch_bounds__(256) moe_combine_sa_kernel(const float* __restrict__ dn, const int* __restrict__ dst_row,
                                                             const float* __restrict__ top_w, const int* __restrict__ top_idx,
                                                             const float* __restrict__ down_scale, int T, int top_k, int H,
                                                             float* __restrict__ out) {
    const int h4 = H / 4;
    const long long total = static_cast<long long>(T) * h4;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / h4), c = static_cast<int>(i - static_cast<long long>(t) * h4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < top_k; ++j) {
            const int r = __ldg(dst_row + t * top_k + j);
            if (r < 0) continue;
            float wgt = __ldg(top_w + t * top_k + j);
            if (down_scale) wgt = __fmul_rn(wgt, __ldg(down_scale + __ldg(top_idx + t * top_k + j)));
            const float4 v = __ldg(reinterpret_cast<const float4*>(dn + static_cast<long long>(r) * H) + c);
            acc.x = fmaf(wgt, v.x, acc.x); acc.y = fmaf(wgt, v.y, acc.y);
            acc.z = fmaf(wgt, v.z, acc.z); acc.w = fmaf(wgt, v.w, acc.w);
        }
        reinterpret_cast<float4*>(out + static_cast<long long>(t) * H)[c] = acc;
    }
}

Scratch g_moe_scratch;

// Upper bounds that hold for every routing of P pairs over E experts.
struct GroupBounds { size_t rows, groups; };
GroupBounds group_bounds(int P, int E) {
    const size_t live = static_cast<size_t>(E < P ? E : P);
    GroupBounds b;
    b.rows = ((static_cast<size_t>(P) + 15 * live + TT - 1) / TT + 1) * TT;       // every expert pads to 16 rows; one box of slack
    b.groups = static_cast<size_t>(P) / TT + live;
    return b;
}

int launch_plan(const int* pair_expert, int P, int E, int rows_max, int* dst_row, int* out_row, int N1, int tiles_n1, int4* tab1,
                int* n_tiles1, int N2, int tiles_n2, int4* tab2, int* n_tiles2, cudaStream_t st) {
    Context& c = ctx();
    const size_t sm = 3 * static_cast<size_t>(E) * sizeof(int);
    if (sm > 40 * 1024) return fail(LAPLACE_ERR_LIMIT, "moe: %d experts are more than the planning kernel holds", E);
    moe_plan_sa_kernel<<<1, 1024, sm, st>>>(pair_expert, P, E, rows_max, dst_row, out_row, N1, tiles_n1, tab1, n_tiles1,
                                            N2, tiles_n2, tab2, n_tiles2, c.d_err);
    c.launches++;
    return cuda_check(cudaGetLastError(), "moe_plan launch");
}

int grid_for_tiles(size_t tiles_max) {
    const size_t sms = static_cast<size_t>(ctx().sm_count);
    return static_cast<int>(tiles_max < 1 ? 1 : (tiles_max < sms ? tiles_max : sms));
}

}  // namespace

void release_moe_sa_scratch() { g_moe_scratch.release(); }

bool moe_sa_supports(uint32_t type, int K, int N) { return gemm_sa_supports(type, 9, K, N); }

int launch_moe_grouped_sa(const float* x, const uint8_t* w, uint32_t type, const int* pair_expert, const int* pair_row,
                          int P, int E, float* y, int K, int N, cudaStream_t st) {
    if (!moe_sa_supports(type, K, N)) return LAPLACE_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(w) & (type == LAPLACE_TYPE_Q4_K ? 15 : 1)) || (reinterpret_cast<uintptr_t>(x) & 15))
        return fail(LAPLACE_ERR_ARG, "moe_grouped: x (16 bytes) or w (16 bytes for Q4_K, else 2) is misaligned on the device");
    Context& c = ctx();
    const int tiles_n = (N + TW - 1) / TW;
    const GroupBounds gb = group_bounds(P, E);
    const size_t pair_bytes = align256(sizeof(int) * static_cast<size_t>(P)), out_bytes = align256(sizeof(int) * gb.rows);
    const size_t tab_bytes = align256(sizeof(int4) * gb.groups * tiles_n);
    const size_t total = operand_bytes(gb.rows, K).total() + pair_bytes + out_bytes + tab_bytes + 256;
    int rc;
    if ((rc = g_moe_scratch.ensure(total, st))) return rc;
    uint8_t* s = static_cast<uint8_t*>(g_moe_scratch.p);
    const SaOperand op = carve_operand(s, gb.rows, K);
    int* dst_row = reinterpret_cast<int*>(s);       s += pair_bytes;
    int* out_row = reinterpret_cast<int*>(s);       s += out_bytes;
    int4* tab = reinterpret_cast<int4*>(s);         s += tab_bytes;
    int* n_tiles = reinterpret_cast<int*>(s);
    if ((rc = launch_plan(pair_expert, P, E, static_cast<int>(gb.rows), dst_row, out_row, N, tiles_n, tab, n_tiles, 0, 0, nullptr, nullptr, st)))
        return rc;
    quantize_sa_mapped_kernel<<<P, 256, 0, st>>>(x, K, pair_row, 1, dst_row, op);
    c.launches++;
    if ((rc = cuda_check(cudaGetLastError(), "moe quantize launch"))) return rc;
    SaLaunch L{};
    L.w = w; L.type = type; L.y = y; L.M = P; L.K = K; L.N = N; L.w_rows = static_cast<long long>(E) * N; L.op = op;
    L.tile_tab = tab; L.n_tiles_dev = n_tiles; L.out_row = out_row;
    L.tiles_m = 1; L.tiles_n = tiles_n; L.grid = grid_for_tiles(gb.groups * tiles_n);
    rc = run_sa_kernel(L, st);
    if (rc == LAPLACE_OK) c.last_path = 3;
    return rc;
}

int launch_moe_ffn_sa(const float* x, const uint8_t* w_gate_up, const uint8_t* w_down, uint32_t type_gu, uint32_t type_dn,
                      const int* top_idx, const float* top_w, const float* down_scale, int T, int top_k, int E, int H, int I,
                      int activation, float* out, float* h_out, cudaStream_t st) {
    if (!moe_sa_supports(type_gu, H, 2 * I) || !moe_sa_supports(type_dn, I, H)) return LAPLACE_UNSUPPORTED;
    if (I % 32 || H % 4) return fail(LAPLACE_ERR_ARG, "moe_ffn: H=%d I=%d", H, I);
    if ((reinterpret_cast<uintptr_t>(w_gate_up) & (type_gu == LAPLACE_TYPE_Q4_K ? 15 : 1)) ||
        (reinterpret_cast<uintptr_t>(w_down) & (type_dn == LAPLACE_TYPE_Q4_K ? 15 : 1)) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail(LAPLACE_ERR_ARG, "moe_ffn: x, out (16 bytes) or the weights (16 bytes for Q4_K, else 2) are misaligned on the device");
    Context& c = ctx();
    const int P = T * top_k;
    const int tiles_n1 = (2 * I + TW - 1) / TW, tiles_n2 = (H + TW - 1) / TW;
    const GroupBounds gb = group_bounds(P, E);
    const size_t pair_bytes = align256(sizeof(int) * static_cast<size_t>(P)), out_bytes = align256(sizeof(int) * gb.rows);
    const size_t tab1_bytes = align256(sizeof(int4) * gb.groups * tiles_n1), tab2_bytes = align256(sizeof(int4) * gb.groups * tiles_n2);
    const size_t gu_bytes = align256(gb.rows * 2 * I * sizeof(float)), dn_bytes = align256(gb.rows * H * sizeof(float));
    const size_t total = operand_bytes(gb.rows, H).total() + operand_bytes(gb.rows, I).total() + pair_bytes + out_bytes +
                         tab1_bytes + tab2_bytes + gu_bytes + dn_bytes + 256;
    int rc;
    if ((rc = g_moe_scratch.ensure(total, st))) return rc;
    uint8_t* s = static_cast<uint8_t*>(g_moe_scratch.p);
    const SaOperand op1 = carve_operand(s, gb.rows, H);
    const SaOperand op2 = carve_operand(s, gb.rows, I);
    int* dst_row = reinterpret_cast<int*>(s);       s += pair_bytes;
    int* out_row = reinterpret_cast<int*>(s);       s += out_bytes;
    int4* tab1 = reinterpret_cast<int4*>(s);        s += tab1_bytes;
    int4* tab2 = reinterpret_cast<int4*>(s);        s += tab2_bytes;
    float* gu = reinterpret_cast<float*>(s);        s += gu_bytes;
    float* dn = reinterpret_cast<float*>(s);        s += dn_bytes;
    int* n_tiles1 = reinterpret_cast<int*>(s);
    int* n_tiles2 = n_tiles1 + 1;
    if ((rc = launch_plan(top_idx, P, E, static_cast<int>(gb.rows), dst_row, out_row, 2 * I, tiles_n1, tab1, n_tiles1, H, tiles_n2, tab2, n_tiles2, st)))
        return rc;
    quantize_sa_mapped_kernel<<<P, 256, 0, st>>>(x, H, nullptr, top_k, dst_row, op1);
    c.launches++;
    if ((rc = cuda_check(cudaGetLastError(), "moe quantize launch"))) return rc;

    SaLaunch L{};
    L.w = w_gate_up; L.type = type_gu; L.y = gu; L.M = P; L.K = H; L.N = 2 * I; L.w_rows = static_cast<long long>(E) * 2 * I; L.op = op1;
    L.tile_tab = tab1; L.n_tiles_dev = n_tiles1; L.out_row = out_row; L.out_identity = 1;      // gu stays in operand-row order
    L.tiles_m = 1; L.tiles_n = tiles_n1; L.grid = grid_for_tiles(gb.groups * tiles_n1);
    if ((rc = run_sa_kernel(L, st))) return rc;

    moe_act_quant_sa_kernel<<<P, 256, 0, st>>>(gu, I, activation, dst_row, op2, h_out);
    c.launches++;
    if ((rc = cuda_check(cudaGetLastError(), "moe_act_quant launch"))) return rc;

    SaLaunch L2{};
    L2.w = w_down; L2.type = type_dn; L2.y = dn; L2.M = P; L2.K = I; L2.N = H; L2.w_rows = static_cast<long long>(E) * H; L2.op = op2;
    L2.tile_tab = tab2; L2.n_tiles_dev = n_tiles2; L2.out_row = out_row; L2.out_identity = 1;
    L2.tiles_m = 1; L2.tiles_n = tiles_n2; L2.grid = grid_for_tiles(gb.groups * tiles_n2);
    if ((rc = run_sa_kernel(L2, st))) return rc;

    const long long total4 = static_cast<long long>(T) * (H / 4);
    long long blocks = (total4 + 255) / 256;
    if (blocks > static_cast<long long>(c.sm_count) * 8) blocks = static_cast<long long>(c.sm_count) * 8;
    moe_combine_sa_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), 256, 0, st>>>(dn, dst_row, top_w, top_idx, down_scale, T, top_k, H, out);
    c.launches++;
    c.last_path = 4;
    return cuda_check(cudaGetLastError(), "moe_combine launch");
}


// ---- router ------------------------------------------------------------------------------------------------
// The reference's expert selection for one token (src/arch_gemma4.cpp:547-565), operation for operation: softmax
// over the router logits (maximum, exp(l - max) summed in index order, division), then top_k times the largest
// remaining probability - the FIRST index wins among equal values, as its strict comparison does - and the selected
// probabilities renormalised by their sum (added in selection order). One thread per token walks the experts in
// order, so every fp32 operation happens in the reference's order; with a few hundred experts that is microseconds.
namespace {

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int T, int E, int top_k,
                                                        int* __restrict__ top_idx, float* __restrict__ top_w) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const float* l = logits + static_cast<size_t>(t) * E;
    float maxl = l[0];
    for (int e = 1; e < E; ++e) if (l[e] > maxl) maxl = l[e];
    float suml = 0.0f;
    for (int e = 0; e < E; ++e) suml = __fadd_rn(suml, expf(__fsub_rn(l[e], maxl)));
    int* ti = top_idx + static_cast<size_t>(t) * top_k;
    float* tw = top_w + static_cast<size_t>(t) * top_k;
    float wsum = 0.0f;
    for (int k = 0; k < top_k; ++k) {
        int best = -1;
        float best_p = 0.0f;
        for (int e = 0; e < E; ++e) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= ti[j] == e;
            // a taken expert's probability has been replaced by -1e30 in the reference
            const float p = taken ? -1e30f : __fdiv_rn(expf(__fsub_rn(l[e], maxl)), suml);
            if (best < 0 || p > best_p) { best = e; best_p = p; }
        }
        ti[k] = best;
        tw[k] = best_p;
        wsum = __fadd_rn(wsum, best_p);
    }
    for (int k = 0; k < top_k; ++k) tw[k] = __fdiv_rn(tw[k], wsum);
}

}  // namespace

int launch_moe_route(const float* logits, int T, int E, int top_k, int* top_idx, float* top_w, cudaStream_t st) {
    Context& c = ctx();
    moe_route_kernel<<<(T + 127) / 128, 128, 0, st>>>(logits, T, E, top_k, top_idx, top_w);
    c.launches++;
    return cuda_check(cudaGetLastError(), "moe_route launch");
}


// ---- exchange helpers of the expert-parallel layer ---------------------------------------
// One all-gather moves [x | expert ids | weights] per token. pack builds a rank's send rows,
// unpack splits the gathered rows and turns global expert ids into local ones (-1 = another GPU's).
namespace {

__global__ void moe_pack_kernel(const float* __restrict__ x, const int* __restrict__ idx, const float* __restrict__ wts,
                                int T, int H, int k, float* __restrict__ packed) {
    const int stride = H + 2 * k;
    const long long total = static_cast<long long>(T) * stride;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / stride), c = static_cast<int>(i - static_cast<long long>(t) * stride);
        float v;
        if (c < H) v = x[static_cast<long long>(t) * H + c];
        else if (c < H + k) v = __int_as_float(idx[t * k + (c - H)]);
        else v = wts[t * k + (c - H - k)];
        packed[i] = v;
    }
}

__global__ void moe_unpack_kernel(const float* __restrict__ packed, int T, int H, int k, int first, int count,
                                  float* __restrict__ x, int* __restrict__ idx_local, float* __restrict__ wts) {
    const int stride = H + 2 * k;
    const long long total = static_cast<long long>(T) * stride;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / stride), c = static_cast<int>(i - static_cast<long long>(t) * stride);
        const float v = packed[i];
        if (c < H) x[static_cast<long long>(t) * H + c] = v;
        else if (c < H + k) {
            const int e = __float_as_int(v) - first;
            idx_local[t * k + (c - H)] = (e >= 0 && e < count) ? e : -1;
        } else wts[t * k + (c - H - k)] = v;
    }
}

}  // namespace

int launch_moe_pack(const float* x, const int* idx, const float* wts, int T, int H, int k, float* packed, cudaStream_t st) {
    Context& c = ctx();
    const long long total = static_cast<long long>(T) * (H + 2 * k);
    long long blocks = (total + 255) / 256;
    if (blocks > static_cast<long long>(c.sm_count) * 8) blocks = static_cast<long long>(c.sm_count) * 8;
    moe_pack_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), 256, 0, st>>>(x, idx, wts, T, H, k, packed);
    c.launches++;
    return cuda_check(cudaGetLastError(), "moe_pack launch");
}

int launch_moe_unpack(const float* packed, int T, int H, int k, int first, int count, float* x, int* idx_local, float* wts,
                      cudaStream_t st) {
    Context& c = ctx();
    const long long total = static_cast<long long>(T) * (H + 2 * k);
    long long blocks = (total + 255) / 256;
    if (blocks > static_cast<long long>(c.sm_count) * 8) blocks = static_cast<long long>(c.sm_count) * 8;
    moe_unpack_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), 256, 0, st>>>(packed, T, H, k, first, count, x, idx_local, wts);
    c.launches++;
    return cuda_check(cudaGetLastError(), "moe_unpack launch");
}

// ---- the entry point that allocates nothing -------------------------------------------
// Some hosts of this library must not (or cannot) call the CUDA allocator on the request
// path: a serving process that has handed all free HBM to its own pools (KV cache,
// activations), so that cudaMalloc would fail or fragment them, and latency-bound loops that
// cannot take the allocator's locks or the implicit device synchronisation that comes with
// cudaFree when a buffer has to grow. For them the scratch of the prefill GEMM
// (the quantized activations) lives in a fixed array inside the library image instead of a
// growable cudaMalloc'd buffer.
//
// The array is part of every context that loads the library (NOALLOC_SCRATCH_BYTES of HBM
// per GPU until the process exits). In host code its name is only a handle; the device
// address comes from cudaGetSymbolAddress, asked once per device with that device current.
constexpr size_t NOALLOC_SCRATCH_BYTES = 10u << 20;    // 10 MiB: e.g. M = 512, K = 4096 needs 8.3 MiB
static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

namespace {
uint8_t* g_noalloc_ptr = nullptr;     // device address of g_noalloc_scratch on g_noalloc_dev
int      g_noalloc_dev = -1;
}  // namespace

}  // namespace lp

extern "C" int laplace_cuda_gemm_noalloc_dev(const float* x, const uint8_t* w, uint32_t type, float* y,
                                             int M, int K, int N, void* stream) {
    using namespace lp;
    Context& c = ctx();
    if (!c.ready) return fail(LAPLACE_ERR_STATE, "laplace_cuda_init has not been called (or found no GPU)");
    if (!x || !w || !y) return fail(LAPLACE_ERR_ARG, "gemm_noalloc: null pointer");
    if (!gemm_sa_supports(type, M, K, N))
        return fail(LAPLACE_ERR_ARG, "gemm_noalloc: only the prefill shapes are served here (M > 8, K %% 256 == 0, Q4_0 / Q8_0 / Q4_K / "
                                     "Q6_K); decode calls (M <= 8) use no scratch at all, call laplace_cuda_gemm_dev");
    if (g_noalloc_dev != c.device) {
        // first call on this device: resolve the array's device address (the library is bound to c.device,
        // make sure it is the current one for the lookup)
        int cur = -1;
        cudaError_t e = cudaGetDevice(&cur);
        if (e == cudaSuccess && cur != c.device) e = cudaSetDevice(c.device);
        void* ptr = nullptr;
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e == cudaSuccess && cur >= 0 && cur != c.device) e = cudaSetDevice(cur);
        if (e != cudaSuccess || !ptr) return cuda_check(e == cudaSuccess ? cudaErrorInvalidSymbol : e, "cudaGetSymbolAddress(scratch)");
        g_noalloc_ptr = static_cast<uint8_t*>(ptr);
        g_noalloc_dev = c.device;
    }
    // the same K-split as laplace_cuda_gemm_dev (hence bit-identical results) whenever its partial results fit the
    // array too; otherwise no split (results then agree to fp32 rounding)
    return launch_gemm_sa_prealloc(g_noalloc_ptr, NOALLOC_SCRATCH_BYTES, x, w, type, y, M, K, N,
                                   stream ? static_cast<cudaStream_t>(stream) : c.stream);
}
