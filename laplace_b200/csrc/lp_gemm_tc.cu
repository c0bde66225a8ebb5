// lp_gemm_tc.cu - prefill GEMM (M >= 9 activation rows) on the 5th-generation
// tensor cores: Q4_K weights x Q8 activations with exact per-block integer
// sums. Replaces gemm_int<dot_row_q4_k_int_neon> of Laplace's NEON back-end
// (src/matmul_simd.cpp:226-283, 432-455) for large M.
//
// Why fp16 operands for an "int8" dot: every 32-value block carries its own
// fp32 activation scale d_x, so the integer sum of each block has to leave the
// tensor core and be scaled on CUDA cores; that per-block drain, not the MMA,
// bounds throughput. With kind::f16 the accumulator already holds the block sum
// as an exact fp32 integer (|sum| <= 32*945*127 < 2^24), so the drain is one
// fused multiply-add per element - no int->float conversion - and the 6-bit
// sub-block scale rides inside the weight operand (sc*nibble <= 945 is exact in
// fp16). Per super-block sb of 8 blocks:
//
//   y[m,n] += d[n,sb] * sum_{j<8} d_x[m,8sb+j] * F[m,n,8sb+j]  -  dmin[n,sb] * G[m,n,sb]
//   F[m,n,b]  = sum_{k in b} q_x[m,k] * (sc*nibble)[n,k]          (tcgen05.mma kind::f16, fp16, exact)
//   G[m,n,sb] = sum_{j<8} sum_x[m,8sb+j] * mn[n,8sb+j]            (tcgen05.mma kind::f16, bf16)
//
// G, the "min" correction of Q4_K, would cost a second multiply-add per element
// and block on CUDA cores; instead sum_x (fp32) is split into three bf16 pieces
// (exact to 24 bits), the 6-bit mins are exact in bf16, and one K=32 MMA per
// super-block accumulates G in TMEM, drained once per super-block.
//
// Roles in one 512-thread CTA (one CTA per SM, persistent over 128x128 tiles):
//   warp 0      TMA: activation tiles (fp16 q values, 128 tokens x 64 k, 128-byte swizzle)
//   warps 1, 2  MMA issue (one lane each: first / second block of every 64-k chunk, each
//               owning one TMEM block-sum buffer); warp 1 also issues G and owns TMEM
//   warp 3      TMA: packed Q4_K super-blocks (128 rows x 144 bytes) and the bf16 pieces
//               of sum_x (one tile per pair of super-blocks)
//   warps 4-7   converters: packed super-blocks (shared memory) -> fp16 weight operand
//               tile, bf16 mins operand and d / dmin tables in shared memory
//   warps 8-15  epilogue: tcgen05.ld of each block's 128x128 fp32 tile (double
//               buffered in TMEM), scaling into a per-super-block partial in registers;
//               the tile's running y lives in TMEM and is updated once per super-block
// All mbarrier waits are bounded; a wait that gives up raises the status word
// and every role leaves its loop.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>
#include <vector>

#include "lp_common.cuh"

namespace lp {

namespace {

constexpr int BM = 128, BN = 128, BKC = 64;        // tile; BKC = k per pipeline stage (two 32-value blocks)
constexpr int STAGES = 3;                          // main ring: activation + weight operand tiles
constexpr int RAW_STAGES = 3;                      // ring of packed super-blocks (128 rows x 144 bytes) ahead of the converters
constexpr int RAW_TILE = BN * Q4_K_BYTES;          // 18 KB
constexpr int GST = 2;                             // ring of "pair of super-blocks" stages for the G operands
constexpr int A_TILE = BM * BKC * 2;               // 16 KB, fp16
constexpr int B_TILE = BN * BKC * 2;               // 16 KB, fp16
constexpr int G_TILE = 128 * 64 * 2;               // 16 KB, bf16: 32 k per super-block, two super-blocks per row
constexpr int GTAB_BYTES = 2 * 2 * BN * 4;         // per G stage: [super-block of the pair][d, dmin][column]
constexpr int THREADS = 512;
constexpr int TMEM_COLS = 512;                     // F0, F1 (block sums, double buffered), G, running y
constexpr uint32_t TM_F = 0, TM_G = 256, TM_ACC = 384;

// shared-memory map (dynamic, 1024-byte aligned base)
constexpr uint32_t OFF_A = 0;
constexpr uint32_t OFF_B = OFF_A + STAGES * A_TILE;
constexpr uint32_t OFF_GA = OFF_B + STAGES * B_TILE;
constexpr uint32_t OFF_GB = OFF_GA + GST * G_TILE;
constexpr uint32_t OFF_GTAB = OFF_GB + GST * G_TILE;
constexpr uint32_t OFF_RAW = OFF_GTAB + GST * GTAB_BYTES;
constexpr uint32_t OFF_BAR = OFF_RAW + RAW_STAGES * RAW_TILE;
constexpr uint32_t BAR_FULL_A = OFF_BAR, BAR_FULL_B = BAR_FULL_A + 8 * STAGES, BAR_EMPTY = BAR_FULL_B + 8 * STAGES,
                   BAR_TMEM_FULL = BAR_EMPTY + 8 * STAGES, BAR_TMEM_EMPTY = BAR_TMEM_FULL + 16,
                   BAR_G_FULL_A = BAR_TMEM_EMPTY + 16, BAR_G_FULL_B = BAR_G_FULL_A + 8 * GST,
                   BAR_G_EMPTY = BAR_G_FULL_B + 16 * GST, BAR_G_TAB_EMPTY = BAR_G_EMPTY + 8 * GST,
                   BAR_GT_FULL = BAR_G_TAB_EMPTY + 8 * GST, BAR_GT_EMPTY = BAR_GT_FULL + 8,
                   BAR_RAW_FULL = BAR_GT_EMPTY + 8, BAR_RAW_EMPTY = BAR_RAW_FULL + 8 * RAW_STAGES,
                   OFF_TMEM_PTR = BAR_RAW_EMPTY + 8 * RAW_STAGES, OFF_ABORT = OFF_TMEM_PTR + 8;
constexpr uint32_t SMEM_BYTES = OFF_ABORT + 8 + 1024;   // + slack for the 1024-byte alignment

struct TcParams {
    const uint8_t* w;        // Q4_K weights, N rows of rb bytes
    const float*   dx;       // [M][K/32] activation scales
    float*         y;        // [M][N]
    int*           err;
    int            M, N, K;
    uint32_t       rb;
    int            tiles_m, tiles_n;
    // expert-grouped calls: tiles come from a table built on the device, rows of the activation
    // operand are scattered back through out_row (-1 = padding row)
    const int4*    tile_tab;     // {m0, n0, first weight row of the expert, unused}; nullptr = dense tiling
    const int*     n_tiles_dev;
    const int*     out_row;
    int            out_identity; // 1: a live row m is written to row m of y (y is in operand-row order), not to out_row[m]
    // split-K (dense tiling with few output tiles): ksplit CTAs share an output tile, each takes sb_per
    // super-blocks (an even number) and writes its partial result to y_part[k-slice][M][N]; a second kernel
    // adds the slices in a fixed order
    int            ksplit, sb_per;
    float*         y_part;
};

struct TileRef { int m0, n0, wrow0, sb0, sb1, ks; };
__device__ __forceinline__ TileRef tile_ref(const TcParams& p, int tile) {
    const int nsb = p.K / 256;
    if (p.tile_tab) {
        const int4 t = __ldg(p.tile_tab + tile);
        return {t.x, t.y, t.z, 0, nsb, 0};
    }
    const int out_tiles = p.tiles_m * p.tiles_n;
    const int ks = tile / out_tiles, t = tile - ks * out_tiles;
    const int sb0 = ks * p.sb_per;
    const int sb1 = sb0 + p.sb_per < nsb ? sb0 + p.sb_per : nsb;
    return {(t % p.tiles_m) * BM, (t / p.tiles_m) * BN, 0, sb0, sb1, ks};
}
__device__ __forceinline__ int tile_count(const TcParams& p) {
    return p.tile_tab ? __ldg(p.n_tiles_dev) : p.tiles_m * p.tiles_n * p.ksplit;
}

// ---- tcgen05 / TMA wrappers ---------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        :: "r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
           "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
           "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
           "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);          // start address
    d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (Blackwell)
    d |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
    return d;
}
// kind::f16: D fp32, A fp16, B fp16, both K-major, M = 128, N = 128.
constexpr uint32_t IDESC_F16 = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) |
                               (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);

// Same shape with bf16 operands (the G product).
constexpr uint32_t IDESC_BF16 = IDESC_F16 | (1u << 7) | (1u << 10);

// Waits that also give up when another role has raised the abort flag. The MMA-issuing
// thread is the pipeline's metronome: it polls without a suspend hint, and every other
// role waits suspended in hardware so that it does not take issue slots from it.
template <bool SPIN>
__device__ __forceinline__ bool wait_or_abort_t(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    for (uint32_t it = 0; it < (SPIN ? (1u << 26) : (1u << 22)); ++it) {
        if (SPIN ? mbar_try_wait_nohint(bar, parity) : mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    report_status(err, code);
    return false;
}
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    return wait_or_abort_t<false>(bar, parity, abort_flag, err, code);
}
__device__ __forceinline__ bool spin_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    return wait_or_abort_t<true>(bar, parity, abort_flag, err, code);
}

// ---- the kernel -----------------------------------------------------------------
// Counters shared by all roles (each role advances its own copy in the same order):
//   it   main-ring chunk counter (64 k each), stage = it % STAGES
//   bc   block counter (32 k each), TMEM block-sum buffer = bc & 1
//   gp   pair-of-super-blocks counter, G stage = gp % GST
// A tile walks super-blocks 0 .. nsb_pad-1, nsb_pad = K/256 rounded up to even; a
// padding super-block has no chunks and contributes zeros to G.
__global__ void __launch_bounds__(THREADS, 1)
gemm_q4k_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_g,
                   const __grid_constant__ CUtensorMap tmap_w, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_ABORT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sbase + BAR_FULL_A + 8 * s, 1);
            mbar_init(sbase + BAR_FULL_B + 8 * s, 4);        // one arrive per converter warp
            mbar_init(sbase + BAR_EMPTY + 8 * s, 2);         // tcgen05.commit from each of the two MMA threads
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(sbase + BAR_TMEM_FULL + 8 * t, 1);     // tcgen05.commit
            mbar_init(sbase + BAR_TMEM_EMPTY + 8 * t, 8);    // one arrive per epilogue warp
        }
        for (int g = 0; g < GST; ++g) {
            mbar_init(sbase + BAR_G_FULL_A + 8 * g, 1);
            mbar_init(sbase + BAR_G_FULL_B + 16 * g, 4);     // per super-block of the pair: 4 converter warps
            mbar_init(sbase + BAR_G_FULL_B + 16 * g + 8, 4);
            mbar_init(sbase + BAR_G_EMPTY + 8 * g, 1);       // tcgen05.commit
            mbar_init(sbase + BAR_G_TAB_EMPTY + 8 * g, 8);   // one arrive per epilogue warp
        }
        for (int q = 0; q < RAW_STAGES; ++q) {
            mbar_init(sbase + BAR_RAW_FULL + 8 * q, 1);
            mbar_init(sbase + BAR_RAW_EMPTY + 8 * q, 4);     // one arrive per converter warp
        }
        mbar_init(sbase + BAR_GT_FULL, 1);                   // tcgen05.commit
        mbar_init(sbase + BAR_GT_EMPTY, 8);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(sbase + OFF_TMEM_PTR), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + OFF_TMEM_PTR);

    const int n_tiles = tile_count(p);
    const int nsb = p.K / 256;
    const int n_pairs = (nsb + 1) / 2;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer: activation tiles ----------------
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                const int m0 = tr.m0;
                for (int kc = tr.sb0 * 4; kc < tr.sb1 * 4; ++kc, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_FULL_A + 8 * s, A_TILE);
                    tma_load_2d(sbase + OFF_A + s * A_TILE, &tmap_a, kc * BKC, m0, sbase + BAR_FULL_A + 8 * s);
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
            // ---------------- TMA producer: packed weights, one super-block of 128 rows per tile ----------------
            // (rows past N are zero-filled by the copy engine: d = 0, every scale 0)
            // The same thread also brings the bf16 pieces of sum_x, one tile per pair of super-blocks.
            int rq = 0, gp = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                const int m0 = tr.m0, n0 = tr.wrow0 + tr.n0;
                for (int sb = tr.sb0; sb < tr.sb1; ++sb, ++rq) {
                    const int q = rq % RAW_STAGES;
                    if (!wait_or_abort(sbase + BAR_RAW_EMPTY + 8 * q, ((rq / RAW_STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_RAW_FULL + 8 * q, RAW_TILE);
                    tma_load_2d(sbase + OFF_RAW + q * RAW_TILE, &tmap_w, sb * Q4_K_BYTES, n0, sbase + BAR_RAW_FULL + 8 * q);
                    if ((sb & 1) == 0) {
                        const int g = gp % GST;
                        if (!wait_or_abort(sbase + BAR_G_EMPTY + 8 * g, ((gp / GST) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                        mbar_expect_tx(sbase + BAR_G_FULL_A + 8 * g, G_TILE);
                        tma_load_2d(sbase + OFF_GA + g * G_TILE, &tmap_g, (sb >> 1) * 64, m0, sbase + BAR_G_FULL_A + 8 * g);
                        ++gp;
                    }
                }
            }
            if (!ok) {
                for (int k = 0; k < RAW_STAGES; ++k) {
                    const int v = rq - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_RAW_FULL + 8 * (v % RAW_STAGES), (v / RAW_STAGES) & 1);
                }
                for (int k = 0; k < GST; ++k) {
                    const int v = gp - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_G_FULL_A + 8 * (v % GST), (v / GST) & 1);
                }
            }
        } else if ((warp == 1 || warp == 2) && lane == 0) {
            // ---------------- MMA issuers: warp 1 takes the first block of every chunk (and G),
            // warp 2 the second; each owns one of the two TMEM block-sum buffers ----------------
            const int which = warp - 1;
            int it = 0, bc = 0, gp = 0, gsb = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                for (int pr = tr.sb0 / 2; pr < (tr.sb1 + 1) / 2 && ok; ++pr, ++gp) {
                    const int g = gp % GST;
                    const uint32_t gph = (gp / GST) & 1;
                    for (int e = 0; e < 2 && ok; ++e) {
                        if (2 * pr + e >= tr.sb1) break;
                        for (int kc = 0; kc < 4 && ok; ++kc, ++it) {
                            const int s = it % STAGES;
                            const uint32_t ph = (it / STAGES) & 1;
                            if (!spin_or_abort(sbase + BAR_FULL_A + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                                !spin_or_abort(sbase + BAR_FULL_B + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                            tc_fence_after();
                            const uint64_t adesc = smem_desc_sw128(sbase + OFF_A + s * A_TILE);
                            const uint64_t bdesc = smem_desc_sw128(sbase + OFF_B + s * B_TILE);
                            {
                                // this thread's block of the chunk: block `which`, TMEM buffer `which`, use number `it`
                                const int t = which;
                                if (!spin_or_abort(sbase + BAR_TMEM_EMPTY + 8 * t, (it & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_TMEM)) { ok = false; break; }
                                tc_fence_after();
#pragma unroll
                                for (int k = 0; k < 2; ++k) {
                                    const uint64_t off = static_cast<uint64_t>((which * 64 + k * 32) >> 4);   // bytes >> 4 inside the swizzle row
                                    tc_mma_f16(tmem_base + TM_F + t * BN, adesc + off, bdesc + off, IDESC_F16, k);
                                }
                                tc_commit(sbase + BAR_TMEM_FULL + 8 * t);      // block sum complete -> epilogue
                            }
                            tc_commit(sbase + BAR_EMPTY + 8 * s);              // operands consumed -> producers (needs both threads)
                        }
                        if (!ok) break;
                        if (which != 0) continue;
                        // G of this super-block: K = 32 bf16, the e-th half of the pair's 128-byte rows
                        if ((e == 0 && !spin_or_abort(sbase + BAR_G_FULL_A + 8 * g, gph, abort_flag, p.err, DEV_TIMEOUT_FULL)) ||
                            !spin_or_abort(sbase + BAR_G_FULL_B + 16 * g + 8 * e, gph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                            !spin_or_abort(sbase + BAR_GT_EMPTY, (gsb & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_TMEM)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t gadesc = smem_desc_sw128(sbase + OFF_GA + g * G_TILE);
                        const uint64_t gbdesc = smem_desc_sw128(sbase + OFF_GB + g * G_TILE);
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const uint64_t off = static_cast<uint64_t>((e * 64 + k * 32) >> 4);
                            tc_mma_f16(tmem_base + TM_G, gadesc + off, gbdesc + off, IDESC_BF16, k);
                        }
                        tc_commit(sbase + BAR_GT_FULL);
                        ++gsb;
                    }
                    if (ok && which == 0) tc_commit(sbase + BAR_G_EMPTY + 8 * g);     // the pair's G operands are consumed
                }
            }
        }
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
        // ---------------- converters: thread r owns weight row n0 + r ----------------
        const int r = threadIdx.x - 128;
        int it = 0, gp = 0, rq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const uint4 zero4 = make_uint4(0, 0, 0, 0);
            const TileRef tr = tile_ref(p, tile);
            for (int pr = tr.sb0 / 2; pr < (tr.sb1 + 1) / 2 && ok; ++pr, ++gp) {
                const int g = gp % GST;
                {
                    const uint32_t gph = ((gp / GST) & 1) ^ 1;
                    if (!wait_or_abort(sbase + BAR_G_EMPTY + 8 * g, gph, abort_flag, p.err, DEV_TIMEOUT_EMPTY) ||
                        !wait_or_abort(sbase + BAR_G_TAB_EMPTY + 8 * g, gph, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                }
                for (int e = 0; e < 2 && ok; ++e) {
                    const int sb = 2 * pr + e;
                    const bool exists = sb < tr.sb1;
                    const int q = rq % RAW_STAGES;
                    const uint32_t raw = sbase + OFF_RAW + q * RAW_TILE + r * Q4_K_BYTES;      // this row's 144 bytes
                    if (exists && !wait_or_abort(sbase + BAR_RAW_FULL + 8 * q, (rq / RAW_STAGES) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                    const uint4 hdr = exists ? lds128(raw) : zero4;
                    const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
                    // 6-bit scales / mins, eight of each (Laplace src/kernels.h:82-90), one per byte
                    const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, mn_lo = hdr.z & 0x3f3f3f3fu;
                    const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
                    const uint32_t mn_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
                    {
                        // G operand: k'' = 3j + piece  ->  mn_j as bf16 (exact), 24 values + 8 zeros = 64 bytes,
                        // the e-th half of row r. Two j per three 32-bit words: (a,a) (a,b) (b,b).
                        uint32_t gw[16];
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const uint32_t mw = jj < 2 ? mn_lo : mn_hi;
                            const uint32_t a = (mw >> (16 * (jj & 1))) & 0xff, b = (mw >> (16 * (jj & 1) + 8)) & 0xff;
                            const uint32_t ab = __float_as_uint(static_cast<float>(a)) >> 16;     // bf16 bits of a small integer
                            const uint32_t bb = __float_as_uint(static_cast<float>(b)) >> 16;
                            gw[3 * jj] = ab | (ab << 16);
                            gw[3 * jj + 1] = ab | (bb << 16);
                            gw[3 * jj + 2] = bb | (bb << 16);
                        }
                        gw[12] = gw[13] = gw[14] = gw[15] = 0;
                        uint8_t* grow = smem + OFF_GB + g * G_TILE + r * 128;
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            *reinterpret_cast<uint4*>(grow + (((e * 4 + q) ^ (r & 7)) << 4)) =
                                make_uint4(gw[4 * q], gw[4 * q + 1], gw[4 * q + 2], gw[4 * q + 3]);
                        float* gtab = reinterpret_cast<float*>(smem + OFF_GTAB + g * GTAB_BYTES) + e * 2 * BN;
                        gtab[r] = d;
                        gtab[BN + r] = dmin;
                        fence_proxy_async();          // generic-proxy stores -> visible to the tensor core's reads
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sbase + BAR_G_FULL_B + 16 * g + 8 * e);
                    }
                    if (!exists) continue;
#pragma unroll
                    for (int c = 0; c < 4; ++c, ++it) {
                        const uint4 qa = lds128(raw + 16 + 32 * c), qb = lds128(raw + 32 + 32 * c);
                        const int s = it % STAGES;
                        if (!wait_or_abort(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
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
                        uint8_t* brow = smem + OFF_B + s * B_TILE + r * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<uint4*>(brow + ((j ^ (r & 7)) << 4)) = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sbase + BAR_FULL_B + 8 * s);
                    }
                    // the packed super-block has been read: its slot may be refilled
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + BAR_RAW_EMPTY + 8 * q);
                    ++rq;
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        // ---------------- epilogue: lane = token row, 64 columns per warp ----------------
        // Registers hold only the current block's sums and the super-block's partial result;
        // the running y of the tile lives in TMEM (TM_ACC) and is touched once per super-block.
        const int e8 = warp - 8;
        const int quad = e8 & 3, half = e8 >> 2;
        const uint32_t t_lane = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_acc = tmem_base + t_lane + TM_ACC + half * 64;
        const uint32_t t_g = tmem_base + t_lane + TM_G + half * 64;
        int bc = 0, gp = 0, gsb = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const TileRef tr = tile_ref(p, tile);
            const int m0 = tr.m0, n0 = tr.n0;
            const int m = m0 + quad * 32 + lane;
            int orow = p.out_row ? __ldg(p.out_row + m) : (m < p.M ? m : -1);            // row of y, -1 = padding
            if (p.out_identity && orow >= 0) orow = m;
            const bool row_live = orow >= 0;
            const float2* dxr = reinterpret_cast<const float2*>(p.dx + static_cast<size_t>(row_live ? m : 0) * (p.K / 32));
            float2 acc2[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) acc2[c] = make_float2(0.f, 0.f);
            float2 dx_n = row_live ? __ldg(dxr + tr.sb0 * 4) : make_float2(0.f, 0.f);
            for (int pr = tr.sb0 / 2; pr < (tr.sb1 + 1) / 2 && ok; ++pr, ++gp) {
                const int g = gp % GST;
                const uint32_t gtab = sbase + OFF_GTAB + g * GTAB_BYTES;
                for (int e = 0; e < 2 && ok; ++e) {
                    const int sb = 2 * pr + e;
                    if (sb >= tr.sb1) break;
                    for (int kc = 0; kc < 4 && ok; ++kc) {
                        const float2 dx2 = dx_n;
                        {
                            const int nchunk = sb * 4 + kc + 1;
                            if (row_live && nchunk < tr.sb1 * 4) dx_n = __ldg(dxr + nchunk);
                        }
#pragma unroll
                        for (int blk = 0; blk < 2; ++blk, ++bc) {
                            const int t = bc & 1;
                            if (!wait_or_abort(sbase + BAR_TMEM_FULL + 8 * t, (bc >> 1) & 1, abort_flag, p.err, DEV_TIMEOUT_MMA)) { ok = false; break; }
                            tc_fence_after();
                            const float dxv = blk ? dx2.y : dx2.x;
                            const float2 dxx = make_float2(dxv, dxv);
                            const uint32_t taddr = tmem_base + t_lane + TM_F + t * BN + half * 64;
                            // all 64 columns in one round trip, then the TMEM buffer goes straight back to the MMA
                            float f0[16], f1[16], f2[16], f3[16];
                            tc_ld16(taddr, f0);
                            tc_ld16(taddr + 16, f1);
                            tc_ld16(taddr + 32, f2);
                            tc_ld16(taddr + 48, f3);
                            tc_wait_ld();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(sbase + BAR_TMEM_EMPTY + 8 * t);
#pragma unroll
                            for (int c2 = 0; c2 < 8; ++c2) {
                                acc2[c2] = __ffma2_rn(dxx, make_float2(f0[2 * c2], f0[2 * c2 + 1]), acc2[c2]);
                                acc2[8 + c2] = __ffma2_rn(dxx, make_float2(f1[2 * c2], f1[2 * c2 + 1]), acc2[8 + c2]);
                                acc2[16 + c2] = __ffma2_rn(dxx, make_float2(f2[2 * c2], f2[2 * c2 + 1]), acc2[16 + c2]);
                                acc2[24 + c2] = __ffma2_rn(dxx, make_float2(f3[2 * c2], f3[2 * c2 + 1]), acc2[24 + c2]);
                            }
                        }
                    }
                    if (!ok) break;
                    // end of a super-block: y += d * partial - dmin * G, 16 columns at a time through TMEM
                    if (!wait_or_abort(sbase + BAR_GT_FULL, gsb & 1, abort_flag, p.err, DEV_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t dtab = gtab + (e * 2 * BN + half * 64) * 4, mtab = dtab + BN * 4;
                    const bool first = sb == tr.sb0;
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) {
                        float gv[16], av[16];
                        tc_ld16(t_g + 16 * gq, gv);
                        if (!first) {
                            tc_ld16(t_acc + 16 * gq, av);
                        } else {
#pragma unroll
                            for (int c = 0; c < 16; ++c) av[c] = 0.f;
                        }
                        tc_wait_ld();
                        if (gq == 3) {
                            // G is in registers: the MMA may overwrite it with the next super-block's
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(sbase + BAR_GT_EMPTY);
                        }
#pragma unroll
                        for (int c4 = 0; c4 < 4; ++c4) {
                            const uint4 d4 = lds128(dtab + (16 * gq + 4 * c4) * 4), m4 = lds128(mtab + (16 * gq + 4 * c4) * 4);
                            const float dd[4] = {__uint_as_float(d4.x), __uint_as_float(d4.y), __uint_as_float(d4.z), __uint_as_float(d4.w)};
                            const float mm[4] = {__uint_as_float(m4.x), __uint_as_float(m4.y), __uint_as_float(m4.z), __uint_as_float(m4.w)};
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const int c = 4 * c4 + k;
                                const float part = (c & 1) ? acc2[8 * gq + (c >> 1)].y : acc2[8 * gq + (c >> 1)].x;
                                av[c] = fmaf(-mm[k], gv[c], fmaf(dd[k], part, av[c]));
                            }
                        }
                        tc_st16(t_acc + 16 * gq, av);
                    }
                    tc_wait_st();
#pragma unroll
                    for (int c = 0; c < 32; ++c) acc2[c] = make_float2(0.f, 0.f);
                    ++gsb;
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + BAR_G_TAB_EMPTY + 8 * g);    // the pair's d / dmin tables are free
            }
            if (ok) {
                float* ybase = p.ksplit > 1 ? p.y_part + static_cast<size_t>(tr.ks) * p.M * p.N : p.y;
                float* yr = ybase + static_cast<size_t>(row_live ? orow : 0) * p.N + n0 + half * 64;
                const bool vec = n0 + half * 64 + 64 <= p.N && (reinterpret_cast<uintptr_t>(yr) & 15) == 0;
#pragma unroll
                for (int gq = 0; gq < 4; ++gq) {
                    float av[16];
                    tc_ld16(t_acc + 16 * gq, av);        // warp-wide: every lane takes part, live row or not
                    tc_wait_ld();
                    if (!row_live) continue;
                    if (vec) {
#pragma unroll
                        for (int c4 = 0; c4 < 4; ++c4)
                            *reinterpret_cast<float4*>(yr + 16 * gq + 4 * c4) = make_float4(av[4 * c4], av[4 * c4 + 1], av[4 * c4 + 2], av[4 * c4 + 3]);
                    } else {
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            if (n0 + half * 64 + 16 * gq + c < p.N) yr[16 * gq + c] = av[c];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

#include "lp_gemm_tc_q6k.cuh"

// ---- activation quantizer for both kernels -------------------------------------
// Same arithmetic as quantize_act_kernel (Laplace src/matmul_simd.cpp:348-410); the int8
// values are written as fp16 (exact) in the operand's k order: within every four
// consecutive values, (0, 2, 1, 3). Rows M..M_pad-1 of the operand are zero.
// sum = d * (integer block sum) is written as three bf16 pieces whose sum is sum to 24
// bits: ag[m][sb*32 + 3*j + piece] for block j of super-block sb (the buffer is zeroed
// before the launch, so the 8 padding entries per super-block stay 0).
__global__ void __launch_bounds__(256) quantize_act_f16_kernel(const float* __restrict__ x, int M, int K, long long n_blocks,
                                                               __half* __restrict__ aq, float* __restrict__ dx,
                                                               __nv_bfloat16* __restrict__ ag, int ag_stride) {
    const int t8 = threadIdx.x & 7;
    const long long groups = static_cast<long long>(gridDim.x) * (blockDim.x >> 3);
    const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x >> 3) + (threadIdx.x >> 3);
    const long long iters = (n_blocks + groups - 1) / groups;
    const long long live_blocks = static_cast<long long>(M) * (K / 32);
    for (long long itn = 0; itn < iters; ++itn) {
        const long long b = first + itn * groups;
        const bool in_range = b < n_blocks, live = b < live_blocks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = __ldg(reinterpret_cast<const float4*>(x + b * 32) + t8);
        uint32_t packed; int hs;
        const float d = quantize_block_8lanes(v, packed, hs);
        const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
        if (!in_range) continue;
        const int q0 = static_cast<int8_t>(packed & 0xff), q1 = static_cast<int8_t>((packed >> 8) & 0xff);
        const int q2 = static_cast<int8_t>((packed >> 16) & 0xff), q3 = static_cast<int8_t>(packed >> 24);
        const __half2 lo = __halves2half2(__int2half_rn(q0), __int2half_rn(q2));
        const __half2 hi = __halves2half2(__int2half_rn(q1), __int2half_rn(q3));
        uint2 out;
        out.x = *reinterpret_cast<const uint32_t*>(&lo);
        out.y = *reinterpret_cast<const uint32_t*>(&hi);
        reinterpret_cast<uint2*>(aq + b * 32)[t8] = out;
        if (t8 == 0 && live) {
            const short slo = static_cast<short>(hs), shi = static_cast<short>(hs_hi);
            dx[b] = d;
            const float sum = d * static_cast<float>(static_cast<int>(slo) + static_cast<int>(shi));
            const __nv_bfloat16 p0 = __float2bfloat16_rn(sum);
            const float r1 = sum - __bfloat162float(p0);
            const __nv_bfloat16 p1 = __float2bfloat16_rn(r1);
            const __nv_bfloat16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
            const int bpr = K / 32;
            const long long m = b / bpr;
            const int kb = static_cast<int>(b - m * bpr);
            __nv_bfloat16* dst = ag + m * ag_stride + (kb >> 3) * 32 + 3 * (kb & 7);
            dst[0] = p0; dst[1] = p1; dst[2] = p2;
        }
    }
}

// Scratch owned by this translation unit. A buffer that has been handed to a launch may be baked into a
// captured CUDA graph (its address and the tensor maps built from it), so a buffer is never freed when a
// larger one is needed: superseded buffers are kept until laplace_cuda_shutdown. Growing calls the
// allocator, which is illegal while the call's stream is being captured: such a call is refused and the
// capture stays valid (run the call once outside the capture first, as a warm-up, so that the buffer exists).
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

}  // namespace

void release_gemm_tc_scratch() { g_scratch.release(); }

bool gemm_tc_supports(uint32_t type, int M, int K, int N) {
    if (M <= 8 || N <= 0) return false;
    if (type == LAPLACE_TYPE_Q4_K) return K % 256 == 0;
    // Q6_K rows are 210 bytes per super-block: the row pitch is a 16-byte multiple (what a tensor map
    // needs) only when K is a multiple of 8 super-blocks
    if (type == LAPLACE_TYPE_Q6_K) return K % 2048 == 0;
    return false;
}

namespace {

// Scratch layout of one call: fp16 activation operand, activation scales, bf16 pieces of sum_x.
struct ScratchPlan {
    size_t m_pad, aq_bytes, sc_bytes, ag_bytes, part_bytes;
    int    tiles_m, tiles_n, n_pairs;
    int    ksplit, sb_per;           // split-K: CTAs per output tile, super-blocks per CTA (1, K/256: no split)
    size_t total() const { return aq_bytes + sc_bytes + ag_bytes + part_bytes; }
};
ScratchPlan plan_scratch(int M, int K, int N, uint32_t type = LAPLACE_TYPE_Q4_K, bool allow_split = true) {
    ScratchPlan s;
    s.tiles_m = (M + BM - 1) / BM;
    s.tiles_n = (N + BN - 1) / BN;
    s.m_pad = static_cast<size_t>(s.tiles_m) * BM;
    s.n_pairs = (K / 256 + 1) / 2;
    s.aq_bytes = (s.m_pad * K * sizeof(__half) + 255) & ~size_t(255);
    s.sc_bytes = (static_cast<size_t>(M) * (K / 32) * sizeof(float) + 255) & ~size_t(255);
    s.ag_bytes = (s.m_pad * s.n_pairs * 64 * sizeof(__nv_bfloat16) + 255) & ~size_t(255);
    // Few output tiles (narrow matrices, or a slice of one on each of several GPUs) leave most SMs idle: let up to
    // four CTAs share a tile, each over an even number of super-blocks; partial results are added by a second kernel
    // in a fixed order, so the result stays reproducible.
    const int nsb = K / 256, out_tiles = s.tiles_m * s.tiles_n, sms = ctx().sm_count;
    s.ksplit = 1; s.sb_per = nsb; s.part_bytes = 0;
    // (Splitting calls that already fill the machine - e.g. 448 tiles, to even out the last wave - was measured
    // slower: 0.259 -> 0.280 ms; only calls that leave at least half the SMs idle are split.)
    if (allow_split && nsb >= 8 && out_tiles * 2 <= sms) {
        // cost in "super-blocks of one tile" (~4.7 us each): waves x super-blocks per CTA, plus the reduction's
        // traffic ((slices + 1) x M x N floats at ~6 TB/s).
        double best = static_cast<double>((out_tiles + sms - 1) / sms) * nsb;
        for (int want = 2; want <= 4; ++want) {
            int per = (nsb + want - 1) / want;
            per += per & 1;
            if (per < 4) per = 4;
            const int ks = (nsb + per - 1) / per;
            if (ks < 2) continue;
            const double waves = static_cast<double>((static_cast<long long>(out_tiles) * ks + sms - 1) / sms);
            const double reduce_us = static_cast<double>(ks + 1) * M * N * 4.0 / 6.0e6;
            const double cost = waves * per + reduce_us / 4.7 + 0.5;
            if (cost < best * 0.97) {
                best = cost;
                s.ksplit = ks; s.sb_per = per;
                s.part_bytes = (static_cast<size_t>(ks) * M * N * sizeof(float) + 255) & ~size_t(255);
            }
        }
    }
    return s;
}

// y = sum of the k-slices' partial results, slices added in index order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float4* __restrict__ part, long long n4, int ksplit,
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

// One launch of a tensor-core kernel over prepared operands.
struct TcLaunch {
    const uint8_t* w; uint32_t type; float* y; int M, K, N;
    size_t rows_pad;          // rows of the operand buffers aq / ag
    long long w_rows;         // rows of the (stacked) weight matrix
    __half* aq; float* dx; __nv_bfloat16* ag;
    const int4* tile_tab; const int* n_tiles_dev; const int* out_row; int out_identity;
    int tiles_m, tiles_n, grid;
    int ksplit, sb_per; float* y_part;
};

int run_tc_kernel(const TcLaunch& L, cudaStream_t st) {
    Context& c = ctx();
    const int K = L.K, n_pairs = (K / 256 + 1) / 2;
    const uint32_t type = L.type;
    // 2-D tensor maps: the fp16 operand (inner dimension K) and the bf16 pieces of sum_x
    // (inner dimension 64 per pair of super-blocks); outer dimension tokens.
    CUtensorMap tmap, tmap_g, tmap_w;
    {
        // The driver entry point is looked up at run time so that the library does not link libcuda.
        using encode_fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        static encode_fn cuTensorMapEncodeTiled = nullptr;
        if (!cuTensorMapEncodeTiled) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
            if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
                return fail(LAPLACE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
            cuTensorMapEncodeTiled = reinterpret_cast<encode_fn>(fn);
        }
        const cuuint32_t box[2] = {BKC, BM};
        const cuuint32_t estr[2] = {1, 1};
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(L.rows_pad)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * sizeof(__half)};
        CUresult r = cuTensorMapEncodeTiled(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, L.aq, dims, strides, box, estr,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(LAPLACE_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
        const cuuint64_t gdims[2] = {static_cast<cuuint64_t>(n_pairs) * 64, static_cast<cuuint64_t>(L.rows_pad)};
        const cuuint64_t gstrides[1] = {static_cast<cuuint64_t>(n_pairs) * 64 * sizeof(__nv_bfloat16)};
        r = cuTensorMapEncodeTiled(&tmap_g, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, L.ag, gdims, gstrides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(LAPLACE_ERR_CUDA, "cuTensorMapEncodeTiled (G) failed (%d)", static_cast<int>(r));
        // the packed weights as bytes: rows of rb bytes (stacked experts are just more rows), boxes of 128 rows
        // x one super-block (144 bytes, or 240 for Q6_K: 210 + alignment slop)
        const cuuint64_t wdims[2] = {static_cast<cuuint64_t>(row_bytes(type, K)), static_cast<cuuint64_t>(L.w_rows)};
        const cuuint64_t wstrides[1] = {static_cast<cuuint64_t>(row_bytes(type, K))};
        const cuuint32_t wbox[2] = {static_cast<cuuint32_t>(type == LAPLACE_TYPE_Q6_K ? q6::RAW_PITCH : Q4_K_BYTES), BN};
        r = cuTensorMapEncodeTiled(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(L.w), wdims, wstrides, wbox, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(LAPLACE_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed (%d)", static_cast<int>(r));
    }

    TcParams p{};
    p.w = L.w; p.dx = L.dx; p.y = L.y; p.err = c.d_err;
    p.M = L.M; p.N = L.N; p.K = K; p.rb = static_cast<uint32_t>(row_bytes(type, K));
    p.tiles_m = L.tiles_m; p.tiles_n = L.tiles_n;
    p.tile_tab = L.tile_tab; p.n_tiles_dev = L.n_tiles_dev; p.out_row = L.out_row; p.out_identity = L.out_identity;
    p.ksplit = L.ksplit > 1 ? L.ksplit : 1; p.sb_per = L.ksplit > 1 ? L.sb_per : K / 256; p.y_part = L.y_part;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(q6::gemm_q6k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(q6::SMEM_BYTES));
        if (e != cudaSuccess) return cuda_check(e, "cudaFuncSetAttribute gemm_tc");
        configured = true;
    }
    if (type == LAPLACE_TYPE_Q6_K)
        q6::gemm_q6k_tc_kernel<<<L.grid, THREADS, q6::SMEM_BYTES, st>>>(tmap, tmap_w, p);
    else
        gemm_q4k_tc_kernel<<<L.grid, THREADS, SMEM_BYTES, st>>>(tmap, tmap_g, tmap_w, p);
    c.launches++;
    c.last_path = 2;
    return cuda_check(cudaGetLastError(), "gemm_tc launch");
}

// Quantizes x into `scratch` (device memory of at least plan.total() bytes, 256-byte aligned)
// and runs the tensor-core kernel. Allocates nothing.
int gemm_tc_on_scratch(uint8_t* scratch, const ScratchPlan& sp, const float* x, const uint8_t* w, uint32_t type, float* y,
                       int M, int K, int N, cudaStream_t st) {
    Context& c = ctx();
    const int tiles_m = sp.tiles_m, tiles_n = sp.tiles_n, n_pairs = sp.n_pairs;
    const size_t m_pad = sp.m_pad, bpr = static_cast<size_t>(K / 32);
    const size_t aq_bytes = sp.aq_bytes, sc_bytes = sp.sc_bytes, ag_bytes = sp.ag_bytes;
    int rc;
    __half* aq = reinterpret_cast<__half*>(scratch);
    float* dx = reinterpret_cast<float*>(scratch + aq_bytes);
    __nv_bfloat16* ag = reinterpret_cast<__nv_bfloat16*>(scratch + aq_bytes + sc_bytes);

    {
        if ((rc = cuda_check(cudaMemsetAsync(ag, 0, ag_bytes, st), "cudaMemsetAsync"))) return rc;
        const long long n_blocks = static_cast<long long>(m_pad) * bpr;
        long long want = (n_blocks + 31) / 32;
        const long long cap = static_cast<long long>(c.sm_count) * 8;
        const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
        quantize_act_f16_kernel<<<grid, 256, 0, st>>>(x, M, K, n_blocks, aq, dx, ag, n_pairs * 64);
        c.launches++;
        if ((rc = cuda_check(cudaGetLastError(), "quantize_act_f16 launch"))) return rc;
    }

    TcLaunch L{};
    L.w = w; L.type = type; L.y = y; L.M = M; L.K = K; L.N = N;
    L.rows_pad = m_pad; L.w_rows = N;
    L.aq = aq; L.dx = dx; L.ag = ag;
    L.tiles_m = tiles_m; L.tiles_n = tiles_n;
    L.ksplit = sp.ksplit; L.sb_per = sp.sb_per;
    L.y_part = sp.ksplit > 1 ? reinterpret_cast<float*>(scratch + aq_bytes + sc_bytes + ag_bytes) : nullptr;
    const int n_tiles = tiles_m * tiles_n * (sp.ksplit > 1 ? sp.ksplit : 1);
    L.grid = n_tiles < c.sm_count ? n_tiles : c.sm_count;
    if ((rc = run_tc_kernel(L, st))) return rc;
    if (sp.ksplit > 1) {
        const long long n = static_cast<long long>(M) * N;
        if (n % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
            long long blocks = (n / 4 + 255) / 256;
            if (blocks > static_cast<long long>(c.sm_count) * 8) blocks = static_cast<long long>(c.sm_count) * 8;
            splitk_reduce_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(reinterpret_cast<const float4*>(L.y_part), n / 4, sp.ksplit,
                                                                        reinterpret_cast<float4*>(y));
            c.launches++;
            return cuda_check(cudaGetLastError(), "splitk_reduce launch");
        }
        return fail(LAPLACE_ERR_STATE, "gemm: internal planning error (split-K needs M*N %% 4 == 0 and an aligned y)");
    }
    return LAPLACE_OK;
}

int check_gemm_tc_args(const float* x, const uint8_t* w, uint32_t type, int M, int K, int N) {
    if (!gemm_tc_supports(type, M, K, N)) return LAPLACE_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(w) & 15) return fail(LAPLACE_ERR_ARG, "gemm: weights must be 16-byte aligned on the device");
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(LAPLACE_ERR_ARG, "gemm: x not 16-byte aligned");
    return LAPLACE_OK;
}

}  // namespace

int launch_gemm_tc(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, cudaStream_t st) {
    int rc = check_gemm_tc_args(x, w, type, M, K, N);
    if (rc) return rc;
    // split-K only when its result buffer can be added up with vector loads
    const bool can_split = (static_cast<long long>(M) * N) % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    const ScratchPlan sp = plan_scratch(M, K, N, type, can_split);
    if ((rc = g_scratch.ensure(sp.total(), st))) return rc;
    return gemm_tc_on_scratch(static_cast<uint8_t*>(g_scratch.p), sp, x, w, type, y, M, K, N, st);
}

#include "lp_moe_grouped.cuh"

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
constexpr size_t NOALLOC_SCRATCH_BYTES = 10u << 20;    // 10 MiB: e.g. Q4_K, M = 512, K = 4096 needs 8.2 MiB
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
    const bool sa = gemm_sa_supports(type, M, K, N);          // which prefill kernel laplace_cuda_gemm_dev would run
    int rc = sa ? LAPLACE_OK : check_gemm_tc_args(x, w, type, M, K, N);
    if (rc == LAPLACE_UNSUPPORTED)
        return fail(LAPLACE_ERR_ARG, "gemm_noalloc: only the prefill shapes are served here (M > 8; Q4_K with K %% 256 == 0 or "
                                     "Q6_K with K %% 2048 == 0); decode calls (M <= 8) use no scratch at all, call "
                                     "laplace_cuda_gemm_dev");
    if (rc) return rc;
    // the same K-split as laplace_cuda_gemm_dev (hence bit-identical results) whenever its partial results fit
    // the array too; otherwise no split (results then agree to fp32 rounding)
    const bool can_split = (static_cast<long long>(M) * N) % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    ScratchPlan sp{};
    if (!sa) {
        sp = plan_scratch(M, K, N, type, can_split);
        if (sp.total() > NOALLOC_SCRATCH_BYTES) sp = plan_scratch(M, K, N, type, false);
        if (sp.total() > NOALLOC_SCRATCH_BYTES)
            return fail(LAPLACE_ERR_LIMIT, "gemm_noalloc: M=%d K=%d needs %zu bytes of scratch, the built-in array holds %zu",
                        M, K, sp.total(), NOALLOC_SCRATCH_BYTES);
    }
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
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : c.stream;
    if (sa) return launch_gemm_sa_prealloc(g_noalloc_ptr, NOALLOC_SCRATCH_BYTES, x, w, type, y, M, K, N, st);
    return gemm_tc_on_scratch(g_noalloc_ptr, sp, x, w, type, y, M, K, N, st);
}
