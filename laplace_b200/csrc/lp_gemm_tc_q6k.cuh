// lp_gemm_tc_q6k.cuh - prefill GEMM for Q6_K weights on the tensor cores. Included by
// lp_gemm_tc.cu (inside namespace lp { namespace { ... } }) after the shared tcgen05 / TMA
// wrappers. Replaces gemm_int<dot_row_q6_k_int_neon> of Laplace's NEON back-end
// (src/matmul_simd.cpp:285-342, 432-455) for M > 8.
//
// Q6_K has one int8 scale per 16 values (src/kernels.h:46-54: ql[128], qh[64], scales[16],
// fp16 d). The weight operand carries w = sc * (q6 - 32), |w| <= 4096, which fp16 does not
// hold exactly, so it is split into two exact operands, w = H + L with
//   u = w + 4096 in [0, 8192],  H = 32 * ((u >> 5) - 128),  L = u & 31,
// and every 16-value step issues two MMAs into the same accumulator: F = A*H + A*L. All
// products and partial sums stay below 2^24, so F is the exact integer
// sum_k q_x[k] * sc * (q6[k] - 32) of a 32-value block, the same integer the reference gets
// from vmull_s8/vmlal_s16 before its float conversion. Then, as for Q4_K,
//   y[m,n] += d[n,sb] * sum_{j<8} d_x[m,8sb+j] * F[m,n,8sb+j]      (no min term in Q6_K).
//
// Roles (512 threads, one persistent CTA per SM, 128x128 tiles, 64 k per stage):
//   warp 0      TMA: activation tiles (the same fp16 operand as the Q4_K kernel)
//   warps 1, 2  MMA issue, one 32-block of every chunk each, one TMEM buffer each
//   warp 3      TMA: packed super-blocks, 128 rows x 240 bytes (210 + alignment slop)
//   warps 4-7   converters: lane = (row, 16-byte piece of the operand row)
//   warps 8-15  epilogue, running y in TMEM
namespace q6 {

constexpr int STAGES = 3;
constexpr int RAW_STAGES = 2;
constexpr int RAW_PITCH = 240;                     // bytes per row in a raw stage: 210 + up to 14 of misalignment, 16-byte multiple
constexpr int RAW_TILE = BN * RAW_PITCH;           // 30 KB
constexpr int DT = 4;                              // ring of per-super-block d tables
constexpr uint32_t OFF_A = 0;
constexpr uint32_t OFF_BH = OFF_A + STAGES * A_TILE;
constexpr uint32_t OFF_BL = OFF_BH + STAGES * B_TILE;
constexpr uint32_t OFF_RAW = OFF_BL + STAGES * B_TILE;
constexpr uint32_t OFF_DTAB = OFF_RAW + RAW_STAGES * RAW_TILE;
constexpr uint32_t OFF_BAR = OFF_DTAB + DT * BN * 4;
constexpr uint32_t BAR_FULL_A = OFF_BAR, BAR_FULL_B = BAR_FULL_A + 8 * STAGES, BAR_EMPTY = BAR_FULL_B + 8 * STAGES,
                   BAR_TMEM_FULL = BAR_EMPTY + 8 * STAGES, BAR_TMEM_EMPTY = BAR_TMEM_FULL + 16,
                   BAR_RAW_FULL = BAR_TMEM_EMPTY + 16, BAR_RAW_EMPTY = BAR_RAW_FULL + 8 * RAW_STAGES,
                   BAR_DT_FULL = BAR_RAW_EMPTY + 8 * RAW_STAGES, BAR_DT_EMPTY = BAR_DT_FULL + 8 * DT,
                   OFF_TMEM_PTR = BAR_DT_EMPTY + 8 * DT, OFF_ABORT = OFF_TMEM_PTR + 8;
constexpr uint32_t SMEM_BYTES = OFF_ABORT + 8 + 1024;
constexpr uint32_t TM_F = 0, TM_ACC = 256;
static_assert(SMEM_BYTES <= 227 * 1024, "Q6_K GEMM: shared memory budget");
static_assert(OFF_RAW % 128 == 0 && RAW_TILE % 128 == 0, "TMA destinations are 128-byte aligned");

// 8 bytes from a 2-byte-aligned shared address: three aligned words and two funnel shifts.
__device__ __forceinline__ void lds8B_align2(uint32_t addr, uint32_t& lo, uint32_t& hi) {
    const uint32_t base = addr & ~3u, sh = (addr & 3u) * 8u;
    const uint32_t w0 = lds32(base), w1 = lds32(base + 4), w2 = lds32(base + 8);
    lo = __funnelshift_r(w0, w1, sh);
    hi = __funnelshift_r(w1, w2, sh);
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_q6k_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_ABORT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sbase + BAR_FULL_A + 8 * s, 1);
            mbar_init(sbase + BAR_FULL_B + 8 * s, 4);        // one arrive per converter warp
            mbar_init(sbase + BAR_EMPTY + 8 * s, 2);         // tcgen05.commit from each MMA thread
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(sbase + BAR_TMEM_FULL + 8 * t, 1);
            mbar_init(sbase + BAR_TMEM_EMPTY + 8 * t, 8);    // one arrive per epilogue warp
        }
        for (int q = 0; q < RAW_STAGES; ++q) {
            mbar_init(sbase + BAR_RAW_FULL + 8 * q, 1);
            mbar_init(sbase + BAR_RAW_EMPTY + 8 * q, 4);
        }
        for (int d = 0; d < DT; ++d) {
            mbar_init(sbase + BAR_DT_FULL + 8 * d, 4);
            mbar_init(sbase + BAR_DT_EMPTY + 8 * d, 8);
        }
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
                for (int k = 0; k < STAGES; ++k) {
                    const int v = it - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_FULL_A + 8 * (v % STAGES), (v / STAGES) & 1);
                }
            }
        } else if (warp == 3 && lane == 0) {
            // ---------------- TMA producer: packed super-blocks ----------------
            // A super-block starts at byte 210*sb of its row, which is only 2-byte aligned; the copy
            // starts at the 16-byte boundary below it and the converters skip the difference.
            // Rows past N and bytes past the row end are zero-filled by the copy engine.
            int rq = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                const int n0 = tr.wrow0 + tr.n0;
                for (int sb = tr.sb0; sb < tr.sb1; ++sb, ++rq) {
                    const int q = rq % RAW_STAGES;
                    if (!wait_or_abort(sbase + BAR_RAW_EMPTY + 8 * q, ((rq / RAW_STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(sbase + BAR_RAW_FULL + 8 * q, RAW_TILE);
                    tma_load_2d(sbase + OFF_RAW + q * RAW_TILE, &tmap_w, (sb * Q6_K_BYTES) & ~15, n0, sbase + BAR_RAW_FULL + 8 * q);
                }
            }
            if (!ok) {
                for (int k = 0; k < RAW_STAGES; ++k) {
                    const int v = rq - 1 - k;
                    if (v >= 0) mbar_wait_bounded(sbase + BAR_RAW_FULL + 8 * (v % RAW_STAGES), (v / RAW_STAGES) & 1);
                }
            }
        } else if ((warp == 1 || warp == 2) && lane == 0) {
            // ---------------- MMA issuers: block `which` of every chunk, TMEM buffer `which` ----------------
            const int which = warp - 1;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const TileRef tr = tile_ref(p, tile);
                for (int kc = tr.sb0 * 4; kc < tr.sb1 * 4 && ok; ++kc, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!spin_or_abort(sbase + BAR_FULL_A + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                        !spin_or_abort(sbase + BAR_FULL_B + 8 * s, ph, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                        !spin_or_abort(sbase + BAR_TMEM_EMPTY + 8 * which, (it & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_TMEM)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = smem_desc_sw128(sbase + OFF_A + s * A_TILE);
                    const uint64_t hdesc = smem_desc_sw128(sbase + OFF_BH + s * B_TILE);
                    const uint64_t ldesc = smem_desc_sw128(sbase + OFF_BL + s * B_TILE);
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint64_t off = static_cast<uint64_t>((which * 64 + k * 32) >> 4);
                        tc_mma_f16(tmem_base + TM_F + which * BN, adesc + off, hdesc + off, IDESC_F16, k);
                        tc_mma_f16(tmem_base + TM_F + which * BN, adesc + off, ldesc + off, IDESC_F16, 1);
                    }
                    tc_commit(sbase + BAR_TMEM_FULL + 8 * which);
                    tc_commit(sbase + BAR_EMPTY + 8 * s);
                }
            }
        }
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
        // ---------------- converters ----------------
        // One work item = 8 consecutive k of one weight row = one 16-byte piece of the H operand row
        // and one of the L operand row. A warp takes 4 rows x 8 pieces per step, 8 steps per chunk.
        const int cw = warp - 4;
        const int piece = lane & 7, row_in_step = lane >> 3;
        const int t = piece >> 2, pp = piece & 3;           // block of the chunk, 8-value group inside the block
        int it = 0, rq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const TileRef tr = tile_ref(p, tile);
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++rq) {
                const int q = rq % RAW_STAGES, dsl = rq % DT;
                if (!wait_or_abort(sbase + BAR_RAW_FULL + 8 * q, (rq / RAW_STAGES) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL) ||
                    !wait_or_abort(sbase + BAR_DT_EMPTY + 8 * dsl, ((rq / DT) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                const uint32_t raw = sbase + OFF_RAW + q * RAW_TILE + ((sb * Q6_K_BYTES) & 15);
                {
                    // the super-block's fp16 d of row 32*cw + lane -> fp32 table for the epilogue
                    const int r = 32 * cw + lane;
                    reinterpret_cast<float*>(smem + OFF_DTAB + dsl * BN * 4)[r] = half_bits_to_float(lds16(raw + r * RAW_PITCH + 208));
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + BAR_DT_FULL + 8 * dsl);
                }
#pragma unroll 1
                for (int c = 0; c < 4; ++c, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort(sbase + BAR_EMPTY + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, p.err, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    const int h = c >> 1, nib = c & 1, g = 2 * nib + t;        // activation block of the super-block: 4h + g
                    const uint32_t ql_off = 64 * h + 32 * t + 8 * pp, qh_off = 128 + 32 * h + 8 * pp;
                    const uint32_t sc_off = 192 + 8 * h + 2 * g + (pp >> 1);
                    const int nshift = 4 * nib, hshift = 2 * g;
#pragma unroll 2
                    for (int i = 0; i < 8; ++i) {
                        const int r = 32 * cw + 4 * i + row_in_step;
                        const uint32_t rowaddr = raw + r * RAW_PITCH;
                        uint32_t a[2], b[2];
                        lds8B_align2(rowaddr + ql_off, a[0], a[1]);
                        lds8B_align2(rowaddr + qh_off, b[0], b[1]);
                        const int sc = lds_s8(rowaddr + sc_off);
                        const uint32_t cc = static_cast<uint32_t>(4096 - 32 * sc) * 0x00010001u;
                        uint32_t hw[4], lw[4];
#pragma unroll
                        for (int w = 0; w < 2; ++w) {
                            const uint32_t q6 = ((a[w] >> nshift) & 0x0f0f0f0fu) | (((b[w] >> hshift) << 4) & 0x30303030u);
                            const uint32_t e02 = q6 & 0x00ff00ffu, e13 = (q6 >> 8) & 0x00ff00ffu;
                            // both 16-bit lanes: u = sc * (q6 - 32) + 4096 in [0, 8192]; the 32-bit product cannot borrow
                            const uint32_t u02 = e02 * static_cast<uint32_t>(sc) + cc, u13 = e13 * static_cast<uint32_t>(sc) + cc;
                            // (v | 0x7800) is fp16(32768 + 32 v), (v | 0x6400) is fp16(1024 + v)
                            const uint32_t h02 = ((u02 >> 5) & 0x01ff01ffu) | 0x78007800u, h13 = ((u13 >> 5) & 0x01ff01ffu) | 0x78007800u;
                            const uint32_t l02 = (u02 & 0x001f001fu) | 0x64006400u, l13 = (u13 & 0x001f001fu) | 0x64006400u;
                            const __half2 hoff = __half2half2(__float2half_rn(-36864.f)), loff = __half2half2(__float2half_rn(-1024.f));
                            __half2 x;
                            x = __hadd2(*reinterpret_cast<const __half2*>(&h02), hoff); hw[2 * w] = *reinterpret_cast<uint32_t*>(&x);
                            x = __hadd2(*reinterpret_cast<const __half2*>(&h13), hoff); hw[2 * w + 1] = *reinterpret_cast<uint32_t*>(&x);
                            x = __hadd2(*reinterpret_cast<const __half2*>(&l02), loff); lw[2 * w] = *reinterpret_cast<uint32_t*>(&x);
                            x = __hadd2(*reinterpret_cast<const __half2*>(&l13), loff); lw[2 * w + 1] = *reinterpret_cast<uint32_t*>(&x);
                        }
                        const uint32_t dst = s * B_TILE + r * 128 + ((piece ^ (r & 7)) << 4);
                        *reinterpret_cast<uint4*>(smem + OFF_BH + dst) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                        *reinterpret_cast<uint4*>(smem + OFF_BL + dst) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + BAR_FULL_B + 8 * s);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + BAR_RAW_EMPTY + 8 * q);
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        // ---------------- epilogue: lane = token row, 64 columns per warp ----------------
        const int e8 = warp - 8;
        const int quad = e8 & 3, half = e8 >> 2;
        const uint32_t t_lane = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t t_acc = tmem_base + t_lane + TM_ACC + half * 64;
        int bc = 0, ds = 0;
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
            for (int sb = tr.sb0; sb < tr.sb1 && ok; ++sb, ++ds) {
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
                // end of a super-block: y += d * partial, 16 columns at a time through TMEM
                const int dsl = ds % DT;
                if (!wait_or_abort(sbase + BAR_DT_FULL + 8 * dsl, (ds / DT) & 1, abort_flag, p.err, DEV_TIMEOUT_FULL)) { ok = false; break; }
                const uint32_t dtab = sbase + OFF_DTAB + (dsl * BN + half * 64) * 4;
                const bool first = sb == tr.sb0;
#pragma unroll
                for (int gq = 0; gq < 4; ++gq) {
                    float av[16];
                    if (!first) {
                        tc_ld16(t_acc + 16 * gq, av);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int c = 0; c < 16; ++c) av[c] = 0.f;
                    }
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        const uint4 d4 = lds128(dtab + (16 * gq + 4 * c4) * 4);
                        const float dd[4] = {__uint_as_float(d4.x), __uint_as_float(d4.y), __uint_as_float(d4.z), __uint_as_float(d4.w)};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int c = 4 * c4 + k;
                            const float part = (c & 1) ? acc2[8 * gq + (c >> 1)].y : acc2[8 * gq + (c >> 1)].x;
                            av[c] = fmaf(dd[k], part, av[c]);
                        }
                    }
                    tc_st16(t_acc + 16 * gq, av);
                }
                tc_wait_st();
#pragma unroll
                for (int c = 0; c < 32; ++c) acc2[c] = make_float2(0.f, 0.f);
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + BAR_DT_EMPTY + 8 * dsl);
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

}  // namespace q6
