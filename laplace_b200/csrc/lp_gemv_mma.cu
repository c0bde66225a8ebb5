// lp_gemv_mma.cu - decode GEMV for 3..8 activation rows (the kernel takes 2..8), Q4_K weights: the integer block sums on the warp-level
// int8 tensor-core instruction.
//
// gemm_int<dot_row_q4_k_int_neon> (Laplace src/matmul_simd.cpp:226-283, 432-455) with a handful of activation rows
// streams every weight row once and forms, per 32-value block and activation row, the integer U = sum nibble * q,
// then acc += (d * sc * d_x) * U and acc_min += (dmin * m) * sum_x. The streaming kernel of lp_gemv.cu does the
// integer part with dp4a, one weight row against one or two activation rows per instruction; with 8 rows that is 32
// times the instructions of one mma.sync.m16n8k32 (16 weight rows x 8 activation rows x one 32-value block), and the
// kernel is bound by the latency of those instruction chains, not by HBM (0.16 of the copy rate at M = 8). Here:
//   - one persistent CTA per SM: a producer warp copies groups of 16 weight rows (whole rows for K <= 4096, 16
//     super-blocks of every row otherwise) into a ring of shared-memory slots, one bulk copy per row, rows staggered by
//     16 bytes so that the fragment loads below meet no bank conflicts;
//   - the activations are quantized ONCE per call by a small kernel exactly as the reference does (ActQ8: d = amax /
//     127 in fp32, q = rne(x * (1 / d)), sums from the unclamped integers) into an image of the shared-memory layout
//     in device memory, which every CTA then fetches with two bulk copies (quantizing all rows in every CTA cost 3.4 to
//     8.3 us per launch: two IEEE divisions per block, 148 times over);
//   - sixteen consumer warps share every 16-row group, each taking every sixteenth super-block: A fragment = masked nibbles
//     (u8), B fragment = activations (s8), C = the sixteen-by-eight integer block sums, bit for bit the reference's;
//     the fp32 scale chain follows in the reference's order ((d * sc) * d_x) * U and (dmin * m) * sum_x;
//   - the warps' partial results of a group meet in shared memory and are added in warp order.
// Every wait is bounded; a wait that gives up raises the status word and the CTA drains its copies and leaves.
// Measured at 4096 x 14336: 15.1-15.2 us for any row count (quantizer launch included), against 11.4 / 16.7 / 18.2 / 31.5 us
// of the dp4a kernel at 2 / 3 / 4 / 8 rows. History of the figure: 20.8-21.7 us with every CTA quantizing all rows itself
// (3.4 us at <= 4 rows, 8.3 us at 8) and with each block's loads, MMA, shuffles and fp32 chain issued one after the other
// (the arithmetic then added 5.6 us that the 8 us of streaming did not hide); 17.2 us before the consumer warps went from
// eight to sixteen.
#include "lp_common.cuh"

namespace lp {
namespace {

constexpr int CW = 16;                     // consumer warps
constexpr int THREADS = (CW + 1) * 32;     // + one producer warp
constexpr int GROUP = 16;                  // weight rows per unit (MMA M)
constexpr int SLICE_SB = 16;               // super-blocks of a row per unit
constexpr int ROW_PITCH = SLICE_SB * Q4_K_BYTES + 16;     // 2320: 16-byte aligned, 16 mod 128
constexpr int SLOT_BYTES = GROUP * ROW_PITCH;             // 37,120
constexpr int MAXM = 8;

struct MmaParams {
    const float*   x;
    const uint8_t* w;
    float*         y;
    int*           err;
    int            M, K, N;
    int            n_slots;
    uint32_t       rb;             // bytes per weight row
    uint32_t       act_stride;     // bytes per quantized activation row in shared memory (K + 16)
    uint32_t       off_act, off_ds, off_part, off_ring;
    const uint8_t* act_img;        // [8][act_stride] int8 then [K / 32][8] (d, d * sum): written by quantize_rows_kernel
    uint32_t       act_bytes, ds_bytes;
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

constexpr int MAX_K = 16384;
// The quantized activations of the call in flight (one per device; calls on different streams would race for it).
__device__ __align__(128) uint8_t g_act_img[MAXM * (MAX_K + 16) + (MAX_K / 32) * MAXM * 8];

// int8 values [8][K + 16] (rows M..7 zero) and per block and row (d, d * sum), 8 lanes per 32-value block.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ x, int M, int K, uint32_t act_stride,
                                                            uint8_t* __restrict__ img) {
    const int bpr = K >> 5, nblk = MAXM * bpr;
    uint8_t* ds = img + MAXM * act_stride;
    const int t8 = threadIdx.x & 7;
    for (int base = blockIdx.x * 32; base < nblk; base += gridDim.x * 32) {      // whole warps iterate together
        const int b = base + (threadIdx.x >> 3);
        const bool inside = b < nblk;
        const int m = inside ? b / bpr : 0, kb = inside ? b - m * bpr : 0;
        const bool live = inside && m < M;
        const float4 v = live ? __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * K + kb * 32) + t8) : make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t packed; int hs;
        const float d = quantize_block_8lanes(v, packed, hs);
        const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
        if (inside) {
            *reinterpret_cast<uint32_t*>(img + m * act_stride + kb * 32 + t8 * 4) = live ? packed : 0u;
            if (t8 == 0) {
                const int isum = static_cast<int>(static_cast<short>(hs)) + static_cast<int>(static_cast<short>(hs_hi));
                *reinterpret_cast<float2*>(ds + (static_cast<size_t>(kb) * MAXM + m) * 8) = live ? make_float2(d, d * static_cast<float>(isum)) : make_float2(0.f, 0.f);
            }
        }
    }
}

__global__ void __launch_bounds__(THREADS, 1) gemv_mma_q4k_kernel(const MmaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K / 256, n_slices = (nsb + SLICE_SB - 1) / SLICE_SB;
    // this CTA's contiguous range of 16-row groups
    const int groups = (p.N + GROUP - 1) / GROUP;
    const int g_begin = static_cast<int>(static_cast<long long>(groups) * blockIdx.x / gridDim.x);
    const int g_end = static_cast<int>(static_cast<long long>(groups) * (blockIdx.x + 1) / gridDim.x);
    const int n_units = (g_end - g_begin) * n_slices;
    auto bar_full = [&](int s) { return sbase + 8 * s; };
    auto bar_empty = [&](int s) { return sbase + 64 + 8 * s; };
    const uint32_t bar_act = sbase + 48;                   // full barriers use 0..31, empty barriers 64..95

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.n_slots; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), CW); }
        mbar_init(bar_act, 1);
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == CW) {
        // ------------------------------ producer: lane r copies row r of the unit ------------------------------
        bool gave_up = false;
        int u = 0;
        for (; u < n_units && !gave_up; ++u) {
            const int slot = u % p.n_slots, round = u / p.n_slots;
            if (round > 0) {
                bool ok = false;
                for (uint32_t it = 0; it < (1u << 22) && !ok; ++it) {
                    ok = mbar_try_wait(bar_empty(slot), (round - 1) & 1);
                    if (!ok) __nanosleep(40);
                }
                if (!ok) { gave_up = true; break; }
            }
            const int g = g_begin + u / n_slices, sl = u % n_slices;
            const int row0 = g * GROUP;
            const int sbs = (nsb - sl * SLICE_SB) < SLICE_SB ? (nsb - sl * SLICE_SB) : SLICE_SB;
            const uint32_t bytes = static_cast<uint32_t>(sbs) * Q4_K_BYTES;
            const int rows = (p.N - row0) < GROUP ? (p.N - row0) : GROUP;
            if (lane == 0) mbar_expect_tx(bar_full(slot), bytes * rows);
            __syncwarp();
            if (lane < rows)
                bulk_g2s(sbase + p.off_ring + slot * SLOT_BYTES + lane * ROW_PITCH,
                         p.w + static_cast<size_t>(row0 + lane) * p.rb + static_cast<size_t>(sl) * SLICE_SB * Q4_K_BYTES, bytes, bar_full(slot));
        }
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may start as SMs free up
        if (gave_up && lane == 0) report_status(p.err, DEV_TIMEOUT_EMPTY);
        // copies still in flight must land before the CTA gives its shared memory back
        const int pending = u < p.n_slots ? u : p.n_slots;
        for (int k = 0; k < pending; ++k) {
            const int v = u - 1 - k;
            if (!mbar_wait_bounded(bar_full(v % p.n_slots), (v / p.n_slots) & 1) && lane == 0) report_status(p.err, DEV_TIMEOUT_DRAIN);
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    // x may be produced, and y read, by the kernel before this one in the stream (the weights are not, so the producer
    // starts at once)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // (1) the quantized activation rows (written by quantize_rows_kernel, the launch before this one) into shared memory
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar_act, p.act_bytes + p.ds_bytes);
        bulk_g2s(sbase + p.off_act, p.act_img, p.act_bytes, bar_act);
        bulk_g2s(sbase + p.off_ds, p.act_img + p.act_bytes, p.ds_bytes, bar_act);
    }
    if (!mbar_wait_bounded(bar_act, 0)) { if (lane == 0) report_status(p.err, DEV_TIMEOUT_FULL); return; }

    // (2) the units. Fragment coordinates of this lane: weight rows gq and gq + 8 of the group, activation rows
    // 2 tq and 2 tq + 1 (C), activation row gq (B), k bytes 4 tq .. 4 tq + 3 and 16 + 4 tq .. (A and B).
    const int gq = lane >> 2, tq = lane & 3;
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, accm[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    for (int u = 0; u < n_units; ++u) {
        const int slot = u % p.n_slots;
        const int g = g_begin + u / n_slices, sl = u % n_slices;
        if (!mbar_wait_bounded(bar_full(slot), (u / p.n_slots) & 1)) { ok = false; break; }
        const int sbs = (nsb - sl * SLICE_SB) < SLICE_SB ? (nsb - sl * SLICE_SB) : SLICE_SB;
        const uint32_t row_a = sbase + p.off_ring + slot * SLOT_BYTES + gq * ROW_PITCH, row_b = row_a + 8 * ROW_PITCH;
        for (int s = warp; s < sbs; s += CW) {
            const int sb = sl * SLICE_SB + s;                      // super-block of the row
            const uint32_t blk_a = row_a + s * Q4_K_BYTES, blk_b = row_b + s * Q4_K_BYTES;
            // scales of sub-blocks tq and tq + 4 of both rows (Laplace src/kernels.h:82-90); the other six come by shuffle
            float dsc[2][2], dmn[2][2];                             // [row a / b][sub-block tq / tq + 4]
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint32_t blk = r ? blk_b : blk_a;
                const uint32_t hdr = lds32(blk);
                const uint32_t q0 = lds32(blk + 4), q1 = lds32(blk + 8), q2 = lds32(blk + 12);     // scale bytes 0-3, 4-7, 8-11
                const uint32_t b_lo = (q0 >> (8 * tq)) & 0xff, b_mid = (q1 >> (8 * tq)) & 0xff, b_hi = (q2 >> (8 * tq)) & 0xff;
                const float d = half_bits_to_float(hdr), dmin = half_bits_to_float(hdr >> 16);
                dsc[r][0] = d * static_cast<float>(b_lo & 63);
                dmn[r][0] = dmin * static_cast<float>(b_mid & 63);
                dsc[r][1] = d * static_cast<float>((b_hi & 0xF) | ((b_lo >> 6) << 4));
                dmn[r][1] = dmin * static_cast<float>((b_hi >> 4) | ((b_mid >> 6) << 4));
            }
            // The super-block in phases - every load, then the eight MMAs, then shuffles and the fp32 chain - so that each
            // kind of latency is paid once per super-block, not once per block.
            uint32_t wa[8], wb[8], bq[16];
            uint4 ds[8];
#pragma unroll
            for (int jb = 0; jb < 4; ++jb) {                        // 64-value chunk: low nibbles, then high nibbles
                wa[2 * jb] = lds32(blk_a + 16 + 32 * jb + 4 * tq); wa[2 * jb + 1] = lds32(blk_a + 32 + 32 * jb + 4 * tq);
                wb[2 * jb] = lds32(blk_b + 16 + 32 * jb + 4 * tq); wb[2 * jb + 1] = lds32(blk_b + 32 + 32 * jb + 4 * tq);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int bx = sb * 8 + j;                          // activation block
                const uint32_t act = sbase + p.off_act + gq * p.act_stride + bx * 32 + 4 * tq;
                bq[2 * j] = lds32(act); bq[2 * j + 1] = lds32(act + 16);
                ds[j] = lds128(sbase + p.off_ds + (static_cast<uint32_t>(bx) * MAXM + 2 * tq) * 8);      // (d, sum) of rows 2 tq, 2 tq + 1
            }
            int c[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {                           // sub-block j: chunk j / 2, low or high nibbles
                const int jb = j >> 1, hi = j & 1;
                const uint32_t a[4] = {(wa[2 * jb] >> (4 * hi)) & 0x0f0f0f0fu, (wb[2 * jb] >> (4 * hi)) & 0x0f0f0f0fu,
                                       (wa[2 * jb + 1] >> (4 * hi)) & 0x0f0f0f0fu, (wb[2 * jb + 1] >> (4 * hi)) & 0x0f0f0f0fu};
                mma_u8s8(c[j], a, bq[2 * j], bq[2 * j + 1]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // the block's weight scales live in lane (gq, j & 3), first or second value
                const int src = (lane & ~3) | (j & 3);
                const float sa = __shfl_sync(0xffffffffu, dsc[0][j >> 2], src), sb_ = __shfl_sync(0xffffffffu, dsc[1][j >> 2], src);
                const float ma = __shfl_sync(0xffffffffu, dmn[0][j >> 2], src), mb = __shfl_sync(0xffffffffu, dmn[1][j >> 2], src);
                const float d0 = __uint_as_float(ds[j].x), s0 = __uint_as_float(ds[j].y), d1 = __uint_as_float(ds[j].z), s1 = __uint_as_float(ds[j].w);
                acc[0] = fmaf(sa * d0, static_cast<float>(c[j][0]), acc[0]);
                acc[1] = fmaf(sa * d1, static_cast<float>(c[j][1]), acc[1]);
                acc[2] = fmaf(sb_ * d0, static_cast<float>(c[j][2]), acc[2]);
                acc[3] = fmaf(sb_ * d1, static_cast<float>(c[j][3]), acc[3]);
                accm[0] = fmaf(ma, s0, accm[0]);
                accm[1] = fmaf(ma, s1, accm[1]);
                accm[2] = fmaf(mb, s0, accm[2]);
                accm[3] = fmaf(mb, s1, accm[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty(slot));               // the slot may be refilled
        if (sl == n_slices - 1) {
            // the group is complete: the warps' partial results meet in shared memory (two areas, used in turn, so that
            // one barrier per group is enough) and are added in warp order
            const int gi = u / n_slices;
            float* part = reinterpret_cast<float*>(smem + p.off_part) + (gi & 1) * (CW * GROUP * MAXM);
            float* mine = part + warp * (GROUP * MAXM);
            mine[gq * MAXM + 2 * tq] = acc[0] - accm[0];
            mine[gq * MAXM + 2 * tq + 1] = acc[1] - accm[1];
            mine[(gq + 8) * MAXM + 2 * tq] = acc[2] - accm[2];
            mine[(gq + 8) * MAXM + 2 * tq + 1] = acc[3] - accm[3];
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[i] = 0.f; accm[i] = 0.f; }
            named_bar_sync(2, CW * 32);
            if (threadIdx.x < GROUP * MAXM) {
                const int row = threadIdx.x >> 3, col = threadIdx.x & 7;
                float v = part[row * MAXM + col];
#pragma unroll
                for (int w = 1; w < CW; ++w) v += part[w * (GROUP * MAXM) + row * MAXM + col];
                const int j = g * GROUP + row;
                if (col < p.M && j < p.N) p.y[static_cast<size_t>(col) * p.N + j] = v;
            }
        }
    }
    if (!ok && lane == 0) report_status(p.err, DEV_TIMEOUT_FULL);
}

}  // namespace

// Serves plain Q4_K matrices with 2..8 activation rows whose shared-memory plan fits; LAPLACE_UNSUPPORTED otherwise
// (the caller falls back to the dp4a kernel).
int launch_gemv_mma_q4k(const float* x, const uint8_t* w, float* y, int M, int K, int N, cudaStream_t st) {
    Context& c = ctx();
    if (M < 2 || M > MAXM || K <= 0 || K % 256 || K > MAX_K || N <= 0) return LAPLACE_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return LAPLACE_UNSUPPORTED;
    MmaParams p{};
    p.x = x; p.w = w; p.y = y; p.err = c.d_err; p.M = M; p.K = K; p.N = N;
    p.rb = static_cast<uint32_t>(row_bytes(LAPLACE_TYPE_Q4_K, K));
    p.act_stride = static_cast<uint32_t>(K + 16);
    uint32_t off = 128;                                     // barriers
    p.off_act = off;  off += MAXM * p.act_stride;
    off = (off + 15u) & ~15u;
    p.off_ds = off;   off += static_cast<uint32_t>(K / 32) * MAXM * 8;
    p.off_part = off; off += 2 * CW * GROUP * MAXM * 4;
    off = (off + 127u) & ~127u;
    p.off_ring = off;
    const size_t budget = c.smem_optin;
    if (off + 2u * SLOT_BYTES > budget) return LAPLACE_UNSUPPORTED;
    int slots = static_cast<int>((budget - off) / SLOT_BYTES);
    p.n_slots = slots > 4 ? 4 : slots;
    const size_t smem = off + static_cast<size_t>(p.n_slots) * SLOT_BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_mma_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(c.smem_optin));
        if (e != cudaSuccess) return cuda_check(e, "cudaFuncSetAttribute gemv_mma");
        configured = true;
    }
    static uint8_t* img_of[64] = {};                         // the array's address on every device this process has used
    if (c.device < 0 || c.device >= 64) return LAPLACE_UNSUPPORTED;
    if (!img_of[c.device]) {
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&img_of[c.device]), g_act_img);
        if (e != cudaSuccess) { img_of[c.device] = nullptr; return cuda_check(e, "cudaGetSymbolAddress g_act_img"); }
    }
    uint8_t* img = img_of[c.device];
    p.act_img = img;
    p.act_bytes = MAXM * p.act_stride;
    p.ds_bytes = static_cast<uint32_t>(K / 32) * MAXM * 8;
    {
        const int nblk = MAXM * (K / 32);
        int qgrid = (nblk + 31) / 32;
        if (qgrid > 2 * c.sm_count) qgrid = 2 * c.sm_count;
        quantize_rows_kernel<<<qgrid, 256, 0, st>>>(x, M, K, p.act_stride, img);
        c.launches++;
        const int rc = cuda_check(cudaGetLastError(), "quantize_rows launch");
        if (rc) return rc;
    }
    const int groups = (N + GROUP - 1) / GROUP;
    const int grid = groups < c.sm_count ? groups : c.sm_count;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;      // see griddepcontrol.wait in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_mma_q4k_kernel, p);
    c.launches++;
    c.last_path = 1;
    return cuda_check(e, "gemv_mma launch");
}

}  // namespace lp
