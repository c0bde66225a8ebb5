// lp_moe_grouped.cuh - expert-grouped matmul for a batch of tokens. Included by lp_gemm_tc.cu
// inside namespace lp.
//
// Laplace runs a mixture-of-experts layer token by token: for each token one fused_moe_gemm_idx
// call over its top-k experts (gate/up, src/matmul.cpp:467-482, src/arch_gemma4.cpp:604) and
// one fused_moe_gemm_multi call (down, src/matmul.cpp:484-500, src/arch_gemma4.cpp:626). With a
// batch of tokens every such call streams the selected experts again. Here all
// (token, expert) pairs of the batch are grouped by expert on the device and every expert's
// weights meet all of its tokens in one pass of the tensor-core kernel:
//   for every pair p:  y[p] = W[pair_expert[p]] . quantize(x[pair_row[p]])
// which is exactly what the per-token calls compute (the result of a pair does not depend on
// which other pairs share its tile).
//
// Device-side plan (no host synchronisation, the grid is persistent):
//   1. count pairs per expert, give every pair a slot inside its expert      (moe_count_kernel)
//   2. prefix over experts of the counts rounded up to 128 rows -> first row of each expert in
//      the activation operand; tile table {m0, n0, first weight row}        (moe_plan_kernel)
//   3. destination row of every pair, and the inverse map for the epilogue   (moe_assign_kernel)
//   4. quantize the gathered rows into the operand                           (quantize_act_f16_mapped_kernel)
//   5. the GEMM kernel walks the tile table and scatters rows through out_row.
namespace {

__global__ void moe_count_kernel(const int* __restrict__ pair_expert, int P, int E, int* __restrict__ counts,
                                 int* __restrict__ slot, int* err) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int e = pair_expert[p];
    if (e < 0 || e >= E) {
        slot[p] = -1;                      // the pair is skipped: negative = "not mine" (experts placed on
        if (e >= E) report_status(err, DEV_BAD_INDEX);       // another GPU), too large = the host reports a bad argument
        return;
    }
    slot[p] = atomicAdd(counts + e, 1);
}

// One block. base[e] = first operand row of expert e; tiles ordered by expert, then by 128-row
// group of its tokens, then by 128-column block, so that CTAs running at the same time share
// activation rows and neighbouring weight rows in L2. A second table (another N over the same row
// groups) serves the second matmul of a fused FFN; tiles_n2 = 0 leaves it out.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ base,
                                int N1, int tiles_n1, int4* __restrict__ tab1, int* __restrict__ n_tiles1,
                                int N2, int tiles_n2, int4* __restrict__ tab2, int* __restrict__ n_tiles2) {
    if (threadIdx.x == 0) {
        int rows = 0, groups_total = 0;
        for (int e = 0; e < E; ++e) {
            base[e] = rows;
            base[E + 1 + e] = groups_total;                // row groups before expert e
            const int groups = (counts[e] + BM - 1) / BM;
            rows += groups * BM;
            groups_total += groups;
        }
        base[E] = rows;
        *n_tiles1 = groups_total * tiles_n1;
        if (tiles_n2) *n_tiles2 = groups_total * tiles_n2;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int groups = (counts[e] + BM - 1) / BM;
        const int g0 = base[E + 1 + e];
        for (int g = 0; g < groups; ++g) {
            for (int nt = 0; nt < tiles_n1; ++nt)
                tab1[(g0 + g) * tiles_n1 + nt] = make_int4(base[e] + g * BM, nt * BN, e * N1, 0);
            for (int nt = 0; nt < tiles_n2; ++nt)
                tab2[(g0 + g) * tiles_n2 + nt] = make_int4(base[e] + g * BM, nt * BN, e * N2, 0);
        }
    }
}

__global__ void moe_assign_kernel(const int* __restrict__ pair_expert, const int* __restrict__ slot, int P,
                                  const int* __restrict__ base, int* __restrict__ dst_row, int* __restrict__ out_row) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= P) return;
    const int s = slot[p];
    if (s < 0) { dst_row[p] = -1; return; }
    const int r = base[pair_expert[p]] + s;
    dst_row[p] = r;
    out_row[r] = p;
}

// quantize_act_f16_kernel with a row gather on the way in and a row scatter on the way out:
// pair m reads x row src_rows[m] (m / src_div when src_rows is null: the top-k pairs of a token are
// consecutive) and writes operand row dst_rows[m].
__global__ void __launch_bounds__(256) quantize_act_f16_mapped_kernel(const float* __restrict__ x, int P, int K,
                                                                      const int* __restrict__ src_rows, int src_div,
                                                                      const int* __restrict__ dst_rows,
                                                                      __half* __restrict__ aq, float* __restrict__ dx,
                                                                      __nv_bfloat16* __restrict__ ag, int ag_stride) {
    const int t8 = threadIdx.x & 7;
    const int bpr = K / 32;
    const long long n_blocks = static_cast<long long>(P) * bpr;
    const long long groups = static_cast<long long>(gridDim.x) * (blockDim.x >> 3);
    const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x >> 3) + (threadIdx.x >> 3);
    const long long iters = (n_blocks + groups - 1) / groups;
    for (long long itn = 0; itn < iters; ++itn) {
        const long long b = first + itn * groups;
        bool live = b < n_blocks;
        const int m = live ? static_cast<int>(b / bpr) : 0;
        const int kb = live ? static_cast<int>(b - static_cast<long long>(m) * bpr) : 0;
        const int dr = live ? dst_rows[m] : -1;
        live = live && dr >= 0;
        const long long sr = live ? (src_rows ? src_rows[m] : m / src_div) : 0;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = __ldg(reinterpret_cast<const float4*>(x + (sr * bpr + kb) * 32) + t8);
        uint32_t packed; int hs;
        const float d = quantize_block_8lanes(v, packed, hs);
        const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
        if (!live) continue;
        const int q0 = static_cast<int8_t>(packed & 0xff), q1 = static_cast<int8_t>((packed >> 8) & 0xff);
        const int q2 = static_cast<int8_t>((packed >> 16) & 0xff), q3 = static_cast<int8_t>(packed >> 24);
        const __half2 lo = __halves2half2(__int2half_rn(q0), __int2half_rn(q2));
        const __half2 hi = __halves2half2(__int2half_rn(q1), __int2half_rn(q3));
        uint2 out;
        out.x = *reinterpret_cast<const uint32_t*>(&lo);
        out.y = *reinterpret_cast<const uint32_t*>(&hi);
        const long long ob = static_cast<long long>(dr) * bpr + kb;
        reinterpret_cast<uint2*>(aq + ob * 32)[t8] = out;
        if (t8 == 0) {
            const short slo = static_cast<short>(hs), shi = static_cast<short>(hs_hi);
            dx[ob] = d;
            const float sum = d * static_cast<float>(static_cast<int>(slo) + static_cast<int>(shi));
            const __nv_bfloat16 p0 = __float2bfloat16_rn(sum);
            const float r1 = sum - __bfloat162float(p0);
            const __nv_bfloat16 p1 = __float2bfloat16_rn(r1);
            const __nv_bfloat16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
            __nv_bfloat16* dst = ag + static_cast<long long>(dr) * ag_stride + (kb >> 3) * 32 + 3 * (kb & 7);
            dst[0] = p0; dst[1] = p1; dst[2] = p2;
        }
    }
}

Scratch g_moe_scratch;

inline size_t align256(size_t n) { return (n + 255) & ~size_t(255); }

}  // namespace

void release_moe_grouped_scratch() { g_moe_scratch.release(); }

bool moe_grouped_supports(uint32_t type, int K, int N) {
    return gemm_tc_supports(type, 9, K, N);
}

int launch_moe_grouped(const float* x, const uint8_t* w, uint32_t type, const int* pair_expert, const int* pair_row,
                       int P, int E, float* y, int K, int N, cudaStream_t st) {
    if (!moe_grouped_supports(type, K, N)) return LAPLACE_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
        return fail(LAPLACE_ERR_ARG, "moe_grouped: x and w must be 16-byte aligned on the device");
    if ((static_cast<size_t>(N) * row_bytes(type, K)) % 16)
        return fail(LAPLACE_ERR_ARG, "moe_grouped: expert stride is not a 16-byte multiple");
    Context& c = ctx();
    const int tiles_n = (N + BN - 1) / BN;
    const int n_sb_pairs = (K / 256 + 1) / 2;
    const size_t bpr = static_cast<size_t>(K / 32);
    // every expert's rows are padded to a multiple of 128: at most min(E, P) experts are populated
    const size_t groups_max = static_cast<size_t>(P) / BM + static_cast<size_t>(E < P ? E : P);
    const size_t rows_max = groups_max * BM;
    const size_t tiles_max = groups_max * tiles_n;
    const size_t aq_bytes = align256(rows_max * K * sizeof(__half));
    const size_t dx_bytes = align256(rows_max * bpr * sizeof(float));
    const size_t ag_bytes = align256(rows_max * n_sb_pairs * 64 * sizeof(__nv_bfloat16));
    const size_t cnt_bytes = align256(sizeof(int) * (2 * static_cast<size_t>(E) + 2));      // counts | n_tiles
    const size_t base_bytes = align256(sizeof(int) * (2 * static_cast<size_t>(E) + 2));
    const size_t slot_bytes = align256(sizeof(int) * static_cast<size_t>(P));
    const size_t out_bytes = align256(sizeof(int) * rows_max);
    const size_t tab_bytes = align256(sizeof(int4) * tiles_max);
    const size_t total = aq_bytes + dx_bytes + ag_bytes + cnt_bytes + base_bytes + 2 * slot_bytes + out_bytes + tab_bytes;
    int rc;
    if ((rc = g_moe_scratch.ensure(total, st))) return rc;
    uint8_t* s = static_cast<uint8_t*>(g_moe_scratch.p);
    __half* aq = reinterpret_cast<__half*>(s);                     s += aq_bytes;
    float* dx = reinterpret_cast<float*>(s);                       s += dx_bytes;
    __nv_bfloat16* ag = reinterpret_cast<__nv_bfloat16*>(s);       s += ag_bytes;
    int* counts = reinterpret_cast<int*>(s);                       s += cnt_bytes;
    int* base = reinterpret_cast<int*>(s);                         s += base_bytes;
    int* slot = reinterpret_cast<int*>(s);                         s += slot_bytes;
    int* dst_row = reinterpret_cast<int*>(s);                      s += slot_bytes;
    int* out_row = reinterpret_cast<int*>(s);                      s += out_bytes;
    int4* tile_tab = reinterpret_cast<int4*>(s);
    int* n_tiles = counts + E;                                      // shares the zeroed block with the counters

    if ((rc = cuda_check(cudaMemsetAsync(counts, 0, cnt_bytes, st), "cudaMemsetAsync")) ||
        (rc = cuda_check(cudaMemsetAsync(out_row, 0xff, out_bytes, st), "cudaMemsetAsync")) ||
        (rc = cuda_check(cudaMemsetAsync(ag, 0, ag_bytes, st), "cudaMemsetAsync")))
        return rc;
    const int tb = 256, gb = (P + tb - 1) / tb;
    moe_count_kernel<<<gb, tb, 0, st>>>(pair_expert, P, E, counts, slot, c.d_err);
    moe_plan_kernel<<<1, 256, 0, st>>>(counts, E, base, N, tiles_n, tile_tab, n_tiles, 0, 0, nullptr, nullptr);
    moe_assign_kernel<<<gb, tb, 0, st>>>(pair_expert, slot, P, base, dst_row, out_row);
    {
        const long long n_blocks = static_cast<long long>(P) * static_cast<long long>(bpr);
        long long want = (n_blocks + 31) / 32;
        const long long cap = static_cast<long long>(c.sm_count) * 8;
        const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
        quantize_act_f16_mapped_kernel<<<grid, 256, 0, st>>>(x, P, K, pair_row, 1, dst_row, aq, dx, ag, n_sb_pairs * 64);
    }
    c.launches += 4;
    if ((rc = cuda_check(cudaGetLastError(), "moe_grouped set-up launches"))) return rc;

    TcLaunch L{};
    L.w = w; L.type = type; L.y = y; L.M = P; L.K = K; L.N = N;
    L.rows_pad = rows_max; L.w_rows = static_cast<long long>(E) * N;
    L.aq = aq; L.dx = dx; L.ag = ag;
    L.tile_tab = tile_tab; L.n_tiles_dev = n_tiles; L.out_row = out_row;
    L.tiles_m = 1; L.tiles_n = tiles_n;
    L.grid = static_cast<int>(tiles_max < static_cast<size_t>(c.sm_count) ? tiles_max : static_cast<size_t>(c.sm_count));
    if (L.grid < 1) L.grid = 1;
    rc = run_tc_kernel(L, st);
    if (rc == LAPLACE_OK) c.last_path = 3;
    return rc;
}

// ---- fused expert FFN ---------------------------------------------------------------------
// The per-token sequence of Laplace's MoE layer (src/arch_gemma4.cpp:600-638): gate/up matmul
// over the token's experts, gated activation (ops::swiglu / ops::geglu, src/ops.cpp:128-176),
// down matmul with one input per expert, out = sum_k top_w[k] * expert_out[k] - for a batch of
// tokens with one plan shared by both matmuls. Intermediate results stay in operand-row order
// (rows grouped by expert), so nothing is scattered or gathered between the two matmuls.
namespace {

__device__ __forceinline__ float act_swiglu(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
__device__ __forceinline__ float act_geglu(float g, float u) {
    const float g3 = (g * g) * g;
    const float gelu = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g3)));
    return gelu * u;
}

// Operand rows of the down matmul from the gate/up result: row r of gu holds [gate(I) | up(I)];
// h = act(gate) * up is quantized per 32 values like any activation row. The kernel walks the pairs
// (dst_row[pair] = the pair's operand row, -1 = skipped). h_out (optional) receives h in pair order.
__global__ void __launch_bounds__(256) moe_act_quant_kernel(const float* __restrict__ gu, int I, int activation,
                                                            int n_pairs, const int* __restrict__ dst_row,
                                                            __half* __restrict__ aq, float* __restrict__ dx,
                                                            __nv_bfloat16* __restrict__ ag, int ag_stride,
                                                            float* __restrict__ h_out) {
    const int t8 = threadIdx.x & 7;
    const int bpr = I / 32;
    const long long n_blocks = static_cast<long long>(n_pairs) * bpr;        // walk the pairs, not the padded operand rows
    const long long groups = static_cast<long long>(gridDim.x) * (blockDim.x >> 3);
    const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x >> 3) + (threadIdx.x >> 3);
    const long long iters = (n_blocks + groups - 1) / groups;
    for (long long itn = 0; itn < iters; ++itn) {
        const long long b = first + itn * groups;
        bool live = b < n_blocks;
        const int pair = live ? static_cast<int>(b / bpr) : 0;
        const int kb = live ? static_cast<int>(b - static_cast<long long>(pair) * bpr) : 0;
        const int r = live ? __ldg(dst_row + pair) : -1;                      // operand row of the pair, -1 = skipped pair
        live = live && r >= 0;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            const float* row = gu + static_cast<long long>(r) * (2 * I) + kb * 32;
            const float4 g = __ldg(reinterpret_cast<const float4*>(row) + t8);
            const float4 u = __ldg(reinterpret_cast<const float4*>(row + I) + t8);
            if (activation == 1) v = make_float4(act_geglu(g.x, u.x), act_geglu(g.y, u.y), act_geglu(g.z, u.z), act_geglu(g.w, u.w));
            else v = make_float4(act_swiglu(g.x, u.x), act_swiglu(g.y, u.y), act_swiglu(g.z, u.z), act_swiglu(g.w, u.w));
            if (h_out) reinterpret_cast<float4*>(h_out + static_cast<long long>(pair) * I + kb * 32)[t8] = v;
        }
        uint32_t packed; int hs;
        const float d = quantize_block_8lanes(v, packed, hs);
        const int hs_hi = __shfl_down_sync(0xffffffffu, hs, 4);
        if (!live) continue;
        const int q0 = static_cast<int8_t>(packed & 0xff), q1 = static_cast<int8_t>((packed >> 8) & 0xff);
        const int q2 = static_cast<int8_t>((packed >> 16) & 0xff), q3 = static_cast<int8_t>(packed >> 24);
        const __half2 lo = __halves2half2(__int2half_rn(q0), __int2half_rn(q2));
        const __half2 hi = __halves2half2(__int2half_rn(q1), __int2half_rn(q3));
        uint2 out;
        out.x = *reinterpret_cast<const uint32_t*>(&lo);
        out.y = *reinterpret_cast<const uint32_t*>(&hi);
        const long long ob = static_cast<long long>(r) * bpr + kb;
        reinterpret_cast<uint2*>(aq + ob * 32)[t8] = out;
        if (t8 == 0) {
            const short slo = static_cast<short>(hs), shi = static_cast<short>(hs_hi);
            dx[ob] = d;
            const float sum = d * static_cast<float>(static_cast<int>(slo) + static_cast<int>(shi));
            const __nv_bfloat16 p0 = __float2bfloat16_rn(sum);
            const float r1 = sum - __bfloat162float(p0);
            const __nv_bfloat16 p1 = __float2bfloat16_rn(r1);
            const __nv_bfloat16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
            __nv_bfloat16* dst = ag + static_cast<long long>(r) * ag_stride + (kb >> 3) * 32 + 3 * (kb & 7);
            dst[0] = p0; dst[1] = p1; dst[2] = p2;
        }
    }
}

// out[t][:] = sum over the token's live pairs, in slot order, of top_w[t][j] * dn[row of pair][:]
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ dn, const int* __restrict__ dst_row,
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

Scratch g_ffn_scratch;

}  // namespace

void release_moe_ffn_scratch() { g_ffn_scratch.release(); }

int launch_moe_ffn(const float* x, const uint8_t* w_gate_up, const uint8_t* w_down, uint32_t type_gu, uint32_t type_dn,
                   const int* top_idx, const float* top_w, const float* down_scale, int T, int top_k, int E, int H, int I,
                   int activation, float* out, float* h_out, cudaStream_t st) {
    if (!moe_grouped_supports(type_gu, H, 2 * I) || !moe_grouped_supports(type_dn, I, H)) return LAPLACE_UNSUPPORTED;
    if (I % 32 || H % 4) return fail(LAPLACE_ERR_ARG, "moe_ffn: H=%d I=%d", H, I);
    if ((reinterpret_cast<uintptr_t>(w_gate_up) & 15) || (reinterpret_cast<uintptr_t>(w_down) & 15) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail(LAPLACE_ERR_ARG, "moe_ffn: x, out and the weights must be 16-byte aligned on the device");
    if ((static_cast<size_t>(2 * I) * row_bytes(type_gu, H)) % 16 || (static_cast<size_t>(H) * row_bytes(type_dn, I)) % 16)
        return fail(LAPLACE_ERR_ARG, "moe_ffn: expert stride is not a 16-byte multiple");
    Context& c = ctx();
    const int P = T * top_k;
    const int tiles_n1 = (2 * I + BN - 1) / BN, tiles_n2 = (H + BN - 1) / BN;
    const int sbp1 = (H / 256 + 1) / 2, sbp2 = (I / 256 + 1) / 2;
    const size_t bpr1 = static_cast<size_t>(H / 32), bpr2 = static_cast<size_t>(I / 32);
    const size_t groups_max = static_cast<size_t>(P) / BM + static_cast<size_t>(E < P ? E : P);
    const size_t rows_max = groups_max * BM;
    // zeroed block: bf16 pieces of both operands, counters; then everything else
    const size_t ag1_bytes = align256(rows_max * sbp1 * 64 * sizeof(__nv_bfloat16));
    const size_t ag2_bytes = align256(rows_max * sbp2 * 64 * sizeof(__nv_bfloat16));
    const size_t cnt_bytes = align256(sizeof(int) * (static_cast<size_t>(E) + 4));
    const size_t zero_bytes = ag1_bytes + ag2_bytes + cnt_bytes;
    const size_t out_bytes = align256(sizeof(int) * rows_max);
    const size_t aq1_bytes = align256(rows_max * H * sizeof(__half)), aq2_bytes = align256(rows_max * I * sizeof(__half));
    const size_t dx1_bytes = align256(rows_max * bpr1 * sizeof(float)), dx2_bytes = align256(rows_max * bpr2 * sizeof(float));
    const size_t gu_bytes = align256(rows_max * 2 * I * sizeof(float)), dn_bytes = align256(rows_max * H * sizeof(float));
    const size_t base_bytes = align256(sizeof(int) * (2 * static_cast<size_t>(E) + 2));
    const size_t slot_bytes = align256(sizeof(int) * static_cast<size_t>(P));
    const size_t tab1_bytes = align256(sizeof(int4) * groups_max * tiles_n1), tab2_bytes = align256(sizeof(int4) * groups_max * tiles_n2);
    const size_t total = zero_bytes + out_bytes + aq1_bytes + aq2_bytes + dx1_bytes + dx2_bytes + gu_bytes + dn_bytes +
                         base_bytes + 2 * slot_bytes + tab1_bytes + tab2_bytes;
    int rc;
    if ((rc = g_ffn_scratch.ensure(total, st))) return rc;
    uint8_t* s = static_cast<uint8_t*>(g_ffn_scratch.p);
    uint8_t* zero_block = s;
    __nv_bfloat16* ag1 = reinterpret_cast<__nv_bfloat16*>(s);      s += ag1_bytes;
    __nv_bfloat16* ag2 = reinterpret_cast<__nv_bfloat16*>(s);      s += ag2_bytes;
    int* counts = reinterpret_cast<int*>(s);                       s += cnt_bytes;
    int* out_row = reinterpret_cast<int*>(s);                      s += out_bytes;
    __half* aq1 = reinterpret_cast<__half*>(s);                    s += aq1_bytes;
    __half* aq2 = reinterpret_cast<__half*>(s);                    s += aq2_bytes;
    float* dx1 = reinterpret_cast<float*>(s);                      s += dx1_bytes;
    float* dx2 = reinterpret_cast<float*>(s);                      s += dx2_bytes;
    float* gu = reinterpret_cast<float*>(s);                       s += gu_bytes;
    float* dn = reinterpret_cast<float*>(s);                       s += dn_bytes;
    int* base = reinterpret_cast<int*>(s);                         s += base_bytes;
    int* slot = reinterpret_cast<int*>(s);                         s += slot_bytes;
    int* dst_row = reinterpret_cast<int*>(s);                      s += slot_bytes;
    int4* tab1 = reinterpret_cast<int4*>(s);                       s += tab1_bytes;
    int4* tab2 = reinterpret_cast<int4*>(s);
    int* n_tiles1 = counts + E;
    int* n_tiles2 = counts + E + 1;

    if ((rc = cuda_check(cudaMemsetAsync(zero_block, 0, zero_bytes, st), "cudaMemsetAsync")) ||
        (rc = cuda_check(cudaMemsetAsync(out_row, 0xff, out_bytes, st), "cudaMemsetAsync")))
        return rc;
    const int tb = 256, gb = (P + tb - 1) / tb;
    const long long cap = static_cast<long long>(c.sm_count) * 8;
    auto grid_for = [&](long long n_blocks) {
        long long want = (n_blocks + 31) / 32;
        return static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
    };
    moe_count_kernel<<<gb, tb, 0, st>>>(top_idx, P, E, counts, slot, c.d_err);
    moe_plan_kernel<<<1, 256, 0, st>>>(counts, E, base, 2 * I, tiles_n1, tab1, n_tiles1, H, tiles_n2, tab2, n_tiles2);
    moe_assign_kernel<<<gb, tb, 0, st>>>(top_idx, slot, P, base, dst_row, out_row);
    quantize_act_f16_mapped_kernel<<<grid_for(static_cast<long long>(P) * bpr1), 256, 0, st>>>(
        x, P, H, nullptr, top_k, dst_row, aq1, dx1, ag1, sbp1 * 64);
    c.launches += 4;
    if ((rc = cuda_check(cudaGetLastError(), "moe_ffn set-up launches"))) return rc;

    const int grid_max = static_cast<int>(groups_max * tiles_n1 < static_cast<size_t>(c.sm_count) ? groups_max * tiles_n1
                                                                                                    : static_cast<size_t>(c.sm_count));
    TcLaunch L{};
    L.w = w_gate_up; L.type = type_gu; L.y = gu; L.M = P; L.K = H; L.N = 2 * I;
    L.rows_pad = rows_max; L.w_rows = static_cast<long long>(E) * 2 * I;
    L.aq = aq1; L.dx = dx1; L.ag = ag1;
    L.tile_tab = tab1; L.n_tiles_dev = n_tiles1; L.out_row = out_row; L.out_identity = 1;
    L.tiles_m = 1; L.tiles_n = tiles_n1; L.grid = grid_max < 1 ? 1 : grid_max;
    if ((rc = run_tc_kernel(L, st))) return rc;

    moe_act_quant_kernel<<<grid_for(static_cast<long long>(P) * bpr2), 256, 0, st>>>(
        gu, I, activation, P, dst_row, aq2, dx2, ag2, sbp2 * 64, h_out);
    c.launches++;
    if ((rc = cuda_check(cudaGetLastError(), "moe_act_quant launch"))) return rc;

    TcLaunch L2{};
    L2.w = w_down; L2.type = type_dn; L2.y = dn; L2.M = P; L2.K = I; L2.N = H;
    L2.rows_pad = rows_max; L2.w_rows = static_cast<long long>(E) * H;
    L2.aq = aq2; L2.dx = dx2; L2.ag = ag2;
    L2.tile_tab = tab2; L2.n_tiles_dev = n_tiles2; L2.out_row = out_row; L2.out_identity = 1;
    L2.tiles_m = 1; L2.tiles_n = tiles_n2;
    const size_t g2 = groups_max * tiles_n2;
    L2.grid = static_cast<int>(g2 < static_cast<size_t>(c.sm_count) ? (g2 < 1 ? 1 : g2) : static_cast<size_t>(c.sm_count));
    if ((rc = run_tc_kernel(L2, st))) return rc;

    {
        const long long total4 = static_cast<long long>(T) * (H / 4);
        long long blocks = (total4 + 255) / 256;
        if (blocks > cap) blocks = cap;
        moe_combine_kernel<<<static_cast<int>(blocks < 1 ? 1 : blocks), 256, 0, st>>>(dn, dst_row, top_w, top_idx, down_scale, T, top_k, H, out);
        c.launches++;
    }
    c.last_path = 4;
    return cuda_check(cudaGetLastError(), "moe_combine launch");
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
