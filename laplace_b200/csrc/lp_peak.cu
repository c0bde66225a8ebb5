// lp_peak.cu - measures the dense tensor-core rate of this GPU with a bare tcgen05.mma loop, so that the
// benchmark can state the prefill GEMM's throughput against a measured int8 (and fp16) peak rather than a
// data-sheet figure. No reference counterpart. Operands are whatever shared memory and TMEM hold: the rate
// does not depend on the values.
#include "lp_tc.cuh"

namespace lp {
namespace {

using namespace tc;

__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc) : "memory");
}

// Two threads of different warps issue M = 128, N = 128 instructions into two accumulators (one thread alone
// issues an instruction only every ~115 cycles, less than the tensor core takes). int8: both operands in shared
// memory, K = 32 per instruction; fp16: the A operand in tensor memory, K = 16.
template <bool I8>
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int reps, int* err) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    constexpr uint32_t OFF_A = 0, OFF_B = 16384, OFF_BAR = 32768, OFF_PTR = OFF_BAR + 16;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 32768 / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    if (threadIdx.x == 0) { mbar_init(sbase + OFF_BAR, 1); mbar_init(sbase + OFF_BAR + 8, 1); fence_barrier_init(); }
    fence_proxy_async();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(sbase + OFF_PTR), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + OFF_PTR);
    if ((threadIdx.x & 31) == 0 && warp < 2) {
        const uint64_t ad = smem_desc_sw128(sbase + OFF_A), bd = smem_desc_sw128(sbase + OFF_B);
        // kind::i8: D s32, A and B signed 8-bit; kind::f16: D f32, A and B fp16; M = 128, N = 128, K-major
        const uint32_t idesc = I8 ? ((2u << 4) | (1u << 7) | (1u << 10) | (16u << 17) | (8u << 24)) : idesc_f16_m128(128);
        const uint32_t d = tmem + warp * 128;
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                if (I8) mma_i8(d, ad + ks * 2, bd + ks * 2, idesc);
                else mma_f16_ts(d, tmem + 256 + ks * 8, bd + ks * 2, idesc);
            }
        }
        commit(sbase + OFF_BAR + 8 * warp);
        if (!mbar_wait_bounded(sbase + OFF_BAR + 8 * warp, 0)) report_status(err, DEV_TIMEOUT_MMA);
    }
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512u) : "memory");
    }
}

}  // namespace

// Dense tensor-core rate in Tera-operations per second (2 per multiply-add), all SMs; kind 0 = fp16, 1 = int8.
int measure_tensor_peak(int kind, double* tops) {
    Context& c = ctx();
    const int reps = 4000, smem = 34 * 1024;
    cudaEvent_t e0, e1;
    int rc;
    if ((rc = cuda_check(cudaEventCreate(&e0), "cudaEventCreate")) || (rc = cuda_check(cudaEventCreate(&e1), "cudaEventCreate"))) return rc;
    float best = 0.f;
    for (int pass = 0; pass < 4; ++pass) {
        cudaEventRecord(e0, c.stream);
        if (kind == 1) tensor_peak_kernel<true><<<c.sm_count, 128, smem, c.stream>>>(reps, c.d_err);
        else tensor_peak_kernel<false><<<c.sm_count, 128, smem, c.stream>>>(reps, c.d_err);
        cudaEventRecord(e1, c.stream);
        if ((rc = cuda_check(cudaEventSynchronize(e1), "tensor peak kernel"))) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (pass > 0 && (best == 0.f || ms < best)) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    c.launches += 4;
    if (rc) return rc;
    const double macs = 128.0 * 128.0 * (kind == 1 ? 32.0 : 16.0) * 4.0 * reps * 2.0 * c.sm_count;      // two issuing threads per SM
    *tops = 2.0 * macs / (best * 1e-3) / 1e12;
    return LAPLACE_OK;
}

}  // namespace lp

extern "C" int laplace_cuda_debug_tensor_peak(int kind, double* tops) {
    using namespace lp;
    if (!ctx().ready) return fail(LAPLACE_ERR_STATE, "laplace_cuda_init has not been called (or found no GPU)");
    if (!tops || (kind != 0 && kind != 1)) return fail(LAPLACE_ERR_ARG, "tensor_peak: kind 0 (fp16) or 1 (int8)");
    return measure_tensor_peak(kind, tops);
}
