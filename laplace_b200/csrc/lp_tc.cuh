// lp_tc.cuh - tcgen05 / TMA / tensor-map helpers shared by the tensor-core kernels.
#pragma once

#include <cuda.h>

#include "lp_common.cuh"

namespace lp {
namespace tc {

#ifdef __CUDACC__

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], kind::f16 (fp16 or bf16 operands, fp32 accumulate); acc = 0 overwrites D.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (lane = TMEM lane of the warp's quadrant).
__device__ __forceinline__ void ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 16 lanes x 16 consecutive 32-bit columns in the 16x256b shape -> 8 registers per thread: register 4 g + 2 q + e of
// lane l holds TMEM lane (base + 8 q + l / 4), column 8 g + 2 (l % 4) + e (the layout of an m16n8 accumulator
// fragment, once per 8 columns).
__device__ __forceinline__ void ld16x256_x2(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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
// kind::f16 instruction descriptor: D fp32, A and B fp16, both K-major, M = 128 rows of A, n rows of B.
__device__ __forceinline__ uint32_t idesc_f16_m128(int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

// mbarrier wait that also gives up when another role of the CTA has raised the abort flag. SPIN: poll without
// a suspend hint (the MMA-issuing thread, whose wake-up must follow the phase completion at once).
template <bool SPIN>
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    for (uint32_t it = 0; it < (SPIN ? (1u << 26) : (1u << 22)); ++it) {
        if (SPIN ? mbar_try_wait_nohint(bar, parity) : mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    report_status(err, code);
    return false;
}

#endif  // __CUDACC__

// cuTensorMapEncodeTiled, looked up at run time so that the library does not link libcuda.
using encode_tiled_fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline encode_tiled_fn encode_tiled() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess && p) fn = reinterpret_cast<encode_tiled_fn>(p);
    }
    return fn;
}
// A 2-D row-major tensor [rows][inner] of `esize`-byte elements with row pitch `pitch` bytes, copied in boxes of
// box_rows x box_inner elements. Returns false (message recorded) when the driver refuses the map.
inline bool make_map_2d(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t rows,
                        uint64_t pitch, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw, const char* what) {
    encode_tiled_fn enc = encode_tiled();
    if (!enc) { fail(LAPLACE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver"); return false; }
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fail(LAPLACE_ERR_CUDA, "cuTensorMapEncodeTiled (%s) failed (%d)", what, static_cast<int>(r)); return false; }
    return true;
}

}  // namespace tc
}  // namespace lp
