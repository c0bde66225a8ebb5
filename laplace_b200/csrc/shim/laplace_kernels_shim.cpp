// laplace_kernels_shim.cpp - the reference-side binding: defines the three
// getters that Laplace's matmul front-end asks its SIMD back-end for
// (src/kernels.h:117-119) on top of the C ABI of include/laplace_cuda.h.
//
// Built INSTEAD of src/matmul_simd.cpp (and with -I<Laplace>/src); model.cpp,
// arch_*.cpp, laplace_moe.cpp and matmul.cpp compile and link unchanged. A
// return value of `false` keeps the reference's contract (kernels.h:94-96):
// "this back-end does not handle the call, fall back to the scalar path" -
// that happens only for weight types the library does not take (it takes Q4_0 / Q5_0 / Q8_0 / Q4_K / Q6_K on the int8 path
// and F32 / F16 / BF16 / Q2_K / Q3_K / Q5_K with fp32 activations, as the scalar path computes them). An
// error from the CUDA library (a failed CUDA call, a device-side timeout, a bad
// argument) is NOT turned into a fall-back: the scalar path computes with fp32
// activations, i.e. different numbers, so the process prints the error and aborts.
//
// LAPLACE_CUDA_DEVICE selects the GPU (default 0). LAPLACE_NOSIMD=1 keeps its
// meaning: the front-end never asks for these getters (src/matmul.cpp:48-55).
#include <cstdio>
#include <cstdlib>

#include "kernels.h"          // Laplace src/kernels.h
#include "laplace_cuda.h"

namespace {

bool ensure_init() {
    static const bool ok = [] {
        const char* e = std::getenv("LAPLACE_CUDA_DEVICE");
        const int rc = laplace_cuda_init(e ? std::atoi(e) : 0);
        if (rc != LAPLACE_OK) std::fprintf(stderr, "laplace_cuda: init failed (%d): %s\n", rc, laplace_cuda_last_error());
        return rc == LAPLACE_OK;
    }();
    return ok;
}

// LAPLACE_CUDA_VERBOSE=1: report at exit how many calls ran on the GPU.
struct CallCounter {
    long n = 0;
    ~CallCounter() {
        if (std::getenv("LAPLACE_CUDA_VERBOSE")) std::fprintf(stderr, "laplace_cuda: %ld matmul calls ran on the GPU\n", n);
    }
} g_calls;

bool handled(int rc, const char* what) {
    if (rc == LAPLACE_OK) { g_calls.n++; return true; }
    if (rc != LAPLACE_UNSUPPORTED) {
        std::fprintf(stderr, "laplace_cuda: %s failed (%d): %s\n", what, rc, laplace_cuda_last_error());
        std::abort();
    }
    return false;
}

bool cuda_gemm(const float* x, const uint8_t* w, Laplace::GGMLType type, float* y, int M, int K, int N) {
    if (!ensure_init()) return false;
    return handled(laplace_cuda_gemm(x, w, static_cast<uint32_t>(type), y, M, K, N), "gemm");
}

bool cuda_moe_gemv(const float* x, const uint8_t* w, Laplace::GGMLType type, const int* expert_idx, int n_experts,
                   float* y, int K, int N) {
    if (!ensure_init()) return false;
    return handled(laplace_cuda_moe_gemv(x, w, static_cast<uint32_t>(type), expert_idx, n_experts, y, K, N), "moe_gemv");
}

bool cuda_moe_gemv_multi(const float* x, const uint8_t* w, Laplace::GGMLType type, const int* expert_idx,
                         int n_experts, float* y, int K, int N) {
    if (!ensure_init()) return false;
    return handled(laplace_cuda_moe_gemv_multi(x, w, static_cast<uint32_t>(type), expert_idx, n_experts, y, K, N),
                   "moe_gemv_multi");
}

}  // namespace

namespace Laplace {
namespace kernels {

gemm_fn get_simd_gemm() { return ensure_init() ? cuda_gemm : nullptr; }
moe_gemv_fn get_simd_moe_gemv() { return ensure_init() ? cuda_moe_gemv : nullptr; }
moe_gemv_multi_fn get_simd_moe_gemv_multi() { return ensure_init() ? cuda_moe_gemv_multi : nullptr; }

}  // namespace kernels

// Hook for matmul_register_weights (src/matmul.h:26): that function gains one line calling this
// one, so that the mmap'd GGUF region is uploaded to HBM once, at model load.
void cuda_register_weights(const void* base, size_t size) {
    if (!ensure_init()) return;
    const int rc = laplace_cuda_register_weights(base, size);
    if (rc != LAPLACE_OK) std::fprintf(stderr, "laplace_cuda: register_weights failed (%d): %s\n", rc, laplace_cuda_last_error());
}

}  // namespace Laplace
