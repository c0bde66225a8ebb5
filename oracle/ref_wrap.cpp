// ref_wrap.cpp - C entry points around the reference's own (unmodified) matmul
// front-end, so tests and the CPU-baseline timer can call it through ctypes.
// TEST INFRASTRUCTURE ONLY. Linked with the reference's src/matmul.cpp and
// src/matmul_simd.cpp, which are compiled where they lie; on an x86 host the
// latter contributes only its "no SIMD back-end" stubs, so every call below
// runs the reference's scalar fp32-activation path (src/matmul.cpp:84-353).
#include <cstddef>
#include <cstdint>

#include "fp16.h"
#include "matmul.h"
#include "ops.h"
#include "tensor.h"
#include "threadpool.h"

using namespace Laplace;

static Tensor view(const uint8_t* w, uint32_t type, int K, int N, int n_experts) {
    Tensor t;
    t.name = "w";
    t.type = static_cast<GGMLType>(type);
    t.n_dims = n_experts > 1 ? 3 : 2;
    t.dims[0] = static_cast<uint64_t>(K);
    t.dims[1] = static_cast<uint64_t>(N);
    t.dims[2] = static_cast<uint64_t>(n_experts > 1 ? n_experts : 0);
    t.data = w;
    return t;
}

extern "C" {

// src/ops.cpp:34-74, 128-176 (scalar branches on an x86 host)
void ref_rmsnorm_rows(const float* x, const float* w, float* y, int rows, int cols, float eps) { ops::rmsnorm_rows(x, w, y, rows, cols, eps); }
void ref_swiglu(const float* gate, const float* up, float* out, int n) { ops::swiglu(gate, up, out, n); }
void ref_geglu(const float* gate, const float* up, float* out, int n) { ops::geglu(gate, up, out, n); }

void ref_set_threads(int t) { ThreadPool::get().set_threads(t); }
int  ref_threads() { return ThreadPool::get().threads(); }

void ref_matmul_rows(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N) {
    matmul_rows(x, view(w, type, K, N, 1), y, M, K, N);
}

void ref_fused_moe_gemm_idx(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                            int n_slots, int n_experts_total, float* y, int K, int N) {
    fused_moe_gemm_idx(x, view(w, type, K, N, n_experts_total), y, expert_idx, n_slots, K, N);
}

void ref_fused_moe_gemm_multi(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                              int n_slots, int n_experts_total, float* y, int K, int N) {
    fused_moe_gemm_multi(x, view(w, type, K, N, n_experts_total), y, expert_idx, n_slots, K, N);
}

void ref_dequantize(const uint8_t* w, uint32_t type, float* dst, int n) {
    Tensor t = view(w, type, n, 1, 1);
    dequantize(t, dst, n);
}

float    ref_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }
uint16_t ref_fp32_to_fp16(float f) { return fp32_to_fp16(f); }

size_t ref_bytes_per_block(uint32_t type) { return bytes_per_block(static_cast<GGMLType>(type)); }
int    ref_elements_per_block(uint32_t type) { return elements_per_block(static_cast<GGMLType>(type)); }

}
