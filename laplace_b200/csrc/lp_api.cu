// lp_api.cu - the C ABI (include/laplace_cuda.h): process state, the weight
// registry, host-pointer entry points that mirror Laplace's back-end function
// pointers (src/kernels.h:92-119), and their device-pointer twins.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <chrono>
#include <cstring>
#include <mutex>
#include <vector>

#include "lp_common.cuh"

namespace lp {

namespace {

std::mutex g_mu;
char g_err[512] = "";

// A registered host region and its HBM copy (Laplace's Metal path keeps the
// same kind of table, src/metal.mm:552-621).
struct Region {
    const uint8_t* host;
    size_t         size;
    uint8_t*       dev;
};
std::vector<Region> g_regions;

// Growable device / pinned-host staging for the host-pointer entry points.
struct Buf {
    void*  p = nullptr;
    size_t cap = 0;
    bool   pinned = false;
    int ensure(size_t n) {
        if (n <= cap) return LAPLACE_OK;
        release();
        size_t want = n + n / 4 + 256;
        cudaError_t e = pinned ? cudaMallocHost(&p, want) : cudaMalloc(&p, want);
        if (e != cudaSuccess) { p = nullptr; return cuda_check(e, pinned ? "cudaMallocHost" : "cudaMalloc"); }
        cap = want;
        return LAPLACE_OK;
    }
    void release() {
        if (p) { if (pinned) cudaFreeHost(p); else cudaFree(p); }
        p = nullptr; cap = 0;
    }
};
Buf g_dx, g_dy, g_dw, g_didx, g_dq;          // device
Buf g_hx{nullptr, 0, true}, g_hy{nullptr, 0, true};   // pinned host

Context g_ctx;

// LAPLACE_PROF=1, the reference's switch (src/matmul.cpp:355-379: wall time inside the matmuls, reported at process
// exit): per host-pointer entry point the number of calls, the wall time of the whole call and, inside it, the time
// spent waiting for the device (copies + kernel), so that a Laplace user sees where a decode step goes without a
// profiler. Device-pointer entry points only enqueue work and are not timed.
struct EntryProf { const char* name; long calls = 0; double wall = 0.0, device_wait = 0.0; };
struct Prof {
    bool on = std::getenv("LAPLACE_PROF") != nullptr;
    EntryProf e[3] = {{"gemm"}, {"moe_gemv"}, {"moe_gemv_multi"}};
    ~Prof() {
        if (!on) return;
        for (const EntryProf& p : e)
            if (p.calls)
                std::fprintf(stderr, "PROF laplace_cuda_%s: %.3f s over %ld calls (%.1f us per call; %.1f us of it waiting for the GPU)\n",
                             p.name, p.wall, p.calls, 1e6 * p.wall / p.calls, 1e6 * p.device_wait / p.calls);
    }
};
Prof g_prof;
struct ProfScope {
    EntryProf& p;
    std::chrono::steady_clock::time_point t0;
    explicit ProfScope(int which) : p(g_prof.e[which]) { if (g_prof.on) t0 = std::chrono::steady_clock::now(); }
    ~ProfScope() {
        if (g_prof.on) { p.wall += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); p.calls++; }
    }
};

}  // namespace

Context& ctx() { return g_ctx; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

int cuda_check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return LAPLACE_OK;
    return fail(LAPLACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

namespace {

int require_ready() {
    if (!g_ctx.ready) return fail(LAPLACE_ERR_STATE, "laplace_cuda_init has not been called (or found no GPU)");
    return LAPLACE_OK;
}

// Drains the stream, then reads and clears the status word. The word lives in
// mapped pinned host memory, so reading it costs no copy.
int check_device_status(cudaStream_t st, EntryProf* prof = nullptr) {
    const auto t0 = std::chrono::steady_clock::now();
    cudaError_t e = cudaStreamSynchronize(st);
    if (prof && g_prof.on) prof->device_wait += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (e != cudaSuccess) return cuda_check(e, "stream synchronize");
    const int h = *static_cast<volatile int*>(g_ctx.h_err);
    if (h != DEV_OK) {
        *g_ctx.h_err = DEV_OK;
        if (h == DEV_BAD_INDEX) return fail(LAPLACE_ERR_ARG, "an expert index on the device was out of range");
        return fail(LAPLACE_ERR_TIMEOUT, "a bounded device-side wait gave up (code %d)", h);
    }
    return LAPLACE_OK;
}

const uint8_t* resolve_registered(const uint8_t* w, size_t bytes) {
    for (const Region& r : g_regions)
        if (w >= r.host && w + bytes <= r.host + r.size) return r.dev + (w - r.host);
    return nullptr;
}

// Device address of `bytes` of weights at host pointer w: inside a registered
// region by offset, otherwise uploaded for this call. Q4_K rows are read with
// 16-byte vector loads and the tensor-core kernels (need_align16) read every type
// through a tensor map, so a registered tensor at an odd offset is re-staged for
// those calls as well.
int weights_on_device(const uint8_t* w, size_t bytes, uint32_t type, bool need_align16, const uint8_t** out) {
    const uint8_t* d = resolve_registered(w, bytes);
    if (d && !((type == LAPLACE_TYPE_Q4_K || need_align16) && (reinterpret_cast<uintptr_t>(d) & 15))) { *out = d; return LAPLACE_OK; }
    int rc = g_dw.ensure(bytes + 64);
    if (rc) return rc;
    rc = cuda_check(cudaMemcpyAsync(g_dw.p, w, bytes, cudaMemcpyHostToDevice, g_ctx.stream), "weight upload");
    *out = static_cast<const uint8_t*>(g_dw.p);
    return rc;
}

int dispatch_gemm_dev(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N,
                      cudaStream_t st) {
    if (f32act_type(type)) {
        // no int8 kernel in the reference for this type: fp32 activations against dequantized rows (its scalar path)
        if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return fail(LAPLACE_ERR_ARG, "gemm: null pointer or M=%d K=%d N=%d", M, K, N);
        return launch_gemm_f32act(x, w, type, y, M, K, N, st);
    }
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !y) return fail(LAPLACE_ERR_ARG, "gemm: null pointer");
    if (M <= 0 || N <= 0 || K <= 0) return fail(LAPLACE_ERR_ARG, "gemm: M=%d K=%d N=%d", M, K, N);
    if (K % block_elems(type)) return fail(LAPLACE_ERR_ARG, "gemm: K=%d is not a multiple of %d", K, block_elems(type));
    // Prefill: tensor-core GEMM where one exists for the type.
    if (gemm_sa_supports(type, M, K, N)) return launch_gemm_sa(x, w, type, y, M, K, N, st);
    // Small M (or a K that is not a multiple of 256): one streaming pass per group of up to 8 activation rows.
    // Rows per pass: up to 8, fewer when K is so long that 8 quantized activation rows
    // (~1.45 bytes per value) would leave the weight rings under half of shared memory.
    int per = 8;
    while (per > 1 && static_cast<double>(per) * K * 1.45 > 112.0 * 1024.0) --per;
    for (int m0 = 0; m0 < M; m0 += per) {
        GemvArgs a{};
        a.x = x + static_cast<size_t>(m0) * K;
        a.w = w;
        a.y = y + static_cast<size_t>(m0) * N;
        a.type = type;
        a.M = (M - m0) < per ? (M - m0) : per;
        a.K = K; a.N = N; a.n_seg = 1; a.per_seg_x = 0; a.expert_idx = nullptr;
        int rc = launch_gemv_stream(a, st);
        if (rc) return rc;
    }
    return LAPLACE_OK;
}

int dispatch_moe_dev(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx, int n_experts,
                     float* y, int K, int N, int per_expert_x, cudaStream_t st) {
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !y || !expert_idx) return fail(LAPLACE_ERR_ARG, "moe_gemv: null pointer");
    if (n_experts <= 0 || N <= 0 || K <= 0) return fail(LAPLACE_ERR_ARG, "moe_gemv: n_experts=%d K=%d N=%d", n_experts, K, N);
    GemvArgs a{};
    a.x = x; a.w = w; a.y = y; a.type = type; a.M = 1; a.K = K; a.N = N;
    a.n_seg = n_experts; a.per_seg_x = per_expert_x ? 1 : 0; a.expert_idx = expert_idx;
    return launch_gemv_stream(a, st);
}

int moe_host(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx, int n_experts,
             float* y, int K, int N, int per_expert_x) {
    std::lock_guard<std::mutex> lk(g_mu);
    ProfScope prof(per_expert_x ? 2 : 1);
    int rc = require_ready();
    if (rc) return rc;
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !y || !expert_idx) return fail(LAPLACE_ERR_ARG, "moe_gemv: null pointer");
    if (n_experts <= 0 || N <= 0 || K <= 0 || K % block_elems(type))
        return fail(LAPLACE_ERR_ARG, "moe_gemv: n_experts=%d K=%d N=%d", n_experts, K, N);
    int max_e = 0;
    for (int k = 0; k < n_experts; ++k) {
        if (expert_idx[k] < 0) return fail(LAPLACE_ERR_ARG, "moe_gemv: negative expert index");
        if (expert_idx[k] > max_e) max_e = expert_idx[k];
    }
    cudaStream_t st = g_ctx.stream;
    const size_t per_expert = static_cast<size_t>(N) * row_bytes(type, K);
    const uint8_t* dw = nullptr;
    if ((rc = weights_on_device(w, per_expert * (static_cast<size_t>(max_e) + 1), type, false, &dw))) return rc;
    const size_t xb = sizeof(float) * static_cast<size_t>(per_expert_x ? n_experts : 1) * K;
    const size_t yb = sizeof(float) * static_cast<size_t>(n_experts) * N;
    if ((rc = g_hx.ensure(xb + sizeof(int) * n_experts)) || (rc = g_hy.ensure(yb)) || (rc = g_dx.ensure(xb)) ||
        (rc = g_dy.ensure(yb)) || (rc = g_didx.ensure(sizeof(int) * n_experts)))
        return rc;
    std::memcpy(g_hx.p, x, xb);
    std::memcpy(static_cast<uint8_t*>(g_hx.p) + xb, expert_idx, sizeof(int) * n_experts);
    cudaMemcpyAsync(g_dx.p, g_hx.p, xb, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(g_didx.p, static_cast<uint8_t*>(g_hx.p) + xb, sizeof(int) * n_experts, cudaMemcpyHostToDevice, st);
    rc = dispatch_moe_dev(static_cast<const float*>(g_dx.p), dw, type, static_cast<const int*>(g_didx.p), n_experts,
                          static_cast<float*>(g_dy.p), K, N, per_expert_x, st);
    if (rc) return rc;
    cudaMemcpyAsync(g_hy.p, g_dy.p, yb, cudaMemcpyDeviceToHost, st);
    if ((rc = check_device_status(st, &prof.p))) return rc;
    std::memcpy(y, g_hy.p, yb);
    return LAPLACE_OK;
}

}  // namespace
}  // namespace lp

using namespace lp;

extern "C" {

int laplace_cuda_init(int device) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_ctx.ready && g_ctx.device == device) return LAPLACE_OK;
    if (g_ctx.ready) return fail(LAPLACE_ERR_STATE, "already bound to device %d", g_ctx.device);
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0)
        return fail(LAPLACE_ERR_STATE, "no CUDA device: %s", e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= n) return fail(LAPLACE_ERR_ARG, "device %d out of range (have %d)", device, n);
    int rc;
    if ((rc = cuda_check(cudaSetDevice(device), "cudaSetDevice"))) return rc;
    cudaDeviceProp prop;
    if ((rc = cuda_check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties"))) return rc;
    if (prop.major != 10)
        return fail(LAPLACE_ERR_STATE, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    g_ctx.device = device;
    g_ctx.sm_count = prop.multiProcessorCount;
    g_ctx.smem_optin = prop.sharedMemPerBlockOptin;
    g_ctx.smem_per_sm = prop.sharedMemPerMultiprocessor;
    if ((rc = cuda_check(cudaStreamCreateWithFlags(&g_ctx.stream, cudaStreamNonBlocking), "cudaStreamCreate"))) return rc;
    if ((rc = cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&g_ctx.h_err), sizeof(int), cudaHostAllocMapped),
                         "cudaHostAlloc status"))) return rc;
    *g_ctx.h_err = DEV_OK;
    if ((rc = cuda_check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_ctx.d_err), g_ctx.h_err, 0),
                         "cudaHostGetDevicePointer status"))) return rc;
    g_ctx.ready = true;
    return LAPLACE_OK;
}

void laplace_cuda_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_ctx.ready) return;
    cudaSetDevice(g_ctx.device);
    cudaStreamSynchronize(g_ctx.stream);
    for (Region& r : g_regions) cudaFree(r.dev);
    g_regions.clear();
    g_dx.release(); g_dy.release(); g_dw.release(); g_didx.release(); g_dq.release();
    g_hx.release(); g_hy.release();
    release_gemm_sa_scratch();
    release_moe_sa_scratch();
    cudaFreeHost(g_ctx.h_err);
    cudaStreamDestroy(g_ctx.stream);
    g_ctx = Context{};
}

int laplace_cuda_sync(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = require_ready();
    if (rc) return rc;
    return check_device_status(g_ctx.stream);
}

int laplace_cuda_sync_stream(void* stream) {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = require_ready();
    if (rc) return rc;
    if (stream) {
        cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return cuda_check(e, "stream synchronize");
    }
    return check_device_status(g_ctx.stream);
}

const char* laplace_cuda_last_error(void) { return g_err; }

int laplace_cuda_sm_count(void) { return g_ctx.ready ? g_ctx.sm_count : 0; }

int laplace_cuda_last_path(void) { return g_ctx.last_path; }

long long laplace_cuda_launch_count(int reset) {
    long long v = g_ctx.launches;
    if (reset) g_ctx.launches = 0;
    return v;
}

int laplace_cuda_register_weights(const void* base, size_t size) {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = require_ready();
    if (rc) return rc;
    if (!base || !size) return fail(LAPLACE_ERR_ARG, "register_weights: empty region");
    const uint8_t* h = static_cast<const uint8_t*>(base);
    for (Region& r : g_regions)
        if (r.host == h) {                      // same base registered again: refresh the copy
            if (r.size != size) return fail(LAPLACE_ERR_ARG, "register_weights: region re-registered with another size");
            return cuda_check(cudaMemcpy(r.dev, h, size, cudaMemcpyHostToDevice), "weight upload");
        }
    uint8_t* d = nullptr;
    if ((rc = cuda_check(cudaMalloc(&d, size + 64), "cudaMalloc weights"))) return rc;   // slack: 16-byte read-ahead
    if ((rc = cuda_check(cudaMemcpy(d, h, size, cudaMemcpyHostToDevice), "weight upload"))) { cudaFree(d); return rc; }
    cudaMemset(d + size, 0, 64);
    g_regions.push_back(Region{h, size, d});
    return LAPLACE_OK;
}

int laplace_cuda_unregister_weights(const void* base) {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = require_ready();
    if (rc) return rc;
    for (size_t i = 0; i < g_regions.size(); ++i)
        if (g_regions[i].host == base) {
            cudaStreamSynchronize(g_ctx.stream);
            cudaFree(g_regions[i].dev);
            g_regions.erase(g_regions.begin() + i);
            return LAPLACE_OK;
        }
    return fail(LAPLACE_ERR_ARG, "unregister_weights: region not registered");
}

void laplace_cuda_nsplit(int N, int rank, int world, int* row_begin, int* row_end) {
    if (world < 1) world = 1;
    if (rank < 0) rank = 0;
    if (rank >= world) rank = world - 1;
    // contiguous ranges, sizes differ by at most one 16-row group
    const long long groups = (static_cast<long long>(N) + 15) / 16;
    long long b = groups * rank / world * 16, e = groups * (rank + 1) / world * 16;
    if (b > N) b = N;
    if (e > N) e = N;
    if (row_begin) *row_begin = static_cast<int>(b);
    if (row_end) *row_end = static_cast<int>(e);
}

int laplace_cuda_gemm(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N) {
    std::lock_guard<std::mutex> lk(g_mu);
    ProfScope prof(0);
    int rc = require_ready();
    if (rc) return rc;
    const bool other = f32act_type(type);
    if (!other && !block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !y) return fail(LAPLACE_ERR_ARG, "gemm: null pointer");
    // F32 / F16 / BF16 rows are walked 16 values at a time; another K is left to the caller's scalar path
    if (other && (type == 0 || type == 1 || type == 30) && K > 0 && K % 16) return LAPLACE_UNSUPPORTED;
    if (M <= 0 || N <= 0 || K <= 0 || K % (other ? any_block_elems(type) : block_elems(type))) return fail(LAPLACE_ERR_ARG, "gemm: M=%d K=%d N=%d", M, K, N);
    cudaStream_t st = g_ctx.stream;
    const uint8_t* dw = nullptr;
    if ((rc = weights_on_device(w, static_cast<size_t>(N) * (other ? any_row_bytes(type, K) : row_bytes(type, K)), type, type == 0, &dw))) return rc;
    const size_t xb = sizeof(float) * static_cast<size_t>(M) * K, yb = sizeof(float) * static_cast<size_t>(M) * N;
    if ((rc = g_hx.ensure(xb)) || (rc = g_hy.ensure(yb)) || (rc = g_dx.ensure(xb)) || (rc = g_dy.ensure(yb))) return rc;
    std::memcpy(g_hx.p, x, xb);
    cudaMemcpyAsync(g_dx.p, g_hx.p, xb, cudaMemcpyHostToDevice, st);
    // Decode calls: the kernel writes y straight into the pinned host buffer (which the device can address) in
    // coalesced stores from its epilogue, so no device-to-host copy has to be queued behind it.
    const bool direct = !other && M <= 8 && static_cast<size_t>(M) * (static_cast<size_t>(N) / g_ctx.sm_count + 256) * sizeof(float) < 40 * 1024;
    if (direct) {
        PeerOut po{};
        po.y[0] = static_cast<float*>(g_hy.p);
        po.world = 1; po.rank = 0; po.ld = N; po.col0 = 0;
        GemvArgs a{};
        a.x = static_cast<const float*>(g_dx.p); a.w = dw; a.y = nullptr; a.type = type; a.M = M; a.K = K; a.N = N; a.n_seg = 1;
        a.peers = &po;
        rc = launch_gemv_stream(a, st);
    } else {
        rc = dispatch_gemm_dev(static_cast<const float*>(g_dx.p), dw, type, static_cast<float*>(g_dy.p), M, K, N, st);
        if (rc == LAPLACE_OK) cudaMemcpyAsync(g_hy.p, g_dy.p, yb, cudaMemcpyDeviceToHost, st);
    }
    if (rc) return rc;
    if ((rc = check_device_status(st, &prof.p))) return rc;
    std::memcpy(y, g_hy.p, yb);
    return LAPLACE_OK;
}

int laplace_cuda_moe_gemv(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx, int n_experts,
                          float* y, int K, int N) {
    return moe_host(x, w, type, expert_idx, n_experts, y, K, N, 0);
}

int laplace_cuda_moe_gemv_multi(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                                int n_experts, float* y, int K, int N) {
    return moe_host(x, w, type, expert_idx, n_experts, y, K, N, 1);
}

int laplace_cuda_gemm_dev(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N,
                          void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    return dispatch_gemm_dev(x, w, type, y, M, K, N, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_dequantize_dev(const uint8_t* w, uint32_t type, float* dst, long long n, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    return launch_dequantize(w, type, dst, n, 1.0f, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_embed_rows_dev(const uint8_t* w, uint32_t type, const int* tokens, int M, int H, long long vocab, float scale,
                                float* dst, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    return launch_embed_rows(w, type, tokens, M, H, vocab, scale, dst, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_lm_head_dev(const float* x, const uint8_t* w, uint32_t type, float* y, int M, int K, int N, float softcap,
                             void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream;
    if ((rc = dispatch_gemm_dev(x, w, type, y, M, K, N, st))) return rc;
    if (softcap > 0.0f) return launch_softcap(y, static_cast<long long>(M) * N, softcap, st);
    return LAPLACE_OK;
}

int laplace_cuda_gemm_multi_dev(const float* x, const float* norm_weight, float norm_eps, float* x_norm_out,
                                const laplace_cuda_matrix* mats, int n_mats, uint32_t type, int M, int K, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !mats || n_mats <= 0 || n_mats > 8) return fail(LAPLACE_ERR_ARG, "gemm_multi: null pointer or %d matrices (1..8)", n_mats);
    if (M <= 0 || K <= 0 || K % block_elems(type)) return fail(LAPLACE_ERR_ARG, "gemm_multi: M=%d K=%d", M, K);
    const uint8_t* ws[8]; float* ys[8]; int ns[8];
    for (int i = 0; i < n_mats; ++i) { ws[i] = mats[i].w; ys[i] = mats[i].y; ns[i] = mats[i].N; }
    if (M > 8) {
        // prefill: one (normalising) quantizer launch, then the tensor-core GEMM per matrix on the shared operand
        for (int i = 0; i < n_mats; ++i) {
            if (!ws[i] || !ys[i] || ns[i] <= 0) return fail(LAPLACE_ERR_ARG, "gemm_multi: matrix %d: null pointer or no rows", i);
            if (!gemm_sa_supports(type, M, K, ns[i]))
                return fail(LAPLACE_ERR_ARG, "gemm_multi: M=%d K=%d: prefill calls need K to be a multiple of 256", M, K);
        }
        return launch_gemm_sa_multi(x, norm_weight, norm_eps, x_norm_out, ws, ys, ns, n_mats, type, M, K,
                                    stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
    }
    GemvArgs a{};
    a.x = x; a.type = type; a.M = M; a.K = K; a.n_seg = 1;
    a.n_mats = n_mats; a.mat_w = ws; a.mat_y = ys; a.mat_n = ns;
    a.norm_w = norm_weight; a.norm_eps = norm_eps; a.x_norm_out = x_norm_out;
    return launch_gemv_stream(a, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_moe_gemv_dev(const float* x, const uint8_t* w, uint32_t type, const int* expert_idx,
                              int n_experts, float* y, int K, int N, int per_expert_x, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    return dispatch_moe_dev(x, w, type, expert_idx, n_experts, y, K, N, per_expert_x,
                            stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_moe_grouped_dev(const float* x, const uint8_t* w, uint32_t type, const int* pair_expert,
                                 const int* pair_row, int n_pairs, int n_experts_total, float* y, int K, int N,
                                 void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !y || !pair_expert) return fail(LAPLACE_ERR_ARG, "moe_grouped: null pointer");
    if (n_pairs <= 0 || n_experts_total <= 0 || N <= 0 || K <= 0 || K % block_elems(type))
        return fail(LAPLACE_ERR_ARG, "moe_grouped: pairs=%d experts=%d K=%d N=%d", n_pairs, n_experts_total, K, N);
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream;
    return launch_moe_grouped_sa(x, w, type, pair_expert, pair_row, n_pairs, n_experts_total, y, K, N, st);
}

int laplace_cuda_moe_ffn_dev(const float* x, const uint8_t* w_gate_up, const uint8_t* w_down,
                             uint32_t type_gate_up, uint32_t type_down, const int* top_idx, const float* top_w,
                             const float* down_scale, int n_tokens, int top_k, int n_experts_total, int hidden, int inter,
                             int activation, float* out, float* h_out, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!block_elems(type_gate_up) || !block_elems(type_down)) return LAPLACE_UNSUPPORTED;
    if (!x || !w_gate_up || !w_down || !top_idx || !top_w || !out) return fail(LAPLACE_ERR_ARG, "moe_ffn: null pointer");
    if (n_tokens <= 0 || top_k <= 0 || n_experts_total <= 0 || hidden <= 0 || inter <= 0 ||
        hidden % block_elems(type_gate_up) || inter % block_elems(type_down) || (activation != 0 && activation != 1))
        return fail(LAPLACE_ERR_ARG, "moe_ffn: tokens=%d top_k=%d experts=%d hidden=%d inter=%d activation=%d",
                    n_tokens, top_k, n_experts_total, hidden, inter, activation);
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream;
    return launch_moe_ffn_sa(x, w_gate_up, w_down, type_gate_up, type_down, top_idx, top_w, down_scale, n_tokens, top_k,
                             n_experts_total, hidden, inter, activation, out, h_out, st);
}

int laplace_cuda_moe_route_dev(const float* logits, int n_tokens, int n_experts, int top_k, int* top_idx, float* top_w,
                               void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!logits || !top_idx || !top_w) return fail(LAPLACE_ERR_ARG, "moe_route: null pointer");
    if (n_tokens <= 0 || n_experts <= 0 || top_k <= 0 || top_k > n_experts)
        return fail(LAPLACE_ERR_ARG, "moe_route: tokens=%d experts=%d top_k=%d", n_tokens, n_experts, top_k);
    return launch_moe_route(logits, n_tokens, n_experts, top_k, top_idx, top_w, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_moe_pack_dev(const float* x, const int* top_idx, const float* top_w, int n_tokens, int hidden, int top_k,
                              float* packed, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!x || !top_idx || !top_w || !packed || n_tokens <= 0 || hidden <= 0 || top_k <= 0)
        return fail(LAPLACE_ERR_ARG, "moe_pack: bad argument");
    return launch_moe_pack(x, top_idx, top_w, n_tokens, hidden, top_k, packed, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_moe_unpack_dev(const float* packed, int n_tokens, int hidden, int top_k, int expert_first, int expert_count,
                                float* x, int* idx_local, float* top_w, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!packed || !x || !idx_local || !top_w || n_tokens <= 0 || hidden <= 0 || top_k <= 0 || expert_count <= 0)
        return fail(LAPLACE_ERR_ARG, "moe_unpack: bad argument");
    return launch_moe_unpack(packed, n_tokens, hidden, top_k, expert_first, expert_count, x, idx_local, top_w,
                             stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

/* ---- fused all-gather of a row-split decode matmul over peer memory ---- */

int laplace_cuda_peer_alloc(size_t bytes, void** dev_ptr, unsigned char* handle64) {
    int rc = require_ready();
    if (rc) return rc;
    if (!dev_ptr || !handle64 || bytes == 0) return fail(LAPLACE_ERR_ARG, "peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    void* p = nullptr;
    if ((rc = cuda_check(cudaMalloc(&p, bytes), "cudaMalloc peer buffer"))) return rc;
    if ((rc = cuda_check(cudaMemset(p, 0, bytes), "cudaMemset peer buffer")) ||
        (rc = cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize"))) { cudaFree(p); return rc; }   // zeroed before anyone maps it
    cudaIpcMemHandle_t h;
    if ((rc = cuda_check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle"))) { cudaFree(p); return rc; }
    std::memcpy(handle64, &h, 64);
    *dev_ptr = p;
    return LAPLACE_OK;
}

int laplace_cuda_peer_open(const unsigned char* handle64, void** dev_ptr) {
    int rc = require_ready();
    if (rc) return rc;
    if (!dev_ptr || !handle64) return fail(LAPLACE_ERR_ARG, "peer_open: bad argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* p = nullptr;
    if ((rc = cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle"))) return rc;
    *dev_ptr = p;
    return LAPLACE_OK;
}

int laplace_cuda_peer_close(void* dev_ptr) {
    return dev_ptr ? cuda_check(cudaIpcCloseMemHandle(dev_ptr), "cudaIpcCloseMemHandle") : LAPLACE_OK;
}

int laplace_cuda_peer_free(void* dev_ptr) {
    return dev_ptr ? cuda_check(cudaFree(dev_ptr), "cudaFree peer buffer") : LAPLACE_OK;
}

int laplace_cuda_gemm_allgather_dev(const float* x, const uint8_t* w, uint32_t type,
                                    float* const* peer_y, int* const* peer_flags, int* step_counter,
                                    unsigned* done_counter, int rank, int world, int row_begin, int n_total,
                                    int M, int K, int n_local, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !peer_y || !peer_flags || !step_counter || !done_counter)
        return fail(LAPLACE_ERR_ARG, "gemm_allgather: null pointer");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || M < 1 || M > 8 || n_local <= 0 || K <= 0 ||
        K % block_elems(type) || row_begin < 0 || row_begin + n_local > n_total)
        return fail(LAPLACE_ERR_ARG, "gemm_allgather: rank=%d world=%d M=%d K=%d rows [%d,%d) of %d", rank, world, M, K,
                    row_begin, row_begin + n_local, n_total);
    PeerOut po{};
    for (int r = 0; r < world; ++r) {
        if (!peer_y[r] || !peer_flags[r]) return fail(LAPLACE_ERR_ARG, "gemm_allgather: null peer pointer %d", r);
        po.y[r] = peer_y[r];
        po.flags[r] = peer_flags[r];
    }
    po.step_ctr = step_counter; po.done_ctr = done_counter;
    po.world = world; po.rank = rank; po.ld = n_total; po.col0 = row_begin;
    GemvArgs a{};
    a.x = x; a.w = w; a.y = nullptr; a.type = type; a.M = M; a.K = K; a.N = n_local; a.n_seg = 1;
    a.peers = &po;
    return launch_gemv_stream(a, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_gemm_peers_dev(const float* x, const uint8_t* w, uint32_t type, float* const* peer_y, int world,
                                int row_begin, int n_total, int M, int K, int n_local, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!x || !w || !peer_y) return fail(LAPLACE_ERR_ARG, "gemm_peers: null pointer");
    if (world < 1 || world > MAX_PEERS || M < 1 || n_local <= 0 || K <= 0 || row_begin < 0 || row_begin + n_local > n_total)
        return fail(LAPLACE_ERR_ARG, "gemm_peers: world=%d M=%d K=%d rows [%d,%d) of %d", world, M, K, row_begin, row_begin + n_local, n_total);
    if (!gemm_sa_supports(type, M, K, n_local)) return LAPLACE_UNSUPPORTED;
    PeerOut po{};
    for (int r = 0; r < world; ++r) {
        if (!peer_y[r]) return fail(LAPLACE_ERR_ARG, "gemm_peers: null peer pointer %d", r);
        po.y[r] = peer_y[r];
    }
    po.world = world; po.ld = n_total; po.col0 = row_begin;
    return launch_gemm_sa_peers(x, w, type, po, M, K, n_local, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_allgather_step_wait_dev(int* const* peer_flags, int* step_counter, int rank, int world, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!peer_flags || !step_counter || world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(LAPLACE_ERR_ARG, "allgather_step_wait: bad argument");
    PeerOut po{};
    for (int r = 0; r < world; ++r) {
        if (!peer_flags[r]) return fail(LAPLACE_ERR_ARG, "allgather_step_wait: null peer pointer %d", r);
        po.flags[r] = peer_flags[r];
    }
    po.step_ctr = step_counter; po.world = world; po.rank = rank;
    return launch_allgather_wait(po, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream, true);
}

int laplace_cuda_allgather_wait_dev(int* const* peer_flags, int* step_counter, int rank, int world, void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!peer_flags || !step_counter || world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(LAPLACE_ERR_ARG, "allgather_wait: bad argument");
    PeerOut po{};
    for (int r = 0; r < world; ++r) {
        if (!peer_flags[r]) return fail(LAPLACE_ERR_ARG, "allgather_wait: null peer pointer %d", r);
        po.flags[r] = peer_flags[r];
    }
    po.step_ctr = step_counter; po.world = world; po.rank = rank;
    return launch_allgather_wait(po, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_quantize_act_dev(const float* x, int M, int K, int8_t* q, float* d, float* sum, int16_t* isum,
                                  void* stream) {
    int rc = require_ready();
    if (rc) return rc;
    if (!x) return fail(LAPLACE_ERR_ARG, "quantize: null input");
    return launch_quantize_act(x, M, K, q, d, sum, isum, stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream);
}

int laplace_cuda_debug_blocksums_dev(const float* x, const uint8_t* w, uint32_t type, int32_t* out, int M, int K,
                                     int N, void* stream) {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = require_ready();
    if (rc) return rc;
    if (!block_elems(type)) return LAPLACE_UNSUPPORTED;
    if (!x || !w || !out) return fail(LAPLACE_ERR_ARG, "blocksums: null pointer");
    if (M <= 0 || N <= 0 || K <= 0 || K % block_elems(type)) return fail(LAPLACE_ERR_ARG, "blocksums: M=%d K=%d N=%d", M, K, N);
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : g_ctx.stream;
    if ((rc = g_dq.ensure(static_cast<size_t>(M) * K))) return rc;
    if ((rc = launch_quantize_act(x, M, K, static_cast<int8_t*>(g_dq.p), nullptr, nullptr, nullptr, st))) return rc;
    return launch_blocksums_q(static_cast<const int8_t*>(g_dq.p), w, type, out, M, K, N, st);
}

}  // extern "C"
