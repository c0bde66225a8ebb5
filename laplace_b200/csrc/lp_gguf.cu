// lp_gguf.cu - GGUF file -> HBM, straight from the mapped file, with the placement the matmul path uses.
//
// Laplace opens a GGUF file with GGUFContext::open (src/gguf.cpp:217-335: header, metadata, tensor table, data
// section aligned to general.alignment), keeps the mapping for the life of the process and hands the whole region
// to the back-end once (matmul_register_weights, src/main.cpp:705). On-disk blocks ARE the wire format of the
// matmul kernels (src/tensor.h:130-163), so nothing has to be converted; what a multi-GPU box needs in addition is
// the split: every GPU takes its own rows of a matrix (a row is a contiguous byte range) and its own experts of a
// stacked expert tensor, and copies only those bytes.
//
// The file is parsed here from the published GGUF layout (v2 / v3, little endian):
//   u32 magic 'GGUF', u32 version, u64 tensor count, u64 key/value count,
//   key/values  (string key, u32 value type, value; strings are u64 length + bytes; arrays are u32 element type,
//                u64 count, elements),
//   tensor infos (string name, u32 n_dims, u64 dims[n_dims] innermost first, u32 ggml type, u64 offset),
//   padding to general.alignment (default 32), tensor data.
// Placement of a tensor for rank r of `world`:
//   3 dims and more, quantized   dims = [K, N, E]: whole experts, expert e on GPU e / ceil(E / world)
//                                 (src/model.h:82 stacks an expert's rows contiguously)
//   2 dims, at least 256 rows    dims = [K, N]: rows [b, e) of laplace_cuda_nsplit(N, r, world) - unless the
//                                 caller names the tensor in `replicate` (token embeddings are read by row index)
//   everything else              whole tensor on every GPU (norm weights, biases, small matrices)
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "lp_common.cuh"

namespace lp {
namespace {

struct TypeGeo { int elems, bytes; };
// elements and bytes per block of every ggml type Laplace's tensor table knows (src/tensor.h:41-100)
TypeGeo type_geo(uint32_t t) {
    switch (t) {
        case 0: return {1, 4};        // F32
        case 1: return {1, 2};        // F16
        case 2: return {32, 18};      // Q4_0
        case 3: return {32, 20};      // Q4_1
        case 6: return {32, 22};      // Q5_0
        case 7: return {32, 24};      // Q5_1
        case 8: return {32, 34};      // Q8_0
        case 9: return {32, 36};      // Q8_1
        case 10: return {256, 84};    // Q2_K
        case 11: return {256, 110};   // Q3_K
        case 12: return {256, 144};   // Q4_K
        case 13: return {256, 176};   // Q5_K
        case 14: return {256, 210};   // Q6_K
        case 15: return {256, 354};   // Q8_K as Laplace sizes it (2 + 256 + 64 + 32)
        case 24: return {1, 1};       // I8
        case 25: return {1, 2};       // I16
        case 26: return {1, 4};       // I32
        case 27: return {1, 8};       // I64
        case 28: return {1, 8};       // F64
        case 30: return {1, 2};       // BF16
        default: return {0, 0};
    }
}

struct Reader {
    const uint8_t* p; size_t n, at = 0;
    template <class T> bool get(T& v) { if (n - at < sizeof(T)) return false; std::memcpy(&v, p + at, sizeof(T)); at += sizeof(T); return true; }
    bool str(std::string& s) {
        uint64_t len;
        if (!get(len) || len > n - at) return false;
        s.assign(reinterpret_cast<const char*>(p + at), static_cast<size_t>(len));
        at += static_cast<size_t>(len);
        return true;
    }
    bool skip(size_t k) { if (k > n - at) return false; at += k; return true; }
};
// bytes of a fixed-size metadata value, 0 for strings and arrays
size_t scalar_size(uint32_t vt) {
    switch (vt) {
        case 0: case 1: case 7: return 1;          // u8, i8, bool
        case 2: case 3: return 2;                  // u16, i16
        case 4: case 5: case 6: return 4;          // u32, i32, f32
        case 10: case 11: case 12: return 8;       // u64, i64, f64
        default: return 0;
    }
}

struct Meta { uint32_t vt; uint64_t bits; double f; std::string s; };     // scalars and strings only; arrays are skipped
struct TensorRec {
    std::string name;
    uint32_t type = 0, n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t file_off = 0, bytes = 0;          // whole tensor in the file
    // this rank's part
    int      kind = 0;                          // 0 replicated, 1 rows split, 2 experts split
    uint64_t row_begin = 0, row_end = 0;        // kind 1: rows of this rank; otherwise [0, rows)
    uint64_t exp_begin = 0, exp_end = 0;        // kind 2: experts of this rank; otherwise [0, experts)
    uint64_t part_off = 0, part_bytes = 0;      // byte range of the part inside the tensor
    uint8_t* dev = nullptr;
};

}  // namespace
}  // namespace lp

struct laplace_cuda_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_off = 0;
    int rank = 0, world = 1;
    std::map<std::string, lp::Meta> meta;
    std::vector<lp::TensorRec> tensors;
    std::map<std::string, size_t> by_name;
    uint8_t* arena = nullptr;                    // one allocation holds every part
    size_t arena_bytes = 0;
};

namespace lp {
namespace {

int parse(laplace_cuda_gguf& g) {
    Reader r{g.map, g.size};
    uint32_t magic = 0;
    uint64_t n_tensors = 0, n_kv = 0;
    if (!r.get(magic) || magic != 0x46554747u) return fail(LAPLACE_ERR_ARG, "gguf: bad magic");
    if (!r.get(g.version) || g.version < 2 || g.version > 3) return fail(LAPLACE_ERR_ARG, "gguf: version %u (2 or 3 expected)", g.version);
    if (!r.get(n_tensors) || !r.get(n_kv)) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside the header");
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key;
        uint32_t vt = 0;
        if (!r.str(key) || !r.get(vt)) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside key/value %llu", static_cast<unsigned long long>(i));
        Meta m{vt, 0, 0.0, {}};
        if (vt == 8) {
            if (!r.str(m.s)) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside the value of '%s'", key.c_str());
        } else if (vt == 9) {
            uint32_t et = 0;
            uint64_t cnt = 0;
            if (!r.get(et) || !r.get(cnt)) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside array '%s'", key.c_str());
            if (et == 8) {
                std::string s;
                for (uint64_t k = 0; k < cnt; ++k) if (!r.str(s)) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside array '%s'", key.c_str());
            } else {
                const size_t es = scalar_size(et);
                if (!es || cnt > (r.n - r.at) / es || !r.skip(static_cast<size_t>(cnt) * es))
                    return fail(LAPLACE_ERR_ARG, "gguf: array '%s' of element type %u cannot be read", key.c_str(), et);
            }
        } else {
            const size_t sz = scalar_size(vt);
            if (!sz || r.n - r.at < sz) return fail(LAPLACE_ERR_ARG, "gguf: value type %u of '%s' cannot be read", vt, key.c_str());
            uint64_t bits = 0;
            std::memcpy(&bits, r.p + r.at, sz);
            r.at += sz;
            m.bits = bits;
            switch (vt) {
                case 1: m.f = static_cast<double>(static_cast<int8_t>(bits)); break;
                case 3: m.f = static_cast<double>(static_cast<int16_t>(bits)); break;
                case 5: m.f = static_cast<double>(static_cast<int32_t>(bits)); break;
                case 11: m.f = static_cast<double>(static_cast<int64_t>(bits)); break;
                case 6: { float f; std::memcpy(&f, &bits, 4); m.f = f; break; }
                case 12: { double d; std::memcpy(&d, &bits, 8); m.f = d; break; }
                default: m.f = static_cast<double>(bits);
            }
        }
        g.meta[key] = std::move(m);
    }
    g.tensors.resize(static_cast<size_t>(n_tensors));
    for (TensorRec& t : g.tensors) {
        uint64_t off = 0;
        if (!r.str(t.name) || !r.get(t.n_dims) || t.n_dims > 4) return fail(LAPLACE_ERR_ARG, "gguf: bad tensor record");
        for (uint32_t d = 0; d < t.n_dims; ++d) if (!r.get(t.dims[d])) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside tensor '%s'", t.name.c_str());
        if (!r.get(t.type) || !r.get(off)) return fail(LAPLACE_ERR_ARG, "gguf: file ends inside tensor '%s'", t.name.c_str());
        t.file_off = off;       // relative to the data section for now
    }
    auto al = g.meta.find("general.alignment");
    if (al != g.meta.end() && al->second.bits) g.alignment = al->second.bits;
    g.data_off = (r.at + g.alignment - 1) / g.alignment * g.alignment;
    for (TensorRec& t : g.tensors) {
        const TypeGeo geo = type_geo(t.type);
        uint64_t n = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) n *= t.dims[d];
        if (!geo.elems) return fail(LAPLACE_ERR_ARG, "gguf: tensor '%s' has ggml type %u, which this loader cannot size", t.name.c_str(), t.type);
        t.bytes = (n + geo.elems - 1) / geo.elems * geo.bytes;
        t.file_off += g.data_off;
        if (t.file_off > g.size || t.bytes > g.size - t.file_off)
            return fail(LAPLACE_ERR_ARG, "gguf: tensor '%s' reaches past the end of the file", t.name.c_str());
    }
    return LAPLACE_OK;
}

void place(laplace_cuda_gguf& g, const std::vector<std::string>& replicate) {
    for (size_t i = 0; i < g.tensors.size(); ++i) {
        TensorRec& t = g.tensors[i];
        g.by_name[t.name] = i;
        const TypeGeo geo = type_geo(t.type);
        const uint64_t K = t.dims[0], rows = t.n_dims >= 2 ? t.dims[1] : 1;
        uint64_t experts = 1;
        for (uint32_t d = 2; d < t.n_dims; ++d) experts *= t.dims[d];
        t.row_begin = 0; t.row_end = rows; t.exp_begin = 0; t.exp_end = experts;
        t.part_off = 0; t.part_bytes = t.bytes; t.kind = 0;
        const bool whole_rows = geo.elems && K % geo.elems == 0;      // a row is a whole number of blocks
        const uint64_t rb = whole_rows ? K / geo.elems * geo.bytes : 0;
        const bool keep = std::find(replicate.begin(), replicate.end(), t.name) != replicate.end();
        if (g.world > 1 && whole_rows && !keep) {
            if (t.n_dims >= 3 && experts >= static_cast<uint64_t>(g.world)) {
                const uint64_t per = (experts + g.world - 1) / g.world;
                t.exp_begin = std::min<uint64_t>(experts, per * g.rank);
                t.exp_end = std::min<uint64_t>(experts, per * (g.rank + 1));
                t.part_off = t.exp_begin * rows * rb;
                t.part_bytes = (t.exp_end - t.exp_begin) * rows * rb;
                t.kind = 2;
            } else if (t.n_dims == 2 && rows >= 256 && rows < (1ull << 31)) {
                int b = 0, e = 0;
                laplace_cuda_nsplit(static_cast<int>(rows), g.rank, g.world, &b, &e);
                t.row_begin = static_cast<uint64_t>(b); t.row_end = static_cast<uint64_t>(e);
                t.part_off = t.row_begin * rb;
                t.part_bytes = (t.row_end - t.row_begin) * rb;
                t.kind = 1;
            }
        }
    }
}

}  // namespace
}  // namespace lp

extern "C" {

int laplace_cuda_gguf_open(const char* path, int rank, int world, const char* const* replicate, int n_replicate,
                           laplace_cuda_gguf** out) {
    using namespace lp;
    if (!path || !out || world < 1 || rank < 0 || rank >= world) return fail(LAPLACE_ERR_ARG, "gguf_open: bad argument");
    laplace_cuda_gguf* g = new laplace_cuda_gguf();
    g->rank = rank; g->world = world;
    g->fd = ::open(path, O_RDONLY);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        if (g->fd >= 0) ::close(g->fd);
        delete g;
        return fail(LAPLACE_ERR_ARG, "gguf_open: cannot open '%s'", path);
    }
    g->size = static_cast<size_t>(st.st_size);
    void* m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) { ::close(g->fd); delete g; return fail(LAPLACE_ERR_ARG, "gguf_open: cannot map '%s'", path); }
    g->map = static_cast<const uint8_t*>(m);
    std::vector<std::string> keep;
    for (int i = 0; i < n_replicate; ++i) if (replicate && replicate[i]) keep.emplace_back(replicate[i]);
    const int rc = parse(*g);
    if (rc) { laplace_cuda_gguf_close(g); return rc; }
    place(*g, keep);
    *out = g;
    return LAPLACE_OK;
}

int laplace_cuda_gguf_upload(laplace_cuda_gguf* g) {
    using namespace lp;
    if (!g) return fail(LAPLACE_ERR_ARG, "gguf_upload: null handle");
    if (g->arena) return LAPLACE_OK;
    if (!ctx().ready) return fail(LAPLACE_ERR_STATE, "laplace_cuda_init has not been called (or found no GPU)");
    // every part starts on a 256-byte boundary (bulk copies and tensor maps want 16) and is followed by slack, since
    // the streaming kernels copy whole 16-byte units and may run past a part's last row
    size_t total = 0;
    std::vector<size_t> at(g->tensors.size());
    for (size_t i = 0; i < g->tensors.size(); ++i) {
        at[i] = total;
        total += (static_cast<size_t>(g->tensors[i].part_bytes) + 64 + 255) & ~static_cast<size_t>(255);
    }
    if (total == 0) total = 256;
    int rc = cuda_check(cudaMalloc(reinterpret_cast<void**>(&g->arena), total), "cudaMalloc gguf arena");
    if (rc) { g->arena = nullptr; return rc; }
    g->arena_bytes = total;
    if ((rc = cuda_check(cudaMemsetAsync(g->arena, 0, total, ctx().stream), "cudaMemset gguf arena"))) return rc;
    // The mapping is pageable memory: the copies go through two pinned staging buffers so that reading the file
    // (page faults) and the transfer of the previous piece overlap.
    constexpr size_t CHUNK = 32u << 20;
    uint8_t* stage[2] = {nullptr, nullptr};
    cudaEvent_t ev[2];
    for (int i = 0; i < 2; ++i) {
        if ((rc = cuda_check(cudaMallocHost(reinterpret_cast<void**>(&stage[i]), CHUNK), "cudaMallocHost gguf staging"))) return rc;
        cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming);
    }
    int turn = 0;
    bool used[2] = {false, false};
    for (size_t i = 0; i < g->tensors.size() && !rc; ++i) {
        TensorRec& t = g->tensors[i];
        t.dev = g->arena + at[i];
        const uint8_t* src = g->map + t.file_off + t.part_off;
        for (uint64_t done = 0; done < t.part_bytes && !rc; done += CHUNK) {
            const size_t n = static_cast<size_t>(std::min<uint64_t>(CHUNK, t.part_bytes - done));
            if (used[turn]) cudaEventSynchronize(ev[turn]);
            std::memcpy(stage[turn], src + done, n);      // (six copying threads were measured 8x slower on the test host)
            rc = cuda_check(cudaMemcpyAsync(t.dev + done, stage[turn], n, cudaMemcpyHostToDevice, ctx().stream), "gguf upload");
            cudaEventRecord(ev[turn], ctx().stream);
            used[turn] = true;
            turn ^= 1;
        }
    }
    if (!rc) rc = cuda_check(cudaStreamSynchronize(ctx().stream), "gguf upload");
    for (int i = 0; i < 2; ++i) { cudaFreeHost(stage[i]); cudaEventDestroy(ev[i]); }
    return rc;
}

int laplace_cuda_gguf_tensor_count(const laplace_cuda_gguf* g) { return g ? static_cast<int>(g->tensors.size()) : 0; }

int laplace_cuda_gguf_tensor(const laplace_cuda_gguf* g, int index, const char* name, laplace_cuda_gguf_tensor_info* info) {
    using namespace lp;
    if (!g || !info) return fail(LAPLACE_ERR_ARG, "gguf_tensor: null argument");
    size_t i = static_cast<size_t>(index);
    if (name) {
        auto it = g->by_name.find(name);
        if (it == g->by_name.end()) return LAPLACE_UNSUPPORTED;       // no such tensor: not an error, files differ
        i = it->second;
    } else if (index < 0 || i >= g->tensors.size()) {
        return fail(LAPLACE_ERR_ARG, "gguf_tensor: index %d of %zu", index, g->tensors.size());
    }
    const TensorRec& t = g->tensors[i];
    info->name = t.name.c_str();
    info->type = t.type;
    info->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) info->dims[d] = t.dims[d];
    info->kind = t.kind;
    info->row_begin = t.row_begin; info->row_end = t.row_end;
    info->expert_begin = t.exp_begin; info->expert_end = t.exp_end;
    info->file_offset = t.file_off + t.part_off;
    info->bytes = t.part_bytes;
    info->host = g->map + t.file_off + t.part_off;
    info->dev = t.dev;
    return LAPLACE_OK;
}

int laplace_cuda_gguf_meta_u64(const laplace_cuda_gguf* g, const char* key, unsigned long long* value) {
    if (!g || !key || !value) return lp::fail(LAPLACE_ERR_ARG, "gguf_meta: null argument");
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.vt == 8 || it->second.vt == 9 || it->second.vt == 6 || it->second.vt == 12) return LAPLACE_UNSUPPORTED;
    *value = it->second.bits;
    return LAPLACE_OK;
}
int laplace_cuda_gguf_meta_f64(const laplace_cuda_gguf* g, const char* key, double* value) {
    if (!g || !key || !value) return lp::fail(LAPLACE_ERR_ARG, "gguf_meta: null argument");
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.vt == 8 || it->second.vt == 9) return LAPLACE_UNSUPPORTED;
    *value = it->second.f;
    return LAPLACE_OK;
}
const char* laplace_cuda_gguf_meta_str(const laplace_cuda_gguf* g, const char* key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    return (it == g->meta.end() || it->second.vt != 8) ? nullptr : it->second.s.c_str();
}

void laplace_cuda_gguf_close(laplace_cuda_gguf* g) {
    if (!g) return;
    if (g->arena) cudaFree(g->arena);
    if (g->map) munmap(const_cast<uint8_t*>(g->map), g->size);
    if (g->fd >= 0) ::close(g->fd);
    delete g;
}

}  // extern "C"
