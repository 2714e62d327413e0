// GGUF model files to device-resident weights: the reading half of the reference's loader
// (src/graph/gguf/loader.cpp; file format: GGUF v2/v3 as written by llama.cpp and by the reference's own
// scripts/make_moe_fixture.py) plus the uploads a tensor-parallel rank needs.
//
// The file is memory-mapped; header, metadata and tensor directory are parsed once into an index.  Tensor payloads
// are never copied on the host: a whole tensor or a contiguous range of rows (column-parallel shard) goes to the device
// as one asynchronous copy straight out of the mapping, and a K-range of every row (row-parallel shard: a run of
// blocks out of each row) as one strided 2-D copy, so the packed [F, K / world] matrix a rank computes on is
// assembled by the copy engine, not by host code.
#include "../../include/marmot_cuda.h"

#include "common.cuh"
#include "kernels.h"

#include <cuda_runtime.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

using namespace mcu;

namespace {

enum : uint32_t {
    GV_U8 = 0, GV_I8, GV_U16, GV_I16, GV_U32, GV_I32, GV_F32, GV_BOOL, GV_STRING, GV_ARRAY, GV_U64, GV_I64, GV_F64
};

struct MetaValue {
    uint32_t type = 0;
    uint64_t u = 0;      // integers and bool, widened
    double f = 0.0;      // floats
    std::string s;       // strings
    uint32_t elem_type = 0;
    uint64_t count = 0;  // arrays: element type and count (elements are skipped, not stored)
};

struct TensorEntry {
    std::string name;
    uint32_t type = 0, n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t offset = 0, nbytes = 0;
};

// bytes of `n` values of a ggml type laid out in blocks; 0 for types this library does not know the size of
size_t type_bytes(uint32_t type, uint64_t n) {
    switch (type) {
    case 0: return n * 4;                  // F32
    case 1: return n * 2;                  // F16
    case 8: return n / 32 * 34;            // Q8_0
    case 12: return n / 256 * 144;         // Q4_K
    case 14: return n / 256 * 210;         // Q6_K
    case 2: return n / 32 * 18;            // Q4_0
    case 3: return n / 32 * 20;            // Q4_1
    case 6: return n / 32 * 22;            // Q5_0
    case 7: return n / 32 * 24;            // Q5_1
    case 10: return n / 256 * 84;          // Q2_K
    case 11: return n / 256 * 110;         // Q3_K
    case 13: return n / 256 * 176;         // Q5_K
    case 30: return n * 2;                 // BF16
    default: return 0;
    }
}

// values per block of a ggml tensor type (1 for the plain float / integer types)
uint64_t type_block_values(uint32_t type) {
    if (type == 0 || type == 1 || type == 30) return 1;
    if (type == 8 || (type >= 2 && type <= 7)) return 32;
    return 256;
}

struct Reader {
    const uint8_t *p, *end;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (!ok || (size_t)(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || (uint64_t)(end - p) < n) {
            ok = false;
            return std::string();
        }
        std::string s((const char *)p, (size_t)n);
        p += n;
        return s;
    }
    void skip(uint64_t n) {
        if (!ok || (uint64_t)(end - p) < n) ok = false;
        else p += n;
    }
};

size_t scalar_size(uint32_t t) {
    switch (t) {
    case GV_U8: case GV_I8: case GV_BOOL: return 1;
    case GV_U16: case GV_I16: return 2;
    case GV_U32: case GV_I32: case GV_F32: return 4;
    case GV_U64: case GV_I64: case GV_F64: return 8;
    default: return 0;
    }
}

bool read_value(Reader &r, uint32_t type, MetaValue &out) {
    out.type = type;
    switch (type) {
    case GV_U8: out.u = r.get<uint8_t>(); break;
    case GV_I8: out.u = (uint64_t)(int64_t)r.get<int8_t>(); break;
    case GV_U16: out.u = r.get<uint16_t>(); break;
    case GV_I16: out.u = (uint64_t)(int64_t)r.get<int16_t>(); break;
    case GV_U32: out.u = r.get<uint32_t>(); break;
    case GV_I32: out.u = (uint64_t)(int64_t)r.get<int32_t>(); break;
    case GV_U64: out.u = r.get<uint64_t>(); break;
    case GV_I64: out.u = (uint64_t)r.get<int64_t>(); break;
    case GV_BOOL: out.u = r.get<uint8_t>() != 0; break;
    case GV_F32: out.f = r.get<float>(); break;
    case GV_F64: out.f = r.get<double>(); break;
    case GV_STRING: out.s = r.str(); break;
    case GV_ARRAY: {
        out.elem_type = r.get<uint32_t>();
        out.count = r.get<uint64_t>();
        if (out.elem_type == GV_STRING) {
            for (uint64_t i = 0; i < out.count && r.ok; ++i) r.skip(r.get<uint64_t>());
        } else if (out.elem_type == GV_ARRAY) {
            r.ok = false;  // nested arrays do not occur in model files
        } else {
            const size_t es = scalar_size(out.elem_type);
            uint64_t span = 0;
            if (es == 0 || __builtin_mul_overflow(out.count, (uint64_t)es, &span)) r.ok = false;
            else r.skip(span);
        }
        break;
    }
    default: r.ok = false;
    }
    return r.ok;
}

}  // namespace

struct mcu_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    size_t map_bytes = 0, data_start = 0;
    uint32_t version = 0;
    std::map<std::string, MetaValue> meta;
    std::vector<TensorEntry> tensors;
    std::map<std::string, size_t> by_name;
};

static int gguf_fail(int code, const char *msg) { return set_error(code, msg); }

extern "C" {

int mcu_gguf_open(const char *path, mcu_gguf_t **out) {
    if (out == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    if (path == nullptr) return gguf_fail(MCU_ERROR_INVALID_ARGUMENT, "gguf: null path");
    mcu_gguf *g = new (std::nothrow) mcu_gguf();
    if (g == nullptr) return gguf_fail(MCU_ERROR_OUT_OF_MEMORY, "gguf: allocation failed");
    auto bail = [&](int code, const char *msg) {
        mcu_gguf_close(g);
        return gguf_fail(code, msg);
    };
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: cannot open file");
    struct stat st;
    if (fstat(g->fd, &st) != 0 || st.st_size < 24) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: file too small");
    g->map_bytes = (size_t)st.st_size;
    void *m = mmap(nullptr, g->map_bytes, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) return bail(MCU_ERROR_OUT_OF_MEMORY, "gguf: mmap failed");
    g->map = (const uint8_t *)m;
    Reader r{g->map, g->map + g->map_bytes};
    if (r.get<uint32_t>() != 0x46554747u) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: bad magic");
    g->version = r.get<uint32_t>();
    if (g->version < 2 || g->version > 3) return bail(MCU_ERROR_NOT_IMPLEMENTED, "gguf: only versions 2 and 3 are read");
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: bad header");
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = r.str();
        const uint32_t type = r.get<uint32_t>();
        MetaValue v;
        if (!r.ok || !read_value(r, type, v)) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: malformed metadata");
        g->meta[key] = std::move(v);
    }
    g->tensors.resize((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        TensorEntry &t = g->tensors[(size_t)i];
        t.name = r.str();
        t.n_dims = r.get<uint32_t>();
        if (!r.ok || t.n_dims == 0 || t.n_dims > 4) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: malformed tensor directory");
        // The element count comes from the file: a product that wraps would pass the end-of-file check below with a
        // tiny byte size while row ranges computed from the dimensions point far outside the mapping.
        uint64_t n = 1;
        bool wrapped = false;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            t.dims[d] = r.get<uint64_t>();
            wrapped = wrapped || __builtin_mul_overflow(n, t.dims[d], &n);
        }
        t.type = r.get<uint32_t>();
        t.offset = r.get<uint64_t>();
        if (!r.ok) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: malformed tensor directory");
        if (wrapped || n > ((uint64_t)1 << 48))
            return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: tensor dimensions overflow");
        t.nbytes = type_bytes(t.type, n);
        if (t.nbytes != 0) {
            // rows must be whole blocks, or the per-row byte size used by the uploads would not tile the payload
            uint64_t rows = n / (t.dims[0] ? t.dims[0] : 1);
            if (t.dims[0] == 0 || type_bytes(t.type, t.dims[0]) * rows != t.nbytes ||
                t.dims[0] % type_block_values(t.type) != 0)
                return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: tensor rows are not whole blocks");
        }
        g->by_name[t.name] = (size_t)i;
    }
    uint64_t align = 32;
    auto it = g->meta.find("general.alignment");
    if (it != g->meta.end() && it->second.u > 0) align = it->second.u;
    if ((align & (align - 1)) != 0 || align > ((uint64_t)1 << 20))
        return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: general.alignment must be a power of two up to 1 MiB");
    const size_t at = (size_t)(r.p - g->map);
    g->data_start = (at + align - 1) / align * align;
    if (g->data_start > g->map_bytes) return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: header runs past the end of the file");
    for (const TensorEntry &t : g->tensors)
        if (t.nbytes != 0 && (g->data_start + t.offset > g->map_bytes || t.nbytes > g->map_bytes - g->data_start - t.offset))
            return bail(MCU_ERROR_INVALID_ARGUMENT, "gguf: tensor data runs past the end of the file");
    *out = g;
    return MCU_SUCCESS;
}

void mcu_gguf_close(mcu_gguf_t *g) {
    if (g == nullptr) return;
    if (g->map != nullptr) munmap((void *)g->map, g->map_bytes);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

size_t mcu_gguf_tensor_count(const mcu_gguf_t *g) { return g == nullptr ? 0 : g->tensors.size(); }

int mcu_gguf_find_tensor(const mcu_gguf_t *g, const char *name) {
    if (g == nullptr || name == nullptr) return -1;
    auto it = g->by_name.find(name);
    return it == g->by_name.end() ? -1 : (int)it->second;
}

int mcu_gguf_tensor_info(const mcu_gguf_t *g, size_t index, mcu_gguf_tensor_info_t *out) {
    if (g == nullptr || out == nullptr || index >= g->tensors.size()) return gguf_fail(MCU_ERROR_INVALID_ARGUMENT, "gguf: bad tensor index");
    const TensorEntry &t = g->tensors[index];
    out->name = t.name.c_str();
    out->ggml_type = t.type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
    out->nbytes = t.nbytes;
    out->data = t.nbytes != 0 ? g->map + g->data_start + t.offset : nullptr;
    out->kind = t.type == 12 ? MCU_KIND_Q4_K : t.type == 14 ? MCU_KIND_Q6_K : t.type == 8 ? MCU_KIND_Q8_0 : -1;
    return MCU_SUCCESS;
}

int mcu_gguf_meta_u64(const mcu_gguf_t *g, const char *key, uint64_t *out) {
    if (g == nullptr || key == nullptr || out == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return MCU_ERROR_INVALID_ARGUMENT;
    const MetaValue &v = it->second;
    if (v.type == GV_F32 || v.type == GV_F64 || v.type == GV_STRING) return MCU_ERROR_UNSUPPORTED_DTYPE;
    *out = v.type == GV_ARRAY ? v.count : v.u;  // arrays answer with their length (vocabulary size, ...)
    return MCU_SUCCESS;
}

int mcu_gguf_meta_f64(const mcu_gguf_t *g, const char *key, double *out) {
    if (g == nullptr || key == nullptr || out == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return MCU_ERROR_INVALID_ARGUMENT;
    const MetaValue &v = it->second;
    if (v.type == GV_F32 || v.type == GV_F64) *out = v.f;
    else if (v.type == GV_STRING || v.type == GV_ARRAY) return MCU_ERROR_UNSUPPORTED_DTYPE;
    else *out = (double)(int64_t)v.u;
    return MCU_SUCCESS;
}

int mcu_gguf_meta_str(const mcu_gguf_t *g, const char *key, const char **out, size_t *out_len) {
    if (g == nullptr || key == nullptr || out == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return MCU_ERROR_INVALID_ARGUMENT;
    if (it->second.type != GV_STRING) return MCU_ERROR_UNSUPPORTED_DTYPE;
    *out = it->second.s.c_str();
    if (out_len != nullptr) *out_len = it->second.s.size();
    return MCU_SUCCESS;
}

// Rows [row_lo, row_hi) and, of every row, the bytes of values [k_lo, k_hi) -> dst_dev as a packed
// [row_hi - row_lo][bytes of k_hi - k_lo values] matrix.  Whole rows are one linear copy.
int mcu_gguf_upload(mcu_context_t *ctx, const mcu_gguf_t *g, size_t index, size_t row_lo, size_t row_hi, size_t k_lo,
                    size_t k_hi, void *dst_dev) {
    if (ctx == nullptr) return gguf_fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
    if (g == nullptr || index >= g->tensors.size() || dst_dev == nullptr) return gguf_fail(MCU_ERROR_INVALID_ARGUMENT, "gguf: bad upload arguments");
    const TensorEntry &t = g->tensors[index];
    if (t.nbytes == 0) return gguf_fail(MCU_ERROR_NOT_IMPLEMENTED, "gguf: tensor type has no known layout");
    const uint64_t K = t.dims[0];
    uint64_t rows = 1;
    for (uint32_t d = 1; d < t.n_dims; ++d) rows *= t.dims[d];
    if (row_hi > rows || row_lo > row_hi || k_hi > K || k_lo > k_hi) return gguf_fail(MCU_ERROR_DIMENSION_MISMATCH, "gguf: shard outside the tensor");
    const size_t row_bytes = type_bytes(t.type, K), lo_bytes = type_bytes(t.type, k_lo), hi_bytes = type_bytes(t.type, k_hi);
    // a K shard must fall on block boundaries: the byte offsets of k_lo and k_hi must describe them exactly
    const uint64_t bv = type_block_values(t.type);
    if (k_lo % bv != 0 || k_hi % bv != 0) return gguf_fail(MCU_ERROR_DIMENSION_MISMATCH, "gguf: K shard must be whole blocks");
    if (row_hi == row_lo || k_hi == k_lo) return MCU_SUCCESS;
    cudaError_t e = cudaSetDevice(context_device(ctx));
    const cudaStream_t s = (cudaStream_t)mcu_context_get_stream(ctx);
    const uint8_t *src = g->map + g->data_start + t.offset + row_lo * row_bytes + lo_bytes;
    const size_t width = hi_bytes - lo_bytes, n = row_hi - row_lo;
    if (e == cudaSuccess) {
        if (width == row_bytes) e = cudaMemcpyAsync(dst_dev, src, n * row_bytes, cudaMemcpyHostToDevice, s);
        else e = cudaMemcpy2DAsync(dst_dev, width, src, row_bytes, width, n, cudaMemcpyHostToDevice, s);
    }
    if (e != cudaSuccess) return gguf_fail(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
    return MCU_SUCCESS;
}

}  // extern "C"
