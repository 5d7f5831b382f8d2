// GGUF files straight to registered device weights: the file is memory-mapped, its header is parsed the way
// GgufLoader.LoadMeta does (SharpMind.Model/Format/GgufLoader.cs:124-176: magic, version, tensor and key/value
// counts, typed key/value pairs, tensor infos, data section aligned to general.alignment), and a tensor's bytes go
// from the mapping to the GPU in one copy (smc_weight_register), with the byte count checked against
// GetRawTensorByteCount as LoadSingleTensor does (GgufLoader.cs:512-535).  Host code only; no kernel lives here.
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "smc_common.cuh"

namespace {

struct GgufKv {
    std::string key;
    uint32_t type = 0;      // GGUF value type; arrays keep their element type in `elem`
    uint32_t elem = 0;
    uint64_t count = 0;     // arrays: element count
    uint64_t u = 0;         // integers / bool
    double f = 0.0;         // floats
    std::string s;          // strings
};

struct GgufTensor {
    std::string name;
    uint32_t dtype = 0;
    int n_dims = 0;
    int64_t dims[4] = {1, 1, 1, 1};
    uint64_t offset = 0;    // from the start of the data section
    int64_t bytes = -1;     // -1: a format this library has no byte count for
};

}  // namespace

struct smc_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t data_offset = 0;
    std::vector<GgufKv> kv;
    std::vector<GgufTensor> tensors;
};

namespace {

struct Cursor {
    const uint8_t *p, *end;
    bool ok = true;
    template <class T>
    T get()
    {
        T v{};
        if (!ok || (size_t)(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str()
    {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (uint64_t)(end - p)) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char *>(p), (size_t)n);
        p += n;
        return s;
    }
    void skip(uint64_t n)
    {
        if (!ok || n > (uint64_t)(end - p)) ok = false;
        else p += n;
    }
};

// size in bytes of a scalar GGUF value type (0 for strings and arrays)
size_t scalar_size(uint32_t t)
{
    switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
    }
}

bool read_scalar(Cursor &c, uint32_t t, GgufKv &kv)
{
    switch (t) {
    case 0: kv.u = c.get<uint8_t>(); break;
    case 1: kv.u = (uint64_t)(int64_t)c.get<int8_t>(); break;
    case 2: kv.u = c.get<uint16_t>(); break;
    case 3: kv.u = (uint64_t)(int64_t)c.get<int16_t>(); break;
    case 4: kv.u = c.get<uint32_t>(); break;
    case 5: kv.u = (uint64_t)(int64_t)c.get<int32_t>(); break;
    case 6: kv.f = c.get<float>(); break;
    case 7: kv.u = c.get<uint8_t>() ? 1 : 0; break;
    case 10: kv.u = c.get<uint64_t>(); break;
    case 11: kv.u = (uint64_t)c.get<int64_t>(); break;
    case 12: kv.f = c.get<double>(); break;
    default: return false;
    }
    if (t != 6 && t != 12) kv.f = (double)(int64_t)kv.u;
    else kv.u = (uint64_t)(int64_t)kv.f;
    return c.ok;
}

int64_t tensor_bytes(uint32_t dtype, const int64_t *dims, int n_dims)
{
    int64_t count = 1;
    for (int i = 0; i < n_dims; ++i) count *= dims[i];
    const int64_t K = dims[0], rows = K ? count / K : 0;
    switch (dtype) {
    case 0: return count * 4;  // F32
    case 1: return count * 2;  // F16
    case SMC_Q8_0: case SMC_Q4_K: case SMC_Q6_K: return smc_raw_tensor_bytes((int)dtype, rows, K);
    default: return -1;
    }
}

const GgufKv *find_kv(const smc_gguf *g, const char *key)
{
    for (const GgufKv &kv : g->kv)
        if (kv.key == key) return &kv;
    return nullptr;
}

void close_file(smc_gguf *g)
{
    if (g->map) munmap(const_cast<uint8_t *>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

}  // namespace

extern "C" {

int smc_gguf_open(smc_ctx *ctx, const char *path, smc_gguf **out)
{
    if (!path || !out) return smc_fail(ctx, SMC_E_INVALID, "gguf_open: bad arguments");  // ctx may be null: parsing needs no device
    *out = nullptr;
    smc_gguf *g = new smc_gguf();
    g->fd = open(path, O_RDONLY);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        const int e = errno;
        close_file(g);
        return smc_fail(ctx, SMC_E_INVALID, "gguf_open: cannot open '%s': %s", path, strerror(e));
    }
    g->size = (size_t)st.st_size;
    void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        const int e = errno;
        close_file(g);
        return smc_fail(ctx, SMC_E_INVALID, "gguf_open: cannot map '%s': %s", path, strerror(e));
    }
    g->map = static_cast<const uint8_t *>(m);
    Cursor c{g->map, g->map + g->size};
    const uint32_t magic = c.get<uint32_t>();
    if (magic != 0x46554747u) {  // "GGUF"
        close_file(g);
        return smc_fail(ctx, SMC_E_INVALID, "Not GGUF: %08X", magic);
    }
    g->version = c.get<uint32_t>();
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
        close_file(g);
        return smc_fail(ctx, SMC_E_INVALID, "gguf_open: implausible header in '%s'", path);
    }
    for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
        GgufKv kv;
        kv.key = c.str();
        kv.type = c.get<uint32_t>();
        if (kv.type == 8) {
            kv.s = c.str();
        } else if (kv.type == 9) {
            kv.elem = c.get<uint32_t>();
            kv.count = c.get<uint64_t>();
            if (kv.elem == 8) {
                for (uint64_t j = 0; j < kv.count && c.ok; ++j) c.skip(c.get<uint64_t>());  // string arrays (the vocabulary) are passed over
            } else if (scalar_size(kv.elem)) {
                c.skip(kv.count * scalar_size(kv.elem));
            } else {
                c.ok = false;
            }
        } else if (!read_scalar(c, kv.type, kv)) {
            c.ok = false;
        }
        if (c.ok) g->kv.push_back(std::move(kv));
    }
    for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
        GgufTensor t;
        t.name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd == 0 || nd > 4) {
            c.ok = false;
            break;
        }
        t.n_dims = (int)nd;
        for (uint32_t j = 0; j < nd; ++j) t.dims[j] = (int64_t)c.get<uint64_t>();
        t.dtype = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        t.bytes = tensor_bytes(t.dtype, t.dims, t.n_dims);
        if (c.ok) g->tensors.push_back(std::move(t));
    }
    if (!c.ok) {
        close_file(g);
        return smc_fail(ctx, SMC_E_INVALID, "gguf_open: '%s' ends inside its header", path);
    }
    uint64_t align = 32;
    if (const GgufKv *a = find_kv(g, "general.alignment"))
        if (a->u) align = a->u;
    const uint64_t pos = (uint64_t)(c.p - g->map);
    g->data_offset = (pos + align - 1) / align * align;
    for (const GgufTensor &t : g->tensors)
        if (t.bytes >= 0 && g->data_offset + t.offset + (uint64_t)t.bytes > g->size) {
            std::string name = t.name;
            close_file(g);
            return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "gguf_open: tensor '%s' runs past the end of the file", name.c_str());
        }
    *out = g;
    return SMC_OK;
}

int smc_gguf_close(smc_ctx *ctx, smc_gguf *g)
{
    if (!g) return smc_fail(ctx, SMC_E_INVALID, "gguf_close: bad arguments");
    close_file(g);
    return SMC_OK;
}

int smc_gguf_tensor_count(const smc_gguf *g) { return g ? (int)g->tensors.size() : 0; }

int smc_gguf_find(const smc_gguf *g, const char *name)
{
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); ++i)
        if (g->tensors[i].name == name) return (int)i;
    return -1;
}

int smc_gguf_tensor_info(const smc_gguf *g, int index, const char **name, int *dtype, int *n_dims, int64_t *dims4,
                         int64_t *bytes)
{
    if (!g || index < 0 || index >= (int)g->tensors.size()) return SMC_E_RANGE;
    const GgufTensor &t = g->tensors[index];
    if (name) *name = t.name.c_str();
    if (dtype) *dtype = (int)t.dtype;
    if (n_dims) *n_dims = t.n_dims;
    if (dims4) memcpy(dims4, t.dims, sizeof(t.dims));
    if (bytes) *bytes = t.bytes;
    return SMC_OK;
}

int smc_gguf_meta_int(const smc_gguf *g, const char *key, int64_t *value)
{
    const GgufKv *kv = g && key ? find_kv(g, key) : nullptr;
    if (!kv || kv->type == 8 || kv->type == 9 || !value) return SMC_E_NOT_REGISTERED;
    *value = (int64_t)kv->u;
    return SMC_OK;
}

int smc_gguf_meta_float(const smc_gguf *g, const char *key, double *value)
{
    const GgufKv *kv = g && key ? find_kv(g, key) : nullptr;
    if (!kv || kv->type == 8 || kv->type == 9 || !value) return SMC_E_NOT_REGISTERED;
    *value = kv->f;
    return SMC_OK;
}

const char *smc_gguf_meta_string(const smc_gguf *g, const char *key)
{
    const GgufKv *kv = g && key ? find_kv(g, key) : nullptr;
    return kv && kv->type == 8 ? kv->s.c_str() : nullptr;
}

int smc_gguf_register(smc_ctx *ctx, const smc_gguf *g, int index, int flags, smc_weight **out)
{
    if (!ctx || !g || !out || index < 0 || index >= (int)g->tensors.size()) return smc_fail(ctx, SMC_E_INVALID, "gguf_register: bad arguments");
    const GgufTensor &t = g->tensors[index];
    if (t.dtype != SMC_Q8_0 && t.dtype != SMC_Q4_K && t.dtype != SMC_Q6_K)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "gguf_register: tensor '%s' has dtype %u; Q8_0 (8), Q4_K (12) and Q6_K (14) have kernels", t.name.c_str(), t.dtype);
    if (t.n_dims != 2 || t.dims[0] > INT32_MAX || t.dims[1] > INT32_MAX)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "gguf_register: tensor '%s' is not a matrix", t.name.c_str());
    // GGUF lists the innermost dimension first: dims[0] = inFeatures (K), dims[1] = outFeatures (N)
    return smc_weight_register(ctx, g->map + g->data_offset + t.offset, (size_t)t.bytes, (int)t.dtype, (int)t.dims[1], (int)t.dims[0],
                               flags, out);
}

int smc_gguf_read_f32(smc_ctx *ctx, const smc_gguf *g, int index, float *d_dst, int64_t count)
{
    if (!ctx || !g || !d_dst || index < 0 || index >= (int)g->tensors.size()) return smc_fail(ctx, SMC_E_INVALID, "gguf_read_f32: bad arguments");
    const GgufTensor &t = g->tensors[index];
    int64_t n = 1;
    for (int i = 0; i < t.n_dims; ++i) n *= t.dims[i];
    if (n != count) return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "gguf_read_f32: tensor '%s' holds %lld values, caller expects %lld", t.name.c_str(), (long long)n, (long long)count);
    const uint8_t *src = g->map + g->data_offset + t.offset;
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    if (t.dtype == 0) {
        SMC_CUDA(ctx, cudaMemcpy(d_dst, src, (size_t)n * 4, cudaMemcpyHostToDevice));
        return SMC_OK;
    }
    if (t.dtype == 1) {  // F16 -> F32 on the host (norm vectors and biases: a few thousand values)
        std::vector<float> tmp((size_t)n);
        for (int64_t i = 0; i < n; ++i) {
            uint16_t h;
            memcpy(&h, src + 2 * i, 2);
            tmp[(size_t)i] = __half2float(__ushort_as_half(h));
        }
        SMC_CUDA(ctx, cudaMemcpy(d_dst, tmp.data(), (size_t)n * 4, cudaMemcpyHostToDevice));
        return SMC_OK;
    }
    return smc_fail(ctx, SMC_E_UNSUPPORTED, "gguf_read_f32: tensor '%s' has dtype %u (F32 and F16 are read)", t.name.c_str(), t.dtype);
}

}  // extern "C"
