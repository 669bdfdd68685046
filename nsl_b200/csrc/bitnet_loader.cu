// load_bitnet_b158_safetensors (crates/nsl-codegen/src/bitnet/loader.rs:200-220) with the quantiser on
// the GPU: read a safetensors file, keep the tensors whose names end in one of the seven BitLinear
// projection suffixes (loader.rs:100-111), and turn each into packed ternary bytes plus its absmean scale
// (quantize_float_to_ternary, loader.rs:126-193 = nslq_ternary_quantize_pack).  What the reference
// returns as LoadedTernaryWeight {name, packed_bytes, shape, scale} (loader.rs:47-56) is an entry of the
// set here, with the packed bytes already in device memory, ready for nslq_bitlinear_create.
//
// The container (safetensors 0.4): u64 little-endian header length n, n bytes of JSON
//   { "<name>": {"dtype": "F32", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {..} }
// and the data buffer, to which the offsets are relative.  The reader below parses exactly that much
// JSON (objects, arrays, strings with escapes, non-negative integers) and checks every tensor's byte
// range against the file and against shape x element size before it touches the bytes.
//
// Errors follow the reference's LoaderError: a file that cannot be read or is not a safetensors
// container -> NSLQ_ERR_IO (Io / Safetensors); element count not a multiple of four -> NSLQ_ERR_SHAPE
// (AlignmentError); a projection stored as anything but F32 / F16 / BF16 -> NSLQ_ERR_UNSUPPORTED
// (UnsupportedDtype).  Any error leaves no set behind.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "common.cuh"

namespace nslq {

int ternary_quantize_pack_dispatch(const void *, int, int64_t, uint8_t *, float *, cudaStream_t);

namespace {

struct TensorInfo {
    std::string name, dtype;
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;
    bool has_dtype = false, has_shape = false, has_offsets = false;
};

// A reader for the JSON subset of a safetensors header.
struct Json {
    const char *p, *e;
    std::string err;
    explicit Json(const char *b, size_t n) : p(b), e(b + n) {}
    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char *what) { if (err.empty()) err = what; return false; }
    bool lit(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
    bool string(std::string &out)
    {
        ws();
        if (p >= e || *p != '"') return fail("expected a string");
        ++p;
        out.clear();
        while (p < e && *p != '"') {
            if (*p == '\\') {
                if (++p >= e) return fail("unterminated escape");
                switch (*p) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    if (e - p < 5) return fail("short \\u escape");
                    unsigned v = 0;
                    for (int i = 1; i <= 4; ++i) {
                        const char c = p[i];
                        v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 256);
                        if (v >= 0x10000) return fail("bad \\u escape");
                    }
                    p += 4;
                    if (v < 0x80) out += (char)v;                     // UTF-8 (surrogate pairs are kept as two code units)
                    else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 0x3F)); }
                    else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3F)); out += (char)(0x80 | (v & 0x3F)); }
                    break;
                }
                default: return fail("unknown escape");
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= e) return fail("unterminated string");
        ++p;
        return true;
    }
    bool uint(uint64_t &v)
    {
        ws();
        if (p >= e || *p < '0' || *p > '9') return fail("expected a non-negative integer");
        v = 0;
        while (p < e && *p >= '0' && *p <= '9') {
            if (v > (UINT64_MAX - 9) / 10) return fail("integer overflow");
            v = v * 10 + (uint64_t)(*p++ - '0');
        }
        return true;
    }
    bool uint_array(std::vector<uint64_t> &out)
    {
        out.clear();
        if (!lit('[')) return fail("expected an array");
        if (lit(']')) return true;
        do {
            uint64_t v;
            if (!uint(v)) return false;
            out.push_back(v);
        } while (lit(','));
        return lit(']') || fail("unterminated array");
    }
    // any value, skipped (the __metadata__ object and keys this reader does not know)
    bool skip(int depth = 0)
    {
        if (depth > 32) return fail("nesting too deep");
        ws();
        if (p >= e) return fail("unexpected end");
        if (*p == '"') { std::string s; return string(s); }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool obj = *p == '{';
            ++p;
            if (lit(close)) return true;
            do {
                if (obj) { std::string k; if (!string(k) || !lit(':')) return fail("bad object"); }
                if (!skip(depth + 1)) return false;
            } while (lit(','));
            return lit(close) || fail("unterminated container");
        }
        const char *s = p;                                            // number, true, false, null
        while (p < e && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;
        return p > s || fail("empty value");
    }
    bool tensor(TensorInfo &t)
    {
        if (!lit('{')) return fail("a tensor entry must be an object");
        if (lit('}')) return true;
        do {
            std::string k;
            if (!string(k) || !lit(':')) return fail("bad tensor entry");
            std::vector<uint64_t> a;
            if (k == "dtype") { if (!string(t.dtype)) return false; t.has_dtype = true; }
            else if (k == "shape") { if (!uint_array(a)) return false; t.shape.assign(a.begin(), a.end()); t.has_shape = true; }
            else if (k == "data_offsets") {
                if (!uint_array(a)) return false;
                if (a.size() != 2) return fail("data_offsets must have two entries");
                t.begin = a[0]; t.end = a[1]; t.has_offsets = true;
            } else if (!skip()) return false;
        } while (lit(','));
        return lit('}') || fail("unterminated tensor entry");
    }
    bool header(std::vector<TensorInfo> &out)
    {
        if (!lit('{')) return fail("the header must be an object");
        if (!lit('}')) {
            do {
                TensorInfo t;
                if (!string(t.name) || !lit(':')) return fail("bad header entry");
                if (t.name == "__metadata__") { if (!skip()) return false; continue; }
                if (!tensor(t)) return false;
                if (!t.has_dtype || !t.has_shape || !t.has_offsets) return fail("tensor entry without dtype, shape or data_offsets");
                out.push_back(std::move(t));
            } while (lit(','));
            if (!lit('}')) return fail("unterminated header");
        }
        ws();
        return p == e || fail("bytes after the header object");
    }
};

bool is_bitlinear_weight(const std::string &name)
{
    static const char *suffixes[] = {".self_attn.q_proj.weight", ".self_attn.k_proj.weight", ".self_attn.v_proj.weight",
                                     ".self_attn.o_proj.weight", ".mlp.gate_proj.weight",    ".mlp.up_proj.weight",
                                     ".mlp.down_proj.weight"};
    for (const char *s : suffixes) {
        const size_t n = strlen(s);
        if (name.size() >= n && name.compare(name.size() - n, n, s) == 0) return true;
    }
    return false;
}

}  // namespace
}  // namespace nslq

struct nslq_ternary_set {
    struct Entry {
        std::string name;
        std::vector<int64_t> shape;
        uint8_t *packed = nullptr;          // device
        int64_t packed_bytes = 0;
        float scale = 0.0f;
    };
    std::vector<Entry> entries;
    int device = 0;
};

using namespace nslq;

static void free_set(nslq_ternary_set *s)
{
    if (!s) return;
    for (auto &en : s->entries)
        if (en.packed) cudaFree(en.packed);
    delete s;
}

extern "C" {

int nslq_bitnet_load_safetensors(const char *path, void *stream, nslq_ternary_set_t **out)
{
    if (!path || !out) return fail(NSLQ_ERR_ARG, "nslq_bitnet_load_safetensors: null argument");
    *out = nullptr;
    FILE *f = fopen(path, "rb");
    if (!f) return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: io: cannot open %s", path);
    struct Closer { FILE *f; ~Closer() { fclose(f); } } closer{f};
    if (fseek(f, 0, SEEK_END) != 0) return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: io: cannot seek in %s", path);
    const int64_t file_size = ftell(f);
    rewind(f);
    uint8_t len8[8];
    if (file_size < 8 || fread(len8, 1, 8, f) != 8) return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: safetensors: %s is shorter than a header length", path);
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | len8[i];
    if (n > 100000000ull || (int64_t)n > file_size - 8)       // the safetensors crate's own header limit is 100 MB
        return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: safetensors: header length %llu does not fit the file (%lld bytes)", (unsigned long long)n, (long long)file_size);
    std::string header(n, '\0');
    if (n && fread(&header[0], 1, n, f) != n) return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: io: short read of the header of %s", path);
    std::vector<TensorInfo> tensors;
    Json js(header.data(), header.size());
    if (!js.header(tensors)) return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: safetensors: invalid header: %s", js.err.c_str());
    const uint64_t data0 = 8 + n, data_size = (uint64_t)file_size - data0;

    // Select and check before any byte is moved.  (The reference walks a hash map, so its order is
    // unspecified; entries here come in the order of their bytes in the file.)
    std::vector<const TensorInfo *> picked;
    size_t largest = 0;
    for (const TensorInfo &t : tensors) {
        if (!is_bitlinear_weight(t.name)) continue;
        int dt, es;
        if (t.dtype == "F32") { dt = NSLQ_DTYPE_F32; es = 4; }
        else if (t.dtype == "F16") { dt = NSLQ_DTYPE_FP16; es = 2; }
        else if (t.dtype == "BF16") { dt = NSLQ_DTYPE_BF16; es = 2; }
        else return fail(NSLQ_ERR_UNSUPPORTED, "nslq_bitnet_load_safetensors: tensor %s has unsupported dtype %s (expected F32, F16 or BF16)", t.name.c_str(), t.dtype.c_str());
        (void)dt;
        uint64_t numel = 1;
        for (int64_t d : t.shape) {
            if (d != 0 && numel > (uint64_t)INT64_MAX / (uint64_t)d) return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: safetensors: shape of %s overflows", t.name.c_str());
            numel *= (uint64_t)d;
        }
        if (t.begin > t.end || t.end > data_size || t.end - t.begin != numel * (uint64_t)es)
            return fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: safetensors: byte range [%llu, %llu) of %s does not match its shape or the file",
                        (unsigned long long)t.begin, (unsigned long long)t.end, t.name.c_str());
        if (numel % 4 != 0)
            return fail(NSLQ_ERR_SHAPE, "nslq_bitnet_load_safetensors: tensor %s has %llu elements, not a multiple of 4 (cannot pack)", t.name.c_str(), (unsigned long long)numel);
        if (numel == 0) return fail(NSLQ_ERR_SHAPE, "nslq_bitnet_load_safetensors: tensor %s is empty", t.name.c_str());
        largest = std::max(largest, (size_t)(t.end - t.begin));
        picked.push_back(&t);
    }
    std::sort(picked.begin(), picked.end(), [](const TensorInfo *a, const TensorInfo *b) { return a->begin < b->begin; });

    nslq_ternary_set *set = new nslq_ternary_set();
    cudaGetDevice(&set->device);
    if (picked.empty()) { *out = set; return NSLQ_OK; }
    cudaStream_t st = (cudaStream_t)stream;
    void *host = nullptr, *dev = nullptr;
    float *dscale = nullptr;
    int rc = NSLQ_OK;
    if (cudaHostAlloc(&host, largest, cudaHostAllocDefault) != cudaSuccess || cudaMalloc(&dev, largest) != cudaSuccess ||
        cudaMalloc(&dscale, sizeof(float)) != cudaSuccess)
        rc = fail(NSLQ_ERR_CUDA, "nslq_bitnet_load_safetensors: staging buffers of %zu bytes: %s", largest, cudaGetErrorString(cudaGetLastError()));
    for (size_t i = 0; rc == NSLQ_OK && i < picked.size(); ++i) {
        const TensorInfo &t = *picked[i];
        const size_t bytes = (size_t)(t.end - t.begin);
        const int dt = t.dtype == "F32" ? NSLQ_DTYPE_F32 : (t.dtype == "F16" ? NSLQ_DTYPE_FP16 : NSLQ_DTYPE_BF16);
        const int64_t numel = (int64_t)(bytes / (dt == NSLQ_DTYPE_F32 ? 4 : 2));
        if (fseek(f, (long)(data0 + t.begin), SEEK_SET) != 0 || fread(host, 1, bytes, f) != bytes) {
            rc = fail(NSLQ_ERR_IO, "nslq_bitnet_load_safetensors: io: short read of tensor %s", t.name.c_str());
            break;
        }
        nslq_ternary_set::Entry en;
        en.name = t.name;
        en.shape = t.shape;
        en.packed_bytes = numel / 4;
        if (cudaMalloc(&en.packed, (size_t)en.packed_bytes) != cudaSuccess) {
            rc = fail(NSLQ_ERR_CUDA, "nslq_bitnet_load_safetensors: %lld bytes for %s: %s", (long long)en.packed_bytes, t.name.c_str(), cudaGetErrorString(cudaGetLastError()));
            break;
        }
        set->entries.push_back(en);                                      // owned by the set from here on
        if (cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) {
            rc = fail(NSLQ_ERR_CUDA, "nslq_bitnet_load_safetensors: copy of %s: %s", t.name.c_str(), cudaGetErrorString(cudaGetLastError()));
            break;
        }
        rc = ternary_quantize_pack_dispatch(dev, dt, numel, set->entries.back().packed, dscale, st);
        if (rc) break;
        if (cudaMemcpyAsync(&set->entries.back().scale, dscale, sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess)                   // the staging buffers are reused by the next tensor
            rc = fail(NSLQ_ERR_CUDA, "nslq_bitnet_load_safetensors: quantising %s: %s", t.name.c_str(), cudaGetErrorString(cudaGetLastError()));
    }
    if (host) cudaFreeHost(host);
    if (dev) cudaFree(dev);
    if (dscale) cudaFree(dscale);
    if (rc != NSLQ_OK) { free_set(set); return rc; }
    *out = set;
    return NSLQ_OK;
}

int64_t nslq_ternary_set_size(const nslq_ternary_set_t *set) { return set ? (int64_t)set->entries.size() : 0; }

int nslq_ternary_set_entry(const nslq_ternary_set_t *set, int64_t i, const char **name, const uint8_t **packed, int64_t *packed_bytes,
                           const int64_t **shape, int *ndim, float *scale)
{
    if (!set || i < 0 || i >= (int64_t)set->entries.size()) return fail(NSLQ_ERR_ARG, "nslq_ternary_set_entry: index %lld", (long long)i);
    const auto &en = set->entries[(size_t)i];
    if (name) *name = en.name.c_str();
    if (packed) *packed = en.packed;
    if (packed_bytes) *packed_bytes = en.packed_bytes;
    if (shape) *shape = en.shape.data();
    if (ndim) *ndim = (int)en.shape.size();
    if (scale) *scale = en.scale;
    return NSLQ_OK;
}

void nslq_ternary_set_destroy(nslq_ternary_set_t *set) { free_set(set); }

}  // extern "C"
