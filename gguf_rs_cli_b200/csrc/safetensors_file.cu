// Reader of the safetensors container and uploader of its tensors: 8 bytes of little-endian header
// length, a JSON header {name: {dtype, shape, data_offsets}}, then the bytes.  The file is mapped and
// every entry checked once (known dtype, offsets inside the file, byte count = elements x size); tensors
// are found by index after the host has read the table, and go to the device through two pinned staging
// buffers, converted there when the stored dtype is not the one they are kept in.
//
// It stands where the reference parses GGUF by hand and maps the whole file
// (src/gguf/reader.rs:32-58, src/tensor/storage.rs:15-20, views in src/tensor/dequant.rs:245-268).
#include <cuda_fp16.h>
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"

namespace {

enum StType { ST_F64, ST_F32, ST_F16, ST_BF16, ST_I64, ST_I32, ST_I16, ST_I8, ST_U8, ST_BOOL, ST_TYPES };
const char* const ST_NAMES[ST_TYPES] = {"F64", "F32", "F16", "BF16", "I64", "I32", "I16", "I8", "U8", "BOOL"};
const int ST_SIZES[ST_TYPES] = {8, 4, 2, 2, 8, 4, 2, 1, 1, 1};
enum StKeep { KEEP_F32 = 0, KEEP_BF16 = 1, KEEP_I32 = 2 };

struct StEntry {
    std::string name;
    int type = -1;
    std::vector<long long> shape;
    long long begin = 0, end = -1;
};

struct StFile {
    std::string path;
    int fd = -1;
    size_t size = 0, base = 0;
    const uint8_t* map = nullptr;
    std::vector<StEntry> entries;
    std::vector<std::pair<std::string, std::string>> metadata;
};

// ---------------------------------------------------------------- the header's JSON
struct Json {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char* what) { if (err.empty()) err = what; return false; }
    bool lit(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }

    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out += char(cp);
        else if (cp < 0x800) { out += char(0xC0 | (cp >> 6)); out += char(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += char(0xE0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
        else { out += char(0xF0 | (cp >> 18)); out += char(0x80 | ((cp >> 12) & 0x3F)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
    }
    bool hex4(unsigned& v) {
        if (end - p < 4) return fail("a \\u escape is cut short");
        v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= unsigned(c - '0');
            else if (c >= 'a' && c <= 'f') v |= unsigned(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= unsigned(c - 'A' + 10);
            else return fail("a \\u escape has a digit that is not hexadecimal");
        }
        return true;
    }
    bool string(std::string& out) {
        ws();
        if (p >= end || *p != '"') return fail("a string was expected");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            char c = *p++;
            if (c != '\\') { out += c; continue; }
            if (p >= end) break;
            c = *p++;
            switch (c) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp;
                    if (!hex4(cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned lo;
                        if (!hex4(lo)) return false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: return fail("an unknown escape in a string");
            }
        }
        if (p >= end) return fail("a string does not end");
        ++p;
        return true;
    }
    bool integer(long long& v) {
        ws();
        const char* s = p;
        bool neg = false;
        if (p < end && *p == '-') { neg = true; ++p; }
        if (p >= end || *p < '0' || *p > '9') { p = s; return fail("an integer was expected"); }
        unsigned long long u = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (u > (0x7FFFFFFFFFFFFFFFull - 9) / 10) return fail("an integer is too large");
            u = u * 10 + unsigned(*p++ - '0');
        }
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail("an integer was expected, found a fraction");
        v = neg ? -(long long)u : (long long)u;
        return true;
    }
    bool int_list(std::vector<long long>& out) {
        out.clear();
        if (!lit('[')) return fail("a list was expected");
        if (lit(']')) return true;
        do {
            long long v;
            if (!integer(v)) return false;
            out.push_back(v);
        } while (lit(','));
        return lit(']') || fail("a list does not end");
    }
    // any value, thrown away (keys this reader does not know)
    bool skip(int depth = 0) {
        if (depth > 64) return fail("the header nests too deep");
        ws();
        if (p >= end) return fail("the header ends in the middle of a value");
        if (*p == '"') { std::string s; return string(s); }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool object = *p == '{';
            ++p;
            if (lit(close)) return true;
            do {
                if (object) {
                    std::string k;
                    if (!string(k) || !lit(':')) return fail("an object's key is malformed");
                }
                if (!skip(depth + 1)) return false;
            } while (lit(','));
            return lit(close) || fail("an object or list does not end");
        }
        const char* s = p;
        while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;
        return p > s || fail("a value was expected");
    }
};

int parse_header(StFile& f, const char* text, size_t len) {
    Json j{text, text + len, {}};
    const char* path = f.path.c_str();
    if (!j.lit('{')) return gb_fail("%s: header is not JSON (it is not an object)", path);
    if (!j.lit('}')) {
        do {
            std::string name;
            if (!j.string(name) || !j.lit(':')) return gb_fail("%s: header is not JSON (%s)", path, j.err.empty() ? "a key is malformed" : j.err.c_str());
            if (name == "__metadata__") {
                if (!j.lit('{')) return gb_fail("%s: header is not JSON (__metadata__ is not an object)", path);
                if (!j.lit('}')) {
                    do {
                        std::string k, v;
                        if (!j.string(k) || !j.lit(':')) return gb_fail("%s: header is not JSON (%s)", path, j.err.c_str());
                        j.ws();
                        if (j.p < j.end && *j.p == '"') {
                            if (!j.string(v)) return gb_fail("%s: header is not JSON (%s)", path, j.err.c_str());
                            f.metadata.emplace_back(k, v);
                        } else if (!j.skip()) {
                            return gb_fail("%s: header is not JSON (%s)", path, j.err.c_str());
                        }
                    } while (j.lit(','));
                    if (!j.lit('}')) return gb_fail("%s: header is not JSON (__metadata__ does not end)", path);
                }
                continue;
            }
            for (const StEntry& e : f.entries)
                if (e.name == name) return gb_fail("%s: tensor '%s' is listed twice in the header", path, name.c_str());
            StEntry e;
            e.name = name;
            std::string dtype;
            bool has_shape = false;
            if (!j.lit('{')) return gb_fail("%s: header is not JSON (the entry of '%s' is not an object)", path, name.c_str());
            if (!j.lit('}')) {
                do {
                    std::string k;
                    if (!j.string(k) || !j.lit(':')) return gb_fail("%s: header is not JSON (%s)", path, j.err.c_str());
                    bool ok = true;
                    if (k == "dtype") ok = j.string(dtype);
                    else if (k == "shape") { ok = j.int_list(e.shape); has_shape = ok; }
                    else if (k == "data_offsets") {
                        std::vector<long long> off;
                        ok = j.int_list(off);
                        if (ok && off.size() == 2) { e.begin = off[0]; e.end = off[1]; }
                    } else ok = j.skip();
                    if (!ok) return gb_fail("%s: header is not JSON (tensor '%s': %s)", path, name.c_str(), j.err.c_str());
                } while (j.lit(','));
                if (!j.lit('}')) return gb_fail("%s: header is not JSON (the entry of '%s' does not end)", path, name.c_str());
            }
            for (int t = 0; t < ST_TYPES; ++t)
                if (dtype == ST_NAMES[t]) e.type = t;
            if (e.type < 0) return gb_fail("%s: tensor '%s' has unsupported dtype '%s'", path, name.c_str(), dtype.c_str());
            long long n = 1;
            bool bad = !has_shape && e.end != e.begin;
            for (long long s : e.shape) {
                if (s < 0 || (s > 0 && n > (1ll << 56) / s)) { bad = true; break; }
                n *= s;
            }
            const long long data_bytes = (long long)(f.size - f.base);
            if (bad || e.begin < 0 || e.end < e.begin || e.end > data_bytes || e.end - e.begin != n * ST_SIZES[e.type]) {
                std::string shape = "[";
                for (size_t i = 0; i < e.shape.size(); ++i) shape += (i ? ", " : "") + std::to_string(e.shape[i]);
                shape += "]";
                return gb_fail("%s: tensor '%s' offsets [%lld,%lld) do not match shape %s %s or leave the file (%lld data bytes)",
                               path, name.c_str(), e.begin, e.end, shape.c_str(), dtype.c_str(), data_bytes);
            }
            f.entries.push_back(std::move(e));
        } while (j.lit(','));
        if (!j.lit('}')) return gb_fail("%s: header is not JSON (%s)", path, j.err.empty() ? "it does not end" : j.err.c_str());
    }
    j.ws();
    if (j.p != j.end) return gb_fail("%s: header is not JSON (text after its end)", path);
    return 0;
}

void st_free(StFile* f) {
    if (!f) return;
    if (f->map) munmap(const_cast<uint8_t*>(f->map), f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

// ---------------------------------------------------------------- to the device
template <typename S> __device__ __forceinline__ float st_float(S v) { return float(v); }
template <> __device__ __forceinline__ float st_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float st_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename S, typename D>
__global__ void st_convert_float_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
        dst[i] = gb_from_float<D>(st_float<S>(src[i]));
}
template <typename S>
__global__ void st_convert_int_kernel(const S* __restrict__ src, int* __restrict__ dst, size_t n) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
        dst[i] = int(src[i]);
}

template <typename S>
void convert_float(const void* src, void* dst, int keep, size_t n, cudaStream_t stream) {
    const unsigned grid = unsigned(n / 256 + 1 < 4096 ? n / 256 + 1 : 4096);
    if (keep == KEEP_F32) st_convert_float_kernel<S, float><<<grid, 256, 0, stream>>>((const S*)src, (float*)dst, n);
    else st_convert_float_kernel<S, __nv_bfloat16><<<grid, 256, 0, stream>>>((const S*)src, (__nv_bfloat16*)dst, n);
}
template <typename S>
void convert_int(const void* src, void* dst, size_t n, cudaStream_t stream) {
    const unsigned grid = unsigned(n / 256 + 1 < 4096 ? n / 256 + 1 : 4096);
    st_convert_int_kernel<S><<<grid, 256, 0, stream>>>((const S*)src, (int*)dst, n);
}

constexpr size_t STAGE_BYTES = 32u << 20;
struct Staging {
    uint8_t* host[2] = {nullptr, nullptr};
    uint8_t* dev[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};
    int device = -1;
};
Staging g_stage;
std::mutex g_stage_mu;

int staging_ready(bool need_dev) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return gb_fail("gb_st_upload: no current device");
    for (int i = 0; i < 2; ++i) {
        if (!g_stage.host[i] && cudaHostAlloc((void**)&g_stage.host[i], STAGE_BYTES, cudaHostAllocDefault) != cudaSuccess)
            return gb_fail("gb_st_upload: cannot allocate %zu bytes of pinned memory", STAGE_BYTES);
        if (!g_stage.done[i] && cudaEventCreateWithFlags(&g_stage.done[i], cudaEventDisableTiming) != cudaSuccess)
            return gb_fail("gb_st_upload: cannot create an event");
    }
    if (need_dev && g_stage.device != dev) {
        // staging on the device for tensors that are converted there (kept for the next file)
        for (int i = 0; i < 2; ++i) {
            if (g_stage.busy[i]) { cudaEventSynchronize(g_stage.done[i]); g_stage.busy[i] = false; }
            g_stage.dev[i] = nullptr;           // the old device keeps its 64 MB; a process loads on one device
            if (cudaMalloc((void**)&g_stage.dev[i], STAGE_BYTES) != cudaSuccess)
                return gb_fail("gb_st_upload: cannot allocate %zu bytes of device staging", STAGE_BYTES);
        }
        g_stage.device = dev;
    }
    return 0;
}

}  // namespace

// Opens and checks a file.  *handle stays valid until gb_st_close.
GB_API int gb_st_open(const char* path, void** handle) {
    *handle = nullptr;
    StFile* f = new StFile;
    f->path = path;
    f->fd = open(path, O_RDONLY | O_CLOEXEC);
    if (f->fd < 0) { int e = errno; st_free(f); return gb_fail("%s: cannot open (%s)", path, strerror(e)); }
    struct stat st;
    if (fstat(f->fd, &st) != 0) { int e = errno; st_free(f); return gb_fail("%s: cannot stat (%s)", path, strerror(e)); }
    f->size = size_t(st.st_size);
    if (f->size < 8) { size_t n = f->size; st_free(f); return gb_fail("%s: %zu bytes is too short for a safetensors header", path, n); }
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) { int e = errno; st_free(f); return gb_fail("%s: cannot map (%s)", path, strerror(e)); }
    f->map = static_cast<const uint8_t*>(m);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | f->map[i];
    if (hlen == 0 || hlen > f->size - 8) {
        size_t n = f->size;
        st_free(f);
        return gb_fail("%s: header length %llu does not fit the file (%zu bytes)", path, (unsigned long long)hlen, n);
    }
    f->base = 8 + size_t(hlen);
    if (parse_header(*f, reinterpret_cast<const char*>(f->map + 8), size_t(hlen))) { st_free(f); return 1; }
    *handle = f;
    return 0;
}

GB_API int gb_st_close(void* handle) {
    st_free(static_cast<StFile*>(handle));
    return 0;
}

GB_API int gb_st_count(void* handle) { return int(static_cast<StFile*>(handle)->entries.size()); }

// Entry i: its name and dtype as strings, its shape, and where its bytes lie in this process (all owned by the
// handle).
GB_API int gb_st_entry(void* handle, int i, const char** name, const char** dtype, int* ndim, const long long** shape,
                       const void** bytes, long long* nbytes) {
    StFile* f = static_cast<StFile*>(handle);
    GB_REQUIRE(i >= 0 && size_t(i) < f->entries.size(), "gb_st_entry: %s has no tensor %d", f->path.c_str(), i);
    const StEntry& e = f->entries[i];
    *name = e.name.c_str();
    *dtype = ST_NAMES[e.type];
    *ndim = int(e.shape.size());
    *shape = e.shape.data();
    *bytes = f->map + f->base + e.begin;
    *nbytes = e.end - e.begin;
    return 0;
}

GB_API int gb_st_metadata_count(void* handle) { return int(static_cast<StFile*>(handle)->metadata.size()); }
GB_API int gb_st_metadata(void* handle, int i, const char** key, const char** value) {
    StFile* f = static_cast<StFile*>(handle);
    GB_REQUIRE(i >= 0 && size_t(i) < f->metadata.size(), "gb_st_metadata: %s has no metadata entry %d", f->path.c_str(), i);
    *key = f->metadata[i].first.c_str();
    *value = f->metadata[i].second.c_str();
    return 0;
}

// Tensor i to device memory at dst, kept as `keep` (0: float32, 1: bfloat16, 2: int32): floats of any width become
// float32 or bfloat16, integers int32.  The copies and conversions are queued on `stream`; the call returns when
// the last piece has left the file's map (the staging buffers may still be on their way).
GB_API int gb_st_upload(void* handle, int i, void* dst, int keep, cudaStream_t stream) {
    StFile* f = static_cast<StFile*>(handle);
    GB_REQUIRE(i >= 0 && size_t(i) < f->entries.size(), "gb_st_upload: %s has no tensor %d", f->path.c_str(), i);
    const StEntry& e = f->entries[i];
    const bool is_float = e.type <= ST_BF16;
    GB_REQUIRE(keep == KEEP_F32 || keep == KEEP_BF16 || keep == KEEP_I32, "gb_st_upload: unknown storage type %d", keep);
    GB_REQUIRE(is_float == (keep != KEEP_I32), "gb_st_upload: tensor '%s' is stored as %s and cannot be kept as %s",
               e.name.c_str(), ST_NAMES[e.type], keep == KEEP_F32 ? "float32" : keep == KEEP_BF16 ? "bfloat16" : "int32");
    const size_t total = size_t(e.end - e.begin);
    if (total == 0) return 0;
    const bool same = (e.type == ST_F32 && keep == KEEP_F32) || (e.type == ST_BF16 && keep == KEEP_BF16) ||
                      (e.type == ST_I32 && keep == KEEP_I32);
    const size_t src_size = size_t(ST_SIZES[e.type]), dst_size = keep == KEEP_BF16 ? 2 : 4;
    std::lock_guard<std::mutex> lock(g_stage_mu);
    if (staging_ready(!same)) return 1;
    const uint8_t* src = f->map + f->base + e.begin;
    int b = 0;
    for (size_t off = 0; off < total; off += STAGE_BYTES, b ^= 1) {
        const size_t bytes = total - off < STAGE_BYTES ? total - off : STAGE_BYTES;
        if (g_stage.busy[b]) {
            if (cudaEventSynchronize(g_stage.done[b]) != cudaSuccess) return gb_fail("gb_st_upload: a copy of '%s' failed", e.name.c_str());
            g_stage.busy[b] = false;
        }
        memcpy(g_stage.host[b], src + off, bytes);
        const size_t n = bytes / src_size, first = off / src_size;
        uint8_t* out = static_cast<uint8_t*>(dst) + first * dst_size;
        cudaError_t err;
        if (same) {
            err = cudaMemcpyAsync(out, g_stage.host[b], bytes, cudaMemcpyHostToDevice, stream);
        } else {
            err = cudaMemcpyAsync(g_stage.dev[b], g_stage.host[b], bytes, cudaMemcpyHostToDevice, stream);
            if (err == cudaSuccess) {
                switch (e.type) {
                    case ST_F64: convert_float<double>(g_stage.dev[b], out, keep, n, stream); break;
                    case ST_F32: convert_float<float>(g_stage.dev[b], out, keep, n, stream); break;
                    case ST_F16: convert_float<__half>(g_stage.dev[b], out, keep, n, stream); break;
                    case ST_BF16: convert_float<__nv_bfloat16>(g_stage.dev[b], out, keep, n, stream); break;
                    case ST_I64: convert_int<long long>(g_stage.dev[b], out, n, stream); break;
                    case ST_I16: convert_int<short>(g_stage.dev[b], out, n, stream); break;
                    case ST_I8: convert_int<signed char>(g_stage.dev[b], out, n, stream); break;
                    default: convert_int<unsigned char>(g_stage.dev[b], out, n, stream); break;
                }
                err = cudaGetLastError();
            }
        }
        if (err == cudaSuccess) err = cudaEventRecord(g_stage.done[b], stream);
        if (err != cudaSuccess) return gb_fail("gb_st_upload: tensor '%s': %s", e.name.c_str(), cudaGetErrorString(err));
        g_stage.busy[b] = true;
    }
    return 0;
}
