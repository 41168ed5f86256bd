// GGUF reader (format versions 2 and 3, single file) and the Q2_0 expert loader that fills the
// device arena from it. The reader follows the reference's own (core/gguf.cpp:17-120: the same walk
// over header, key/value pairs and tensor directory, here over an in-memory buffer with bounds
// flags instead of a FILE* with exceptions) and the published description of the container: a header
// (magic "GGUF", version, tensor count, key/value count), typed key/value pairs, a tensor
// directory (name, dimensions with the fastest first, ggml type id, offset into the data section)
// and the data section, which starts at the next multiple of general.alignment (32 by default).
//
// The loader follows the reference's load_experts (arch/qwen4exp/experts.cpp:65-131): per layer
// the tensors blk.<l>.ffn_gate_exps.weight, ffn_up_exps, ffn_down_exps (ggml type 42, expert e's
// matrix at e * mat_bytes inside the tensor) are read in pieces of several experts and repacked.
// Here the pieces go to the GPU as they are (pinned staging, two buffers so that the next read
// overlaps the copy and the kernels), the repack to the planar form and the tiling run on the
// device, and the blobs land in the HBM arena. Split files ("-00001-of-0000N") are not handled.
#include "frx_common.cuh"

#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <map>
#include <string>
#include <vector>

struct frx_gguf {
    std::string path;
    uint32_t version = 0;
    uint64_t alignment = 32, data_start = 0, file_size = 0;
    struct Tensor {
        std::string name;
        int n_dims = 0;
        int64_t dims[4] = {1, 1, 1, 1};
        uint32_t type = 0;
        uint64_t offset = 0, bytes = 0;   // absolute file offset; bytes from the gap to the next tensor
    };
    std::vector<Tensor> tensors;
    std::map<std::string, size_t> by_name;
    std::map<std::string, int64_t> ints;   // integer and boolean metadata, widened
};

namespace {
using frx::fail;

struct Reader {
    const uint8_t* p;
    size_t n, at = 0;
    bool ok = true;
    template <class T>
    T pod() {
        T v{};
        if (at + sizeof(T) > n) {
            ok = false;
            return v;
        }
        std::memcpy(&v, p + at, sizeof(T));
        at += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t len = pod<uint64_t>();
        if (!ok || len > n - at) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char*>(p + at), size_t(len));
        at += size_t(len);
        return s;
    }
    void skip(uint64_t bytes) {
        if (bytes > n - at) ok = false; else at += size_t(bytes);
    }
};

// value type ids of the format
enum : uint32_t { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };

size_t scalar_size(uint32_t t) {
    switch (t) {
        case T_U8: case T_I8: case T_BOOL: return 1;
        case T_U16: case T_I16: return 2;
        case T_U32: case T_I32: case T_F32: return 4;
        case T_U64: case T_I64: case T_F64: return 8;
        default: return 0;
    }
}

// Reads one value; integers and booleans are returned through *as_int (has_int set).
void read_value(Reader& r, uint32_t type, int depth, bool* has_int, int64_t* as_int) {
    *has_int = false;
    switch (type) {
        case T_U8: *as_int = r.pod<uint8_t>(); *has_int = true; break;
        case T_I8: *as_int = r.pod<int8_t>(); *has_int = true; break;
        case T_U16: *as_int = r.pod<uint16_t>(); *has_int = true; break;
        case T_I16: *as_int = r.pod<int16_t>(); *has_int = true; break;
        case T_U32: *as_int = r.pod<uint32_t>(); *has_int = true; break;
        case T_I32: *as_int = r.pod<int32_t>(); *has_int = true; break;
        case T_U64: *as_int = int64_t(r.pod<uint64_t>()); *has_int = true; break;
        case T_I64: *as_int = r.pod<int64_t>(); *has_int = true; break;
        case T_BOOL: *as_int = r.pod<uint8_t>() != 0; *has_int = true; break;
        case T_F32: r.skip(4); break;
        case T_F64: r.skip(8); break;
        case T_STRING: r.str(); break;
        case T_ARRAY: {
            const uint32_t et = r.pod<uint32_t>();
            const uint64_t count = r.pod<uint64_t>();
            if (!r.ok || depth > 2) {
                r.ok = false;
                break;
            }
            if (const size_t sz = scalar_size(et)) {
                if (count > (r.n - r.at) / sz) r.ok = false; else r.skip(count * sz);
            } else {
                bool hi;
                int64_t iv;
                for (uint64_t i = 0; i < count && r.ok; ++i) read_value(r, et, depth + 1, &hi, &iv);
            }
            break;
        }
        default: r.ok = false;
    }
}

// bytes of a tensor of a known ggml type: block bytes * elements / block elements; 0 = unknown type
uint64_t type_bytes(uint32_t type, uint64_t elements) {
    switch (type) {
        case 0: return elements * 4;               // F32
        case 1: return elements * 2;               // F16
        case 30: return elements * 2;              // BF16
        case 42: return elements / 64 * 18;        // Q2_0: fp16 scale + 16 code bytes per 64 weights
        default: return 0;
    }
}

}  // namespace

using namespace frx;

extern "C" {

int frx_gguf_open(frx_gguf** out, const char* path) {
    if (!out || !path) return fail(FRX_ERR_ARG, "frx_gguf_open: null argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(FRX_ERR_ARG, "frx_gguf_open: cannot open %s: %s", path, std::strerror(errno));
    const off_t size = lseek(fd, 0, SEEK_END);
    // the directory of a large model is a few megabytes; read as much as needed, doubling
    std::vector<uint8_t> head;
    size_t want = size_t(1) << 20;
    frx_gguf* g = new frx_gguf();
    g->path = path;
    g->file_size = uint64_t(size);
    for (;;) {
        if (want > size_t(size)) want = size_t(size);
        head.resize(want);
        size_t got = 0;
        while (got < want) {
            const ssize_t r = pread(fd, head.data() + got, want - got, off_t(got));
            if (r <= 0) break;
            got += size_t(r);
        }
        if (got < want) {
            close(fd);
            delete g;
            return fail(FRX_ERR_ARG, "frx_gguf_open: short read of %s", path);
        }
        Reader r{head.data(), head.size()};
        g->tensors.clear();
        g->by_name.clear();
        g->ints.clear();
        const uint32_t magic = r.pod<uint32_t>();
        g->version = r.pod<uint32_t>();
        const uint64_t n_tensors = r.pod<uint64_t>(), n_kv = r.pod<uint64_t>();
        if (r.ok && (magic != 0x46554747u || g->version < 2 || g->version > 3)) {
            close(fd);
            delete g;
            return fail(FRX_ERR_ARG, "frx_gguf_open: %s is not a GGUF file of version 2 or 3", path);
        }
        for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
            const std::string key = r.str();
            const uint32_t type = r.pod<uint32_t>();
            bool has_int = false;
            int64_t iv = 0;
            if (r.ok) read_value(r, type, 0, &has_int, &iv);
            if (r.ok && has_int) g->ints[key] = iv;
        }
        for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
            frx_gguf::Tensor t;
            t.name = r.str();
            const uint32_t nd = r.pod<uint32_t>();
            if (!r.ok || nd < 1 || nd > 4) {
                r.ok = r.ok && false;
                break;
            }
            t.n_dims = int(nd);
            for (uint32_t d = 0; d < nd; ++d) t.dims[d] = int64_t(r.pod<uint64_t>());
            t.type = r.pod<uint32_t>();
            t.offset = r.pod<uint64_t>();   // relative to the data section for now
            if (r.ok) g->tensors.push_back(t);
        }
        if (r.ok) {
            const auto a = g->ints.find("general.alignment");
            if (a != g->ints.end()) g->alignment = uint64_t(a->second);
            if (g->alignment == 0 || (g->alignment & (g->alignment - 1)) || g->alignment > (1u << 20)) {
                close(fd);
                delete g;
                return fail(FRX_ERR_ARG, "frx_gguf_open: bad general.alignment in %s", path);
            }
            g->data_start = (uint64_t(r.at) + g->alignment - 1) / g->alignment * g->alignment;
            break;
        }
        if (want == size_t(size)) {   // the whole file was there and it still did not parse
            close(fd);
            delete g;
            return fail(FRX_ERR_ARG, "frx_gguf_open: %s is truncated or malformed", path);
        }
        want *= 2;
    }
    close(fd);
    // absolute offsets, and each tensor's bytes from its type (or the gap to the next offset)
    std::vector<uint64_t> starts;
    for (auto& t : g->tensors) {
        t.offset += g->data_start;
        starts.push_back(t.offset);
    }
    std::sort(starts.begin(), starts.end());
    for (size_t i = 0; i < g->tensors.size(); ++i) {
        auto& t = g->tensors[i];
        uint64_t elements = 1;
        for (int d = 0; d < t.n_dims; ++d) elements *= uint64_t(t.dims[d]);
        t.bytes = type_bytes(t.type, elements);
        const auto next = std::upper_bound(starts.begin(), starts.end(), t.offset);
        const uint64_t gap = (next == starts.end() ? g->file_size : *next) - t.offset;
        if (t.bytes == 0) t.bytes = gap;
        if (t.offset > g->file_size || t.bytes > g->file_size - t.offset) {
            const int rc = fail(FRX_ERR_ARG, "frx_gguf_open: tensor %s reaches beyond the end of %s", t.name.c_str(), path);
            delete g;
            return rc;
        }
        g->by_name[t.name] = i;
    }
    *out = g;
    return FRX_OK;
}

int frx_gguf_close(frx_gguf* g) {
    delete g;
    return FRX_OK;
}

int frx_gguf_tensor_count(const frx_gguf* g) { return g ? int(g->tensors.size()) : 0; }
const char* frx_gguf_tensor_name(const frx_gguf* g, int i) {
    return g && i >= 0 && size_t(i) < g->tensors.size() ? g->tensors[size_t(i)].name.c_str() : nullptr;
}
int64_t frx_gguf_get_int(const frx_gguf* g, const char* key, int64_t fallback) {
    if (!g || !key) return fallback;
    const auto it = g->ints.find(key);
    return it == g->ints.end() ? fallback : it->second;
}

int frx_gguf_tensor(const frx_gguf* g, const char* name, uint32_t* type, int* n_dims, int64_t* dims4, uint64_t* file_offset, uint64_t* bytes) {
    if (!g || !name) return fail(FRX_ERR_ARG, "frx_gguf_tensor: null argument");
    const auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return fail(FRX_ERR_ARG, "frx_gguf_tensor: no tensor %s", name);
    const auto& t = g->tensors[it->second];
    if (type) *type = t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (dims4) std::memcpy(dims4, t.dims, sizeof t.dims);
    if (file_offset) *file_offset = t.offset;
    if (bytes) *bytes = t.bytes;
    return FRX_OK;
}

int frx_arena_load_gguf(frx_arena* a, const frx_gguf* g, int layer0, int n_layer, int n_expert, int n, int ff, frx_stream_t stream,
                        uint64_t* bytes_read, double* seconds) {
    if (!a || !g) return fail(FRX_ERR_ARG, "frx_arena_load_gguf: null argument");
    if (layer0 < 0 || n_layer < 0 || n_expert < 1) return fail(FRX_ERR_ARG, "frx_arena_load_gguf: layers [%d, +%d), %d experts", layer0, n_layer, n_expert);
    if (n < kUnitK || ff < kUnitK || n % kUnitK || ff % kUnitK) return fail(FRX_ERR_SHAPE, "frx_arena_load_gguf: n %d, ff %d", n, ff);
    const size_t mat_gu = frx_q2_mat_bytes(ff, n), mat_dn = frx_q2_mat_bytes(n, ff), blob = frx_q2_expert_bytes(n, ff);
    const size_t stride = frx_arena_stride(a);
    if (stride < blob) return fail(FRX_ERR_ARG, "frx_arena_load_gguf: the arena was made for another shape");
    // the directory first: every tensor must be there, of type Q2_0 and of the expected size
    struct Slabs {
        uint64_t off[3];
    };
    std::vector<Slabs> layers(size_t(n_layer) > 0 ? size_t(n_layer) : 0);
    const char* names[3] = {"ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"};
    for (int l = 0; l < n_layer; ++l)
        for (int k = 0; k < 3; ++k) {
            const std::string name = "blk." + std::to_string(layer0 + l) + "." + names[k] + ".weight";
            const auto it = g->by_name.find(name);
            if (it == g->by_name.end()) return fail(FRX_ERR_ARG, "frx_arena_load_gguf: missing %s", name.c_str());
            const auto& t = g->tensors[it->second];
            const uint64_t need = uint64_t(n_expert) * (k < 2 ? mat_gu : mat_dn);
            if (t.type != 42) return fail(FRX_ERR_SHAPE, "frx_arena_load_gguf: %s has ggml type %u, not Q2_0 (42)", name.c_str(), t.type);
            if (t.bytes != need) return fail(FRX_ERR_SHAPE, "frx_arena_load_gguf: %s holds %llu bytes, %llu expected", name.c_str(),
                                             (unsigned long long)t.bytes, (unsigned long long)need);
            layers[size_t(l)].off[k] = t.offset;
        }
    if (bytes_read) *bytes_read = 0;
    if (seconds) *seconds = 0.0;
    if (n_layer == 0) return FRX_OK;
    if (!frx_arena_blob(a, layer0 + n_layer - 1, n_expert - 1)) return fail(FRX_ERR_ARG, "frx_arena_load_gguf: layers or experts outside the arena");

    const int piece = n_expert < 64 ? n_expert : 64;   // experts per read
    const size_t piece_ggml = size_t(piece) * blob;
    const int fd = open(g->path.c_str(), O_RDONLY);
    if (fd < 0) return fail(FRX_ERR_ARG, "frx_arena_load_gguf: cannot open %s: %s", g->path.c_str(), std::strerror(errno));
    uint8_t* host[2] = {nullptr, nullptr};
    uint8_t *dev_ggml = nullptr, *dev_planar = nullptr;
    cudaEvent_t copied[2] = {nullptr, nullptr};
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
        e = cudaMallocHost(reinterpret_cast<void**>(&host[i]), piece_ggml);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&copied[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&dev_ggml), 2 * piece_ggml);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&dev_planar), size_t(piece) * stride);
    int rc = e == cudaSuccess ? FRX_OK : cuda_fail(e, "frx_arena_load_gguf: staging allocation");
    const auto t0 = std::chrono::steady_clock::now();
    uint64_t total = 0;
    int it = 0;
    for (int l = 0; l < n_layer && rc == FRX_OK; ++l)
        for (int e0 = 0; e0 < n_expert && rc == FRX_OK; e0 += piece, ++it) {
            const int ne = n_expert - e0 < piece ? n_expert - e0 : piece;
            const int b = it & 1;
            if (it >= 2) e = cudaEventSynchronize(copied[b]);   // the copy that last used this host buffer has finished
            if (e != cudaSuccess) {
                rc = cuda_fail(e, "frx_arena_load_gguf: cudaEventSynchronize");
                break;
            }
            // the three ranges of this piece, one after the other in the staging buffer: gate, up, down
            const size_t len[3] = {size_t(ne) * mat_gu, size_t(ne) * mat_gu, size_t(ne) * mat_dn};
            size_t at = 0;
            for (int k = 0; k < 3 && rc == FRX_OK; ++k) {
                const uint64_t src = layers[size_t(l)].off[k] + uint64_t(e0) * (k < 2 ? mat_gu : mat_dn);
                size_t got = 0;
                while (got < len[k]) {
                    const ssize_t r = pread(fd, host[b] + at + got, len[k] - got, off_t(src + got));
                    if (r <= 0) {
                        rc = fail(FRX_ERR_ARG, "frx_arena_load_gguf: short read of %s at %llu", g->path.c_str(), (unsigned long long)(src + got));
                        break;
                    }
                    got += size_t(r);
                }
                at += len[k];
            }
            if (rc != FRX_OK) break;
            total += at;
            uint8_t* dg = dev_ggml + size_t(b) * piece_ggml;
            e = cudaMemcpyAsync(dg, host[b], at, cudaMemcpyHostToDevice, stream);
            if (e == cudaSuccess) e = cudaEventRecord(copied[b], stream);
            if (e != cudaSuccess) {
                rc = cuda_fail(e, "frx_arena_load_gguf: copy");
                break;
            }
            // ggml -> planar blobs [gate | up | down] at the arena's stride, then planar -> tiled into the arena.
            // (The planar staging is reused by the next piece; the stream orders the kernels.)
            for (int x = 0; x < ne && rc == FRX_OK; ++x) {
                uint8_t* pb = dev_planar + size_t(x) * stride;
                rc = frx_q2_repack(dg + size_t(x) * mat_gu, ff, n, pb, stream);
                if (rc == FRX_OK) rc = frx_q2_repack(dg + len[0] + size_t(x) * mat_gu, ff, n, pb + mat_gu, stream);
                if (rc == FRX_OK) rc = frx_q2_repack(dg + len[0] + len[1] + size_t(x) * mat_dn, n, ff, pb + 2 * mat_gu, stream);
            }
            if (rc == FRX_OK) rc = frx_q2_tile_experts(dev_planar, stride, frx_arena_blob(a, layer0 + l, e0), stride, ne, n, ff, stream);
        }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (rc == FRX_OK && e != cudaSuccess) rc = cuda_fail(e, "frx_arena_load_gguf: cudaStreamSynchronize");
    close(fd);
    for (int i = 0; i < 2; ++i) {
        if (host[i]) cudaFreeHost(host[i]);
        if (copied[i]) cudaEventDestroy(copied[i]);
    }
    cudaFree(dev_ggml);
    cudaFree(dev_planar);
    if (bytes_read) *bytes_read = total;
    if (seconds) *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return rc;
}

}  // extern "C"
