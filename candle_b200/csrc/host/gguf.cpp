// GGUF container reader: header, metadata, tensor directory, and tensor upload straight from the file mapping to the
// device.  Behaviour follows candle-core/src/quantized/gguf_file.rs:
//   magic / versions 1-3 (:36-78), length prefixes u32 in v1 and u64 later (:28-33), strings with trailing NULs stripped
//   (:130-152), the thirteen value types and nested arrays (:154-222, depth cap 64), tensor infos with at most 4
//   dimensions stored innermost-first and reversed on read (:516-556), `general.alignment` (default 32) deciding where
//   tensor data starts (:558-568), and the bounds checks that reject counts, strings, arrays and tensors which cannot
//   fit in the file (:14-26, :478-505, :96-110).
// Unlike the reference, which reads a tensor into a host vector and uploads that, the file stays memory-mapped and a
// tensor - or a range of its rows, for a tensor-parallel shard - is copied from the mapping to the device in one call.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <sstream>

#include "../../../include/candle_q_b200.h"
#include "qtensor.h"

namespace candle_q {
namespace {

constexpr uint64_t kMaxString = 1ull << 30, kMaxArray = 1ull << 30, kDefaultAlignment = 32;
constexpr uint32_t kMaxDims = 4;
constexpr int kMaxDepth = 64;

struct TensorInfo {
    std::string name;
    GgmlDType dtype;
    std::vector<int64_t> dims;      // outermost first (candle's order)
    uint64_t offset, nbytes;
};

struct Cursor {
    const uint8_t *base;
    uint64_t size, pos = 0;
    int version = 0;
    uint64_t remaining() const { return size - pos; }
    template <typename T> T get() {
        if (remaining() < sizeof(T)) throw Error("gguf: unexpected end of file");
        T v;
        std::memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    uint64_t length() { return version == 1 ? (uint64_t)get<uint32_t>() : get<uint64_t>(); }
    std::string str() {
        const uint64_t len = length();
        if (len > kMaxString) throw Error("gguf: string length " + std::to_string(len) + " exceeds max " + std::to_string(kMaxString));
        if (len > remaining())
            throw Error("gguf: string length " + std::to_string(len) + " exceeds remaining file bytes " + std::to_string(remaining()));
        std::string s((const char *)base + pos, (size_t)len);
        pos += len;
        while (!s.empty() && s.back() == '\0') s.pop_back();
        return s;
    }
};

void json_escape(std::ostringstream &o, const std::string &s) {
    o << '"';
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') o << '\\' << c;
        else if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o << b; }
        else o << c;
    }
    o << '"';
}

uint64_t min_disk_size(uint32_t type, int version) {
    const uint64_t prefix = version == 1 ? 4 : 8;
    switch (type) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    case 8: return prefix;
    case 9: return 4 + prefix;
    }
    throw Error("gguf: unrecognized value-type " + std::to_string(type));
}

// One metadata value, appended to `o` as JSON (integers and floats as numbers, bool as true/false).
void read_value(Cursor &c, uint32_t type, int depth, std::ostringstream &o) {
    if (depth > kMaxDepth) throw Error("gguf: value nesting depth exceeds max " + std::to_string(kMaxDepth));
    switch (type) {
    case 0: o << (unsigned)c.get<uint8_t>(); break;
    case 1: o << (int)c.get<int8_t>(); break;
    case 2: o << c.get<uint16_t>(); break;
    case 3: o << c.get<int16_t>(); break;
    case 4: o << c.get<uint32_t>(); break;
    case 5: o << c.get<int32_t>(); break;
    case 6: { const float f = c.get<float>(); if (f != f || f - f != 0.0f) o << "null"; else { o.precision(9); o << f; } break; }
    case 7: {
        const uint8_t b = c.get<uint8_t>();
        if (b > 1) throw Error("gguf: unexpected bool value " + std::to_string(b));
        o << (b ? "true" : "false");
        break;
    }
    case 8: json_escape(o, c.str()); break;
    case 9: {
        const uint32_t et = c.get<uint32_t>();
        const uint64_t len = c.length();
        if (len > kMaxArray) throw Error("gguf: array length " + std::to_string(len) + " exceeds max " + std::to_string(kMaxArray));
        const uint64_t each = min_disk_size(et, c.version);
        if (len > c.remaining() / each)
            throw Error("gguf: array of " + std::to_string(len) + " elements cannot fit in the remaining " + std::to_string(c.remaining()) + " bytes");
        o << '[';
        for (uint64_t i = 0; i < len; ++i) {
            if (i) o << ',';
            read_value(c, et, depth + 1, o);
        }
        o << ']';
        break;
    }
    case 10: o << c.get<uint64_t>(); break;
    case 11: o << c.get<int64_t>(); break;
    case 12: { const double f = c.get<double>(); if (f != f || f - f != 0.0) o << "null"; else { o.precision(17); o << f; } break; }
    default: throw Error("gguf: unrecognized value-type " + std::to_string(type));
    }
}

}  // namespace

struct GgufFile {
    int fd = -1;
    const uint8_t *map = nullptr;
    uint64_t size = 0;
    int version = 0;
    uint64_t tensor_data_offset = 0, alignment = kDefaultAlignment;
    std::vector<TensorInfo> tensors;
    std::map<std::string, size_t> by_name;
    std::string metadata_json;      // {"key": value, ...}

    ~GgufFile() {
        if (map) munmap((void *)map, size);
        if (fd >= 0) close(fd);
    }

    void open(const char *path) {
        fd = ::open(path, O_RDONLY);
        if (fd < 0) throw Error(std::string("gguf: cannot open ") + path);
        struct stat st;
        if (fstat(fd, &st) != 0) throw Error("gguf: cannot stat the file");
        size = (uint64_t)st.st_size;
        if (size == 0) throw Error("gguf: unexpected end of file");
        void *p = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (p == MAP_FAILED) throw Error("gguf: cannot map the file");
        map = (const uint8_t *)p;
        parse();
    }

    void parse() {
        Cursor c{map, size};
        const uint32_t magic = c.get<uint32_t>();
        if (magic != 0x46554747u && magic != 0x47475546u) {
            char b[64];
            std::snprintf(b, sizeof b, "unknown magic 0x%08x", magic);
            throw Error(b);
        }
        const uint32_t ver = c.get<uint32_t>();
        if (ver < 1 || ver > 3) throw Error("gguf: unsupported magic/version Gguf/" + std::to_string(ver));
        version = c.version = (int)ver;
        const uint64_t tensor_count = c.length(), kv_count = c.length();
        if (tensor_count > kMaxArray) throw Error("gguf: tensor_count " + std::to_string(tensor_count) + " exceeds max " + std::to_string(kMaxArray));
        if (kv_count > kMaxArray) throw Error("gguf: metadata_kv_count " + std::to_string(kv_count) + " exceeds max " + std::to_string(kMaxArray));
        const uint64_t prefix = version == 1 ? 4 : 8;
        const uint64_t needed = kv_count * (prefix + 4 + 1) + tensor_count * (prefix + 4 + 4 + 8);
        if (needed > c.remaining())
            throw Error("gguf: header declares " + std::to_string(tensor_count) + " tensors and " + std::to_string(kv_count) +
                        " metadata entries, needs at least " + std::to_string(needed) + " bytes, only " + std::to_string(c.remaining()) + " remaining");
        std::ostringstream js;
        js << '{';
        bool have_alignment = false;
        for (uint64_t i = 0; i < kv_count; ++i) {
            const std::string key = c.str();
            const uint32_t vt = c.get<uint32_t>();
            if (key == "general.alignment" && (vt <= 5)) {       // u8, i8, u16, i16, u32, i32 (non-negative) count
                const uint64_t save = c.pos;
                int64_t v = 0;
                switch (vt) {
                case 0: v = c.get<uint8_t>(); break;
                case 1: v = c.get<int8_t>(); break;
                case 2: v = c.get<uint16_t>(); break;
                case 3: v = c.get<int16_t>(); break;
                case 4: v = c.get<uint32_t>(); break;
                case 5: v = c.get<int32_t>(); break;
                }
                c.pos = save;
                if (v >= 0) { alignment = (uint64_t)v; have_alignment = true; }
            }
            if (i) js << ',';
            json_escape(js, key);
            js << ':';
            read_value(c, vt, 0, js);
        }
        js << '}';
        metadata_json = js.str();
        (void)have_alignment;
        if (alignment == 0) throw Error("gguf: general.alignment is zero");
        tensors.reserve((size_t)tensor_count);
        for (uint64_t i = 0; i < tensor_count; ++i) {
            TensorInfo t;
            t.name = c.str();
            const uint32_t nd = c.get<uint32_t>();
            if (nd > kMaxDims)
                throw Error("gguf: tensor '" + t.name + "' has " + std::to_string(nd) + " dimensions, max is " + std::to_string(kMaxDims));
            t.dims.resize(nd);
            for (uint32_t d = 0; d < nd; ++d) t.dims[nd - 1 - d] = version == 1 ? (int64_t)c.get<uint32_t>() : (int64_t)c.get<uint64_t>();
            t.dtype = ggml_dtype_from_u32(c.get<uint32_t>());
            t.offset = c.get<uint64_t>();
            uint64_t elems = 1;
            for (int64_t d : t.dims) {
                if (d < 0 || (d > 0 && elems > UINT64_MAX / (uint64_t)d)) throw Error("gguf: tensor '" + t.name + "' has an impossible shape");
                elems *= (uint64_t)d;
            }
            if (elems % block_size(t.dtype) != 0)
                throw Error("the number of elements " + std::to_string(elems) + " is not divisible by the block size " +
                            std::to_string(block_size(t.dtype)));
            t.nbytes = elems / block_size(t.dtype) * type_size(t.dtype);
            by_name[t.name] = tensors.size();
            tensors.push_back(std::move(t));
        }
        tensor_data_offset = (c.pos + alignment - 1) / alignment * alignment;
    }

    const uint8_t *tensor_bytes(const TensorInfo &t) const {
        const uint64_t start = tensor_data_offset > UINT64_MAX - t.offset ? UINT64_MAX : tensor_data_offset + t.offset;
        const uint64_t remaining = start > size ? 0 : size - start;
        if (t.nbytes > remaining)
            throw Error("tensor needs " + std::to_string(t.nbytes) + " bytes at offset " + std::to_string(start) + ", only " +
                        std::to_string(remaining) + " remaining in file");
        return map + start;
    }
};

}  // namespace candle_q

using namespace candle_q;

namespace {
thread_local std::string g_err;
template <typename F> int guarded_g(F &&f) {
    try { f(); return 0; }
    catch (const std::exception &e) { g_err = e.what(); return 1; }
}
}  // namespace

extern "C" const char *cqh_gguf_last_error(void) { return g_err.c_str(); }

extern "C" int cqh_gguf_open(const char *path, void **out_handle) {
    return guarded_g([&] {
        std::unique_ptr<GgufFile> f(new GgufFile());
        f->open(path);
        *out_handle = f.release();
    });
}

extern "C" void cqh_gguf_close(void *handle) { delete (GgufFile *)handle; }
extern "C" int cqh_gguf_version(void *handle) { return ((GgufFile *)handle)->version; }
extern "C" uint64_t cqh_gguf_tensor_data_offset(void *handle) { return ((GgufFile *)handle)->tensor_data_offset; }
extern "C" int64_t cqh_gguf_tensor_count(void *handle) { return (int64_t)((GgufFile *)handle)->tensors.size(); }
extern "C" const char *cqh_gguf_metadata_json(void *handle) { return ((GgufFile *)handle)->metadata_json.c_str(); }

extern "C" int64_t cqh_gguf_find_tensor(void *handle, const char *name) {
    auto *f = (GgufFile *)handle;
    auto it = f->by_name.find(name);
    return it == f->by_name.end() ? -1 : (int64_t)it->second;
}

extern "C" int cqh_gguf_tensor_info(void *handle, int64_t index, const char **name, int *ggml_dtype, int64_t *dims, int *ndims,
                                    uint64_t *offset, uint64_t *nbytes) {
    return guarded_g([&] {
        auto *f = (GgufFile *)handle;
        if (index < 0 || (size_t)index >= f->tensors.size()) throw Error("gguf: tensor index out of range");
        const TensorInfo &t = f->tensors[(size_t)index];
        if (name) *name = t.name.c_str();
        if (ggml_dtype) *ggml_dtype = (int)t.dtype;
        if (ndims) *ndims = (int)t.dims.size();
        if (dims) for (size_t i = 0; i < t.dims.size(); ++i) dims[i] = t.dims[i];
        if (offset) *offset = t.offset;
        if (nbytes) *nbytes = t.nbytes;
    });
}

extern "C" int cqh_gguf_read_tensor(void *handle, int64_t index, void *host_out, uint64_t nbytes) {
    return guarded_g([&] {
        auto *f = (GgufFile *)handle;
        if (index < 0 || (size_t)index >= f->tensors.size()) throw Error("gguf: tensor index out of range");
        const TensorInfo &t = f->tensors[(size_t)index];
        if (nbytes != t.nbytes) throw Error("gguf: buffer size does not match the tensor");
        std::memcpy(host_out, f->tensor_bytes(t), (size_t)t.nbytes);
    });
}

extern "C" int cqh_gguf_load_tensor(void *handle, int64_t index, int device, int64_t row_start, int64_t row_count,
                                    void **out_qtensor) {
    return guarded_g([&] {
        auto *f = (GgufFile *)handle;
        if (index < 0 || (size_t)index >= f->tensors.size()) throw Error("gguf: tensor index out of range");
        const TensorInfo &t = f->tensors[(size_t)index];
        const uint8_t *bytes = f->tensor_bytes(t);
        std::vector<int64_t> dims = t.dims;
        uint64_t off = 0, len = t.nbytes;
        if (row_count >= 0) {       // rows [row_start, row_start + row_count) of the outermost dimension
            if (dims.empty() || row_start < 0 || row_start + row_count > dims[0]) throw Error("gguf: row range outside the tensor");
            const uint64_t per_row = dims[0] ? t.nbytes / (uint64_t)dims[0] : 0;
            if (dims[0] && per_row * (uint64_t)dims[0] != t.nbytes) throw Error("gguf: rows of this tensor are not whole blocks");
            off = per_row * (uint64_t)row_start;
            len = per_row * (uint64_t)row_count;
            dims[0] = row_count;
        }
        auto st = QCudaStorage::load_quantized(device, t.dtype, bytes + off, (size_t)len);
        *out_qtensor = new std::shared_ptr<QTensor>(new QTensor(std::move(st), dims));
    });
}
