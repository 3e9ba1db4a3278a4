// Packed-weight file reader: GGUF containers (versions 2 and 3, little-endian) holding GGML tensors.
//
// vortx carries GGML's dimension convention in its layout helpers (GGML_IDS and permute_ggml,
// src/shapes.rs:15-18, :261-265): a GGML tensor lists its dimensions innermost first, so a weight matrix of
// `rows` x `cols` is stored with ne[0] = cols, ne[1] = rows, row after row, each row a whole number of
// blocks.  GGML's Q4_0 (f16 d + 16 bytes, element i in the low nibble of byte i, element i + 16 in the
// high one) and Q8_0 (f16 d + 32 int8) blocks are byte for byte the host block stream of this library, so
// a tensor of those types goes from the mapped file straight into vx_qweights_upload.
//
// The container, restated from its published description: magic "GGUF", u32 version, u64 tensor count, u64
// metadata count; metadata as (string key, u32 type, value) with strings as u64 length + bytes and arrays as
// u32 element type + u64 count + elements; per tensor a string name, u32 number of dimensions, u64
// dimensions, u32 GGML type and u64 offset into the data section; the data section starts at the next
// multiple of the alignment (metadata "general.alignment", 32 by default) after the last tensor record.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "vx_internal.h"

namespace {

enum GgmlType : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q8_0 = 8 };

struct TensorInfo {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    uint32_t type = 0;
    uint64_t offset = 0;   // from the start of the data section
    uint64_t bytes = 0;    // 0 when the type's block size is not known here
};

// bytes per block and elements per block of the types this library can size
bool type_geometry(uint32_t type, uint64_t* block_bytes, uint64_t* block_elems) {
    switch (type) {
        case GGML_F32: *block_bytes = 4; *block_elems = 1; return true;
        case GGML_F16: *block_bytes = 2; *block_elems = 1; return true;
        case GGML_Q4_0: *block_bytes = 18; *block_elems = 32; return true;
        case GGML_Q8_0: *block_bytes = 34; *block_elems = 32; return true;
        default: return false;
    }
}

struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    template <class T>
    T get() {
        T v{};
        if (!ok || (size_t)(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    void skip(uint64_t n) {
        if (!ok || (uint64_t)(end - p) < n) ok = false;
        else p += n;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || (uint64_t)(end - p) < n || n > (1u << 20)) {
            ok = false;
            return {};
        }
        std::string s(reinterpret_cast<const char*>(p), (size_t)n);
        p += n;
        return s;
    }
};

uint64_t scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;   // u8, i8, bool
        case 2: case 3: return 2;           // u16, i16
        case 4: case 5: case 6: return 4;   // u32, i32, f32
        case 10: case 11: case 12: return 8;  // u64, i64, f64
        default: return 0;
    }
}

// Skips one metadata value; keeps a u32 (for the alignment key).
void skip_value(Cursor& c, uint32_t type, uint32_t* as_u32, int depth = 0) {
    if (type == 8) {
        c.str();
    } else if (type == 9) {
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (depth > 4) c.ok = false;
        if (et == 8 || et == 9) {
            for (uint64_t i = 0; i < n && c.ok; ++i) skip_value(c, et, nullptr, depth + 1);
        } else {
            const uint64_t s = scalar_size(et);
            if (s == 0) c.ok = false;
            else c.skip(n * s);
        }
    } else {
        const uint64_t s = scalar_size(type);
        if (s == 0) {
            c.ok = false;
        } else if (type == 4 && as_u32) {
            *as_u32 = c.get<uint32_t>();
        } else {
            c.skip(s);
        }
    }
}

}  // namespace

struct vx_wfile {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t data_start = 0;
    std::vector<TensorInfo> tensors;
    ~vx_wfile() {
        if (map) munmap(const_cast<uint8_t*>(map), size);
        if (fd >= 0) close(fd);
    }
};

extern "C" {

vx_status vx_wfile_open(const char* path, vx_wfile** out) {
    using vx::fail;
    VX_REQUIRE(path && out, VX_ERR_INVALID_ARGUMENT, "vx_wfile_open: null argument");
    *out = nullptr;
    std::unique_ptr<vx_wfile> f(new vx_wfile());
    f->fd = open(path, O_RDONLY);
    VX_REQUIRE(f->fd >= 0, VX_ERR_INVALID_ARGUMENT, "cannot open '%s': %s", path, strerror(errno));
    struct stat st;
    VX_REQUIRE(fstat(f->fd, &st) == 0 && st.st_size >= 24, VX_ERR_INVALID_ARGUMENT, "'%s' is too short to be a weight file", path);
    f->size = (size_t)st.st_size;
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    VX_REQUIRE(m != MAP_FAILED, VX_ERR_INVALID_ARGUMENT, "cannot map '%s': %s", path, strerror(errno));
    f->map = static_cast<const uint8_t*>(m);

    Cursor c{f->map, f->map + f->size};
    const uint32_t magic = c.get<uint32_t>();
    VX_REQUIRE(magic == 0x46554747u, VX_ERR_UNSUPPORTED, "'%s' does not start with GGUF", path);
    f->version = c.get<uint32_t>();
    VX_REQUIRE(f->version == 2 || f->version == 3, VX_ERR_UNSUPPORTED, "GGUF version %u (2 and 3 are read)", f->version);
    const uint64_t n_tensors = c.get<uint64_t>();
    const uint64_t n_kv = c.get<uint64_t>();
    VX_REQUIRE(c.ok && n_tensors <= (1u << 20) && n_kv <= (1u << 20), VX_ERR_INVALID_ARGUMENT, "implausible header in '%s'", path);
    uint32_t alignment = 32;
    for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        uint32_t v = 0;
        const bool is_align = key == "general.alignment";
        skip_value(c, type, is_align ? &v : nullptr);
        if (is_align && type == 4 && v != 0) alignment = v;
    }
    VX_REQUIRE(c.ok, VX_ERR_INVALID_ARGUMENT, "metadata of '%s' runs past the end of the file", path);
    VX_REQUIRE((alignment & (alignment - 1)) == 0, VX_ERR_INVALID_ARGUMENT, "alignment %u is not a power of two", alignment);
    f->tensors.resize((size_t)n_tensors);
    for (auto& t : f->tensors) {
        t.name = c.str();
        t.n_dims = c.get<uint32_t>();
        VX_REQUIRE(c.ok && t.n_dims >= 1 && t.n_dims <= 4, VX_ERR_INVALID_ARGUMENT, "tensor '%s' has %u dimensions", t.name.c_str(), t.n_dims);
        for (uint32_t d = 0; d < t.n_dims; ++d) t.ne[d] = c.get<uint64_t>();
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        uint64_t bb = 0, be = 0;
        if (type_geometry(t.type, &bb, &be) && t.ne[0] % be == 0)
            t.bytes = t.ne[0] / be * bb * t.ne[1] * t.ne[2] * t.ne[3];
    }
    VX_REQUIRE(c.ok, VX_ERR_INVALID_ARGUMENT, "tensor records of '%s' run past the end of the file", path);
    const uint64_t at = (uint64_t)(c.p - f->map);
    f->data_start = (at + alignment - 1) / alignment * alignment;
    for (const auto& t : f->tensors)
        VX_REQUIRE(t.offset % alignment == 0 && f->data_start + t.offset + t.bytes <= f->size, VX_ERR_INVALID_ARGUMENT,
                   "tensor '%s' (offset %llu, %llu bytes) does not lie inside '%s'", t.name.c_str(),
                   (unsigned long long)t.offset, (unsigned long long)t.bytes, path);
    *out = f.release();
    return VX_OK;
}

vx_status vx_wfile_close(vx_wfile* f) {
    delete f;
    return VX_OK;
}

vx_status vx_wfile_count(const vx_wfile* f, size_t* count) {
    VX_REQUIRE(f && count, VX_ERR_INVALID_ARGUMENT, "vx_wfile_count: null argument");
    *count = f->tensors.size();
    return VX_OK;
}

vx_status vx_wfile_tensor(const vx_wfile* f, size_t index, char* name, size_t name_cap, uint32_t* ggml_type,
                          uint32_t* n_dims, uint64_t ne[4], uint64_t* bytes) {
    VX_REQUIRE(f, VX_ERR_INVALID_ARGUMENT, "vx_wfile_tensor: null file");
    VX_REQUIRE(index < f->tensors.size(), VX_ERR_OUT_OF_BOUNDS, "tensor %zu of %zu", index, f->tensors.size());
    const TensorInfo& t = f->tensors[index];
    if (name && name_cap) {
        std::strncpy(name, t.name.c_str(), name_cap - 1);
        name[name_cap - 1] = 0;
    }
    if (ggml_type) *ggml_type = t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (ne) std::memcpy(ne, t.ne, sizeof t.ne);
    if (bytes) *bytes = t.bytes;
    return VX_OK;
}

vx_status vx_wfile_find(const vx_wfile* f, const char* name, size_t* index) {
    VX_REQUIRE(f && name && index, VX_ERR_INVALID_ARGUMENT, "vx_wfile_find: null argument");
    for (size_t i = 0; i < f->tensors.size(); ++i)
        if (f->tensors[i].name == name) {
            *index = i;
            return VX_OK;
        }
    return vx::fail(VX_ERR_INVALID_ARGUMENT, "no tensor named '%s'", name);
}

vx_status vx_wfile_data(const vx_wfile* f, size_t index, const void** data, uint64_t* bytes) {
    VX_REQUIRE(f && data, VX_ERR_INVALID_ARGUMENT, "vx_wfile_data: null argument");
    VX_REQUIRE(index < f->tensors.size(), VX_ERR_OUT_OF_BOUNDS, "tensor %zu of %zu", index, f->tensors.size());
    const TensorInfo& t = f->tensors[index];
    VX_REQUIRE(t.bytes != 0, VX_ERR_UNSUPPORTED, "tensor '%s' has GGML type %u, which this library cannot size", t.name.c_str(), t.type);
    *data = f->map + f->data_start + t.offset;
    if (bytes) *bytes = t.bytes;
    return VX_OK;
}

vx_status vx_wfile_load_qweights(vx_context* ctx, const vx_wfile* f, size_t index, vx_qweights** out) {
    VX_REQUIRE(ctx && f && out, VX_ERR_INVALID_ARGUMENT, "vx_wfile_load_qweights: null argument");
    *out = nullptr;
    VX_REQUIRE(index < f->tensors.size(), VX_ERR_OUT_OF_BOUNDS, "tensor %zu of %zu", index, f->tensors.size());
    const TensorInfo& t = f->tensors[index];
    VX_REQUIRE(t.type == GGML_Q4_0 || t.type == GGML_Q8_0, VX_ERR_UNSUPPORTED,
               "tensor '%s' has GGML type %u; Q4_0 (2) and Q8_0 (8) load as quantised weights", t.name.c_str(), t.type);
    VX_REQUIRE(t.n_dims <= 2 || (t.ne[2] == 1 && t.ne[3] == 1), VX_ERR_UNSUPPORTED, "tensor '%s' is not a matrix", t.name.c_str());
    VX_REQUIRE(t.bytes != 0, VX_ERR_INVALID_ARGUMENT, "tensor '%s': %llu columns are not whole blocks", t.name.c_str(),
               (unsigned long long)t.ne[0]);
    // GGML lists the innermost dimension first: ne[0] columns, ne[1] rows
    return vx_qweights_upload(ctx, t.type == GGML_Q4_0 ? VX_Q4_0 : VX_Q8_0, f->map + f->data_start + t.offset,
                              (size_t)t.ne[1], (size_t)t.ne[0], out);
}

}  // extern "C"
