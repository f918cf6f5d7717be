// GGUF container reader for the expert tensors of the path (host code only; no CUDA call in this file).
//
// Mirrors the reference reader's admission rules (src/gguf_reader.cpp:23-99, :330-373; include/strix/gguf_reader.hpp):
// GGUF v3 little-endian only; bounded counts and strings; duplicate metadata keys or tensor names are rejected;
// `general.alignment` (default 32) must be a power of two; the padding before the tensor data is zero bytes; every
// tensor offset is aligned, every data range lies inside the file and no two ranges overlap; a tensor's byte size is
// rows-of-blocks from its type's block geometry, with the innermost dimension divisible by the block length.
// The on-disk layout of the MoE expert tensors - dims [hidden, inter, experts], i.e. [experts][inter][hidden / B] in
// memory order - is what the kernels consume, so loading is: parse, check the shape, copy the byte ranges.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "common.cuh"

namespace b200moe {
namespace {

struct Tensor {
    std::string name;
    u32 n_dims = 0;
    u64 dims[4] = {1, 1, 1, 1};
    u32 type = 0;
    u64 rel = 0, abs = 0, bytes = 0;
};
struct File {
    u32 version = 0;
    u64 file_size = 0, alignment = 32, data_offset = 0;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, size_t> index;
};

constexpr u64 kMaxCount = 1'000'000, kMaxString = 64ull << 20, kMaxArrayElements = 100'000'000;
constexpr u32 kMaxArrayDepth = 8;

// block elements / block bytes of the GGML types this library can meet in an MoE file
bool type_geometry(u32 t, u64* elems, u64* bytes) {
    switch (t) {
        case 0: *elems = 1; *bytes = 4; return true;      // F32
        case 1: *elems = 1; *bytes = 2; return true;      // F16
        case 2: *elems = 32; *bytes = 18; return true;    // Q4_0
        case 3: *elems = 32; *bytes = 20; return true;    // Q4_1
        case 6: *elems = 32; *bytes = 22; return true;    // Q5_0
        case 7: *elems = 32; *bytes = 24; return true;    // Q5_1
        case 8: *elems = 32; *bytes = 34; return true;    // Q8_0
        case 9: *elems = 32; *bytes = 36; return true;    // Q8_1
        case 10: *elems = 256; *bytes = 84; return true;  // Q2_K
        case 11: *elems = 256; *bytes = 110; return true; // Q3_K
        case 12: *elems = 256; *bytes = 144; return true; // Q4_K
        case 13: *elems = 256; *bytes = 176; return true; // Q5_K
        case 14: *elems = 256; *bytes = 210; return true; // Q6_K
        case 15: *elems = 256; *bytes = 292; return true; // Q8_K
        case 24: *elems = 1; *bytes = 1; return true;     // I8
        case 25: *elems = 1; *bytes = 2; return true;     // I16
        case 26: *elems = 1; *bytes = 4; return true;     // I32
        case 27: *elems = 1; *bytes = 8; return true;     // I64
        case 28: *elems = 1; *bytes = 8; return true;     // F64
        case 30: *elems = 1; *bytes = 2; return true;     // BF16
        default: return false;
    }
}

struct Parser {
    FILE* f;
    u64 size, pos = 0;
    std::string error;

    bool fail_(const char* what) { if (error.empty()) error = what; return false; }
    bool bytes(void* dst, u64 n) {
        if (n > size - pos) return fail_("unexpected end of file");
        if (n && fread(dst, 1, n, f) != n) return fail_("read error");
        pos += n;
        return true;
    }
    template <class T> bool num(T* v) {
        unsigned char b[sizeof(T)];
        if (!bytes(b, sizeof(T))) return false;
        u64 x = 0;
        for (size_t i = 0; i < sizeof(T); ++i) x |= u64(b[i]) << (8 * i);
        *v = static_cast<T>(x);
        return true;
    }
    bool str(std::string* s) {
        u64 n;
        if (!num(&n)) return false;
        if (n > kMaxString) return fail_("string exceeds the limit");
        s->assign(n, '\0');
        return bytes(s->data(), n);
    }
    static u64 scalar_bytes(u32 t) {
        switch (t) {
            case 0: case 1: case 7: return 1;
            case 2: case 3: return 2;
            case 4: case 5: case 6: return 4;
            case 10: case 11: case 12: return 8;
            default: return 0;
        }
    }
    bool skip(u64 n) {
        if (n > size - pos) return fail_("unexpected end of file");
        if (fseeko(f, static_cast<off_t>(n), SEEK_CUR) != 0) return fail_("seek error");
        pos += n;
        return true;
    }
    // Reads one value of type t; *as_u64 receives it when it is an unsigned / signed integer scalar.
    bool value(u32 t, u32 depth, u64* total_elements, bool* is_int, u64* as_u64) {
        *is_int = false;
        if (t == 8) { std::string s; return str(&s); }
        if (t == 9) {
            if (depth >= kMaxArrayDepth) return fail_("array nesting exceeds the limit");
            u32 et; u64 n;
            if (!num(&et) || !num(&n)) return false;
            *total_elements += n;
            if (*total_elements > kMaxArrayElements) return fail_("array elements exceed the limit");
            if (const u64 sb = scalar_bytes(et)) {
                if (n > (size - pos) / sb) return fail_("unexpected end of file");
                return skip(n * sb);
            }
            if (et != 8 && et != 9) return fail_("unknown metadata value type");
            for (u64 i = 0; i < n; ++i) { bool ii; u64 vv; if (!value(et, depth + 1, total_elements, &ii, &vv)) return false; }
            return true;
        }
        const u64 sb = scalar_bytes(t);
        if (!sb) return fail_("unknown metadata value type");
        unsigned char b[8] = {};
        if (!bytes(b, sb)) return false;
        if (t == 0 || t == 2 || t == 4 || t == 10) {  // the unsigned integer types (uint8 / 16 / 32 / 64)
            u64 x = 0;
            for (u64 i = 0; i < sb; ++i) x |= u64(b[i]) << (8 * i);
            *is_int = true;
            *as_u64 = x;
        }
        return true;
    }
};

// Metadata keys (src/gguf_reader.cpp:131-135, :297-313): at most 65,535 bytes of [a-z0-9_.], no leading, trailing or
// doubled dot.
bool valid_key(const std::string& key) {
    if (key.empty() || key.size() > 65535 || key.front() == '.' || key.back() == '.') return false;
    bool previous_dot = false;
    for (const char c : key) {
        const bool ok = (c >= 'a' && c <= 'z') || (c >= '0' && c <= '9') || c == '_' || c == '.';
        if (!ok || (c == '.' && previous_dot)) return false;
        previous_dot = c == '.';
    }
    return true;
}

bool mul_ok(u64 a, u64 b, u64* out) {
    if (a != 0 && b > std::numeric_limits<u64>::max() / a) return false;
    *out = a * b;
    return true;
}

int parse(const char* path, File* out) {
    FILE* f = fopen(path, "rb");
    if (!f) return fail(B200MOE_ERR_INVALID_ARGUMENT, "gguf: cannot open %s", path);
    Parser p{f, 0};
    fseeko(f, 0, SEEK_END);
    p.size = static_cast<u64>(ftello(f));
    fseeko(f, 0, SEEK_SET);
    out->file_size = p.size;
    auto bad = [&](const char* what) {
        fclose(f);
        return fail(B200MOE_ERR_INVALID_ARGUMENT, "gguf: %s", p.error.empty() ? what : p.error.c_str());
    };
    char magic[4];
    if (!p.bytes(magic, 4) || std::memcmp(magic, "GGUF", 4) != 0) return bad("invalid GGUF magic");
    u64 n_tensors, n_kv;
    if (!p.num(&out->version)) return bad("truncated header");
    if (out->version != 3) return bad("only GGUF v3 little-endian is supported");
    if (!p.num(&n_tensors) || !p.num(&n_kv)) return bad("truncated header");
    if (n_tensors > kMaxCount || n_kv > kMaxCount) return bad("tensor or metadata count exceeds the limit");
    std::unordered_set<std::string> keys;
    u64 total_elements = 0;
    for (u64 i = 0; i < n_kv; ++i) {
        std::string key;
        u32 t;
        if (!p.str(&key) || !p.num(&t)) return bad("truncated metadata");
        if (!valid_key(key)) return bad("invalid GGUF metadata key");
        if (!keys.insert(key).second) return bad("duplicate GGUF metadata key");
        bool is_int; u64 v = 0;
        if (!p.value(t, 0, &total_elements, &is_int, &v)) return bad("bad metadata value");
        if (key == "general.alignment") {
            // src/gguf_reader.cpp:271-282: an unsigned integer, a non-zero multiple of 8
            if (!is_int) return bad("general.alignment must be an unsigned integer");
            if (v == 0 || v % 8 != 0) return bad("general.alignment must be a non-zero multiple of 8");
            out->alignment = v;
        }
    }
    out->tensors.resize(n_tensors);
    for (u64 i = 0; i < n_tensors; ++i) {
        Tensor& t = out->tensors[i];
        if (!p.str(&t.name) || !p.num(&t.n_dims)) return bad("truncated tensor info");
        if (t.n_dims == 0 || t.n_dims > 4) return bad("tensor rank must be 1..4");
        for (u32 d = 0; d < t.n_dims; ++d) if (!p.num(&t.dims[d])) return bad("truncated tensor info");
        if (!p.num(&t.type) || !p.num(&t.rel)) return bad("truncated tensor info");
        if (!out->index.emplace(t.name, i).second) return bad("duplicate GGUF tensor name");
    }
    const u64 rem = p.pos % out->alignment;
    out->data_offset = rem ? p.pos + (out->alignment - rem) : p.pos;
    if (out->data_offset > p.size) return bad("aligned tensor-data offset exceeds file size");
    while (p.pos < out->data_offset) {
        unsigned char z;
        if (!p.bytes(&z, 1)) return bad("truncated padding");
        if (z != 0) return bad("GGUF padding must contain zero bytes");
    }
    for (Tensor& t : out->tensors) {
        if (t.rel % out->alignment != 0) return bad("tensor offset is not aligned");
        if (t.rel > p.size - out->data_offset) return bad("tensor offset exceeds file size");
        t.abs = out->data_offset + t.rel;
        u64 be, bb;
        if (!type_geometry(t.type, &be, &bb)) return bad("GGML tensor type has no pinned storage geometry");
        if (t.dims[0] % be != 0) return bad("tensor row is not divisible by its quantization block size");
        u64 bytes = 0;
        if (!mul_ok(t.dims[0] / be, bb, &bytes)) return bad("tensor-size overflow");
        for (u32 d = 1; d < t.n_dims; ++d) if (!mul_ok(bytes, t.dims[d], &bytes)) return bad("tensor-size overflow");
        t.bytes = bytes;
        if (bytes > p.size - t.abs) return bad("tensor data range exceeds file size");
    }
    std::vector<const Tensor*> order;
    for (const Tensor& t : out->tensors) order.push_back(&t);
    std::sort(order.begin(), order.end(), [](const Tensor* a, const Tensor* b) { return a->abs < b->abs; });
    for (size_t i = 1; i < order.size(); ++i)
        if (order[i]->abs < order[i - 1]->abs + order[i - 1]->bytes) return bad("GGUF tensor data ranges overlap");
    fclose(f);
    return B200MOE_OK;
}

void fill(const Tensor& t, b200moe_gguf_tensor_info* o) {
    o->name = t.name.c_str();
    o->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) o->dims[d] = t.dims[d];
    o->ggml_type = t.type;
    o->offset = t.abs;
    o->bytes = t.bytes;
}

}  // namespace
}  // namespace b200moe

extern "C" {

using namespace b200moe;

int b200moe_gguf_open(const char* path, void** file) {
    B200_REQUIRE(path && file, "gguf_open: path / file are null");
    File* f = new File();
    if (int rc = parse(path, f)) { delete f; return rc; }
    *file = f;
    return B200MOE_OK;
}
void b200moe_gguf_close(void* file) { delete static_cast<File*>(file); }
uint64_t b200moe_gguf_tensor_count(const void* file) { return file ? static_cast<const File*>(file)->tensors.size() : 0; }
uint64_t b200moe_gguf_data_offset(const void* file) { return file ? static_cast<const File*>(file)->data_offset : 0; }
uint64_t b200moe_gguf_alignment(const void* file) { return file ? static_cast<const File*>(file)->alignment : 0; }

int b200moe_gguf_tensor_at(const void* file, uint64_t index, b200moe_gguf_tensor_info* out) {
    B200_REQUIRE(file && out, "gguf_tensor_at: file / out are null");
    const File* f = static_cast<const File*>(file);
    B200_REQUIRE(index < f->tensors.size(), "gguf_tensor_at: index %llu of %zu", (unsigned long long)index, f->tensors.size());
    fill(f->tensors[index], out);
    return B200MOE_OK;
}
int b200moe_gguf_find(const void* file, const char* name, b200moe_gguf_tensor_info* out) {
    B200_REQUIRE(file && name && out, "gguf_find: file / name / out are null");
    const File* f = static_cast<const File*>(file);
    const auto it = f->index.find(name);
    if (it == f->index.end()) return fail(B200MOE_ERR_UNSUPPORTED, "gguf: no tensor named %s", name);
    fill(f->tensors[it->second], out);
    return B200MOE_OK;
}

int b200moe_gguf_find_moe_layer(const void* file, uint32_t layer, b200moe_gguf_moe_layer* out) {
    B200_REQUIRE(file && out, "gguf_moe_layer: file / out are null");
    char name[96];
    const char* parts[4] = {"ffn_gate_exps", "ffn_up_exps", "ffn_down_exps", "ffn_gate_inp"};
    b200moe_gguf_tensor_info* dst[4] = {&out->gate, &out->up, &out->down, &out->router};
    for (int i = 0; i < 4; ++i) {
        snprintf(name, sizeof name, "blk.%u.%s.weight", layer, parts[i]);
        if (int rc = b200moe_gguf_find(file, name, dst[i])) return rc;
    }
    const b200moe_gguf_tensor_info &g = out->gate, &u = out->up, &d = out->down, &r = out->router;
    B200_REQUIRE(g.n_dims == 3 && u.n_dims == 3 && d.n_dims == 3 && r.n_dims == 2, "gguf layer %u: expert tensors must have 3 dimensions, the router 2", layer);
    B200_REQUIRE(g.ggml_type == u.ggml_type && g.dims[0] == u.dims[0] && g.dims[1] == u.dims[1] && g.dims[2] == u.dims[2],
                 "gguf layer %u: gate and up tensors differ in type or shape", layer);
    B200_REQUIRE(d.dims[0] == g.dims[1] && d.dims[1] == g.dims[0] && d.dims[2] == g.dims[2],
                 "gguf layer %u: down is not [inter, hidden, experts] of gate's [hidden, inter, experts]", layer);
    B200_REQUIRE(r.ggml_type == 0 && r.dims[0] == g.dims[0] && r.dims[1] == g.dims[2], "gguf layer %u: the router must be F32 [hidden, experts]", layer);
    B200_REQUIRE((g.ggml_type == B200MOE_TYPE_Q8_0 || g.ggml_type == B200MOE_TYPE_Q2_K || g.ggml_type == B200MOE_TYPE_Q4_K || g.ggml_type == B200MOE_TYPE_Q5_K) &&
                     (d.ggml_type == B200MOE_TYPE_Q8_0 || d.ggml_type == B200MOE_TYPE_Q2_K || d.ggml_type == B200MOE_TYPE_Q4_K || d.ggml_type == B200MOE_TYPE_Q5_1),
                 "gguf layer %u: gate / up must be Q8_0, Q2_K, Q4_K or Q5_K and down Q8_0, Q2_K, Q4_K or Q5_1 (types %u / %u)", layer, g.ggml_type, d.ggml_type);
    B200_REQUIRE(g.dims[0] <= 0xffffffffull && g.dims[1] <= 0xffffffffull && g.dims[2] <= 0xffffffffull, "gguf layer %u: a dimension exceeds 32 bits", layer);
    out->shape.hidden = static_cast<u32>(g.dims[0]);
    out->shape.inter = static_cast<u32>(g.dims[1]);
    out->shape.experts = static_cast<u32>(g.dims[2]);
    out->shape.top_k = 0;  // routing metadata is the caller's (it is model metadata, not tensor geometry)
    out->shape.gate_type = g.ggml_type;
    out->shape.down_type = d.ggml_type;
    out->shape.limit = std::numeric_limits<float>::infinity();
    return B200MOE_OK;
}

}  // extern "C"
