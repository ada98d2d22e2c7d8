// Checkpoint front-end (host code only): a memory-mapped safetensors reader and the assembly of
// one bitsandbytes 4-bit weight into an AilaNf4WeightDesc.
//
// Role in the reference: LoadSafetensors (src/utils/SafeTensors.cpp:154-222) maps a file and
// uploads every tensor; LoadBnb4BitWeightRef (:370-489) then collects the side tensors of one
// weight by name, parses the quant_state JSON blob (:281-334) and checks the invariants that
// the kernels rely on. Here the descriptor points straight into the mapping (host pointers), so
// aila_nf4_linear_create uploads a weight directly into its unit-stream layout and no raw copy
// of the checkpoint tensors ever lives on the GPU.
//
// File format: 8-byte little-endian header length N, N bytes of JSON
// {"<name>": {"dtype": "U8", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__":
// {...}}, then the tensor bytes; offsets are relative to the end of the header.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <new>
#include <set>
#include <string>
#include <vector>

#include "nf4_internal.h"

namespace {

// ---------------------------------------------------------------------------------------------
// Minimal JSON reader (objects, arrays, strings, numbers, true/false/null).
// ---------------------------------------------------------------------------------------------
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool integral = false;
    long long i = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    const Json* find(const char* key) const {
        if (kind != Object) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

struct JsonParser {
    const char* p;
    const char* end;
    std::string error;
    int depth = 0;

    bool fail(const char* what) {
        if (error.empty()) error = what;
        return false;
    }
    void skip_ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    bool parse_string(std::string& out) {
        if (p >= end || *p != '"') return fail("expected a string");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            unsigned char c = (unsigned char)*p++;
            if (c == '\\') {
                if (p >= end) return fail("unterminated escape");
                char e = *p++;
                switch (e) {
                    case '"': out.push_back('"'); break;
                    case '\\': out.push_back('\\'); break;
                    case '/': out.push_back('/'); break;
                    case 'b': out.push_back('\b'); break;
                    case 'f': out.push_back('\f'); break;
                    case 'n': out.push_back('\n'); break;
                    case 'r': out.push_back('\r'); break;
                    case 't': out.push_back('\t'); break;
                    case 'u': {
                        if (end - p < 4) return fail("short \\u escape");
                        unsigned cp = 0;
                        for (int k = 0; k < 4; ++k) {
                            char h = *p++;
                            cp <<= 4;
                            if (h >= '0' && h <= '9') cp |= (unsigned)(h - '0');
                            else if (h >= 'a' && h <= 'f') cp |= (unsigned)(h - 'a' + 10);
                            else if (h >= 'A' && h <= 'F') cp |= (unsigned)(h - 'A' + 10);
                            else return fail("bad \\u escape");
                        }
                        // UTF-8 encode the basic-plane code point (surrogate pairs are kept as
                        // two three-byte sequences; tensor names do not use them)
                        if (cp < 0x80) out.push_back((char)cp);
                        else if (cp < 0x800) {
                            out.push_back((char)(0xC0 | (cp >> 6)));
                            out.push_back((char)(0x80 | (cp & 0x3F)));
                        } else {
                            out.push_back((char)(0xE0 | (cp >> 12)));
                            out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
                            out.push_back((char)(0x80 | (cp & 0x3F)));
                        }
                        break;
                    }
                    default: return fail("unknown escape");
                }
            } else {
                out.push_back((char)c);
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool parse_value(Json& v) {
        if (++depth > 64) return fail("nesting too deep");
        skip_ws();
        if (p >= end) return fail("unexpected end of JSON");
        bool ok = true;
        const char c = *p;
        if (c == '{') {
            v.kind = Json::Object;
            ++p;
            skip_ws();
            if (p < end && *p == '}') {
                ++p;
            } else {
                while (ok) {
                    skip_ws();
                    std::string key;
                    if (!parse_string(key)) { ok = false; break; }
                    skip_ws();
                    if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
                    ++p;
                    v.obj.emplace_back(std::move(key), Json());
                    if (!parse_value(v.obj.back().second)) { ok = false; break; }
                    skip_ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == '}') { ++p; break; }
                    ok = fail("expected ',' or '}'");
                }
            }
        } else if (c == '[') {
            v.kind = Json::Array;
            ++p;
            skip_ws();
            if (p < end && *p == ']') {
                ++p;
            } else {
                while (ok) {
                    v.arr.emplace_back();
                    if (!parse_value(v.arr.back())) { ok = false; break; }
                    skip_ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == ']') { ++p; break; }
                    ok = fail("expected ',' or ']'");
                }
            }
        } else if (c == '"') {
            v.kind = Json::String;
            ok = parse_string(v.str);
        } else if (c == 't' && end - p >= 4 && std::strncmp(p, "true", 4) == 0) {
            v.kind = Json::Bool; v.b = true; p += 4;
        } else if (c == 'f' && end - p >= 5 && std::strncmp(p, "false", 5) == 0) {
            v.kind = Json::Bool; v.b = false; p += 5;
        } else if (c == 'n' && end - p >= 4 && std::strncmp(p, "null", 4) == 0) {
            v.kind = Json::Null; p += 4;
        } else if (c == '-' || (c >= '0' && c <= '9')) {
            const char* s = p;
            bool is_int = true;
            if (*p == '-') ++p;
            while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' ||
                               *p == '+' || *p == '-')) {
                if (*p == '.' || *p == 'e' || *p == 'E') is_int = false;
                ++p;
            }
            std::string text(s, p);
            v.kind = Json::Number;
            v.num = std::strtod(text.c_str(), nullptr);
            v.integral = is_int;
            if (is_int) {
                errno = 0;
                v.i = std::strtoll(text.c_str(), nullptr, 10);
                if (errno != 0) v.integral = false;
            }
        } else {
            ok = fail("unexpected character in JSON");
        }
        --depth;
        return ok;
    }
};

bool parse_json(const char* text, size_t n, Json& out, std::string& error) {
    JsonParser ps{text, text + n, std::string()};
    if (!ps.parse_value(out)) {
        error = ps.error;
        return false;
    }
    ps.skip_ws();
    // trailing NUL or space padding is tolerated (the header may be padded for alignment)
    while (ps.p < ps.end && (*ps.p == '\0' || *ps.p == ' ')) ++ps.p;
    if (ps.p != ps.end) {
        error = "trailing characters after JSON value";
        return false;
    }
    return true;
}

struct StTensor {
    int dtype = AILA_ST_DTYPE_UNKNOWN;
    std::vector<int64_t> shape;
    size_t begin = 0, end = 0;  // byte range inside the data section
};

int dtype_from_string(const std::string& s) {
    if (s == "U8") return AILA_ST_U8;
    if (s == "I8") return AILA_ST_I8;
    if (s == "F16") return AILA_ST_F16;
    if (s == "BF16") return AILA_ST_BF16;
    if (s == "F32") return AILA_ST_F32;
    if (s == "F64") return AILA_ST_F64;
    if (s == "I32") return AILA_ST_I32;
    if (s == "I64") return AILA_ST_I64;
    if (s == "BOOL") return AILA_ST_BOOL;
    return AILA_ST_DTYPE_UNKNOWN;
}

int dtype_size(int dt) {
    switch (dt) {
        case AILA_ST_U8: case AILA_ST_I8: case AILA_ST_BOOL: return 1;
        case AILA_ST_F16: case AILA_ST_BF16: return 2;
        case AILA_ST_F32: case AILA_ST_I32: return 4;
        case AILA_ST_F64: case AILA_ST_I64: return 8;
        default: return 0;
    }
}

}  // namespace

struct AilaStFile {
    std::string path;
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t map_bytes = 0;
    const uint8_t* data = nullptr;  // start of the tensor bytes
    size_t data_bytes = 0;
    std::vector<std::string> names;  // file order
    std::map<std::string, StTensor> tensors;
};

using nf4::fail;

namespace {

// Element count of a tensor from an untrusted header; -1 when a dimension is negative or the
// product does not fit 63 bits.
int64_t numel_of(const StTensor& t) {
    int64_t n = 1;
    for (int64_t d : t.shape)
        if (d < 0 || __builtin_mul_overflow(n, d, &n)) return -1;
    return n;
}

const StTensor* find_tensor(const AilaStFile* f, const std::string& name) {
    auto it = f->tensors.find(name);
    return it == f->tensors.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

AILA_NF4_API AilaNf4Status aila_st_open(const char* path, AilaStFile** out) {
    if (!path || !out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    *out = nullptr;
    std::unique_ptr<AilaStFile> f(new (std::nothrow) AilaStFile());
    if (!f) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    f->path = path;
    f->fd = ::open(path, O_RDONLY | O_CLOEXEC);
    if (f->fd < 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    std::string("cannot open safetensors file ") + path + ": " + std::strerror(errno));
    auto bail = [&](const std::string& why) {
        if (f->map) ::munmap(const_cast<uint8_t*>(f->map), f->map_bytes);
        ::close(f->fd);
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "safetensors file " + f->path + ": " + why);
    };
    struct stat stbuf;
    if (::fstat(f->fd, &stbuf) != 0) return bail("fstat failed");
    f->map_bytes = (size_t)stbuf.st_size;
    if (f->map_bytes < 8) return bail("shorter than its 8-byte header length");
    void* m = ::mmap(nullptr, f->map_bytes, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) {
        f->map = nullptr;
        return bail(std::string("mmap failed: ") + std::strerror(errno));
    }
    f->map = static_cast<const uint8_t*>(m);
    uint64_t header_len = 0;
    for (int i = 0; i < 8; ++i) header_len |= (uint64_t)f->map[i] << (8 * i);
    if (header_len == 0 || header_len > f->map_bytes - 8 || header_len > (1ull << 30))
        return bail("header length " + std::to_string(header_len) + " does not fit the file");
    Json root;
    std::string jerr;
    if (!parse_json(reinterpret_cast<const char*>(f->map + 8), (size_t)header_len, root, jerr))
        return bail("header is not valid JSON (" + jerr + ")");
    if (root.kind != Json::Object) return bail("header is not a JSON object");
    f->data = f->map + 8 + header_len;
    f->data_bytes = f->map_bytes - 8 - (size_t)header_len;
    for (const auto& kv : root.obj) {
        if (kv.first == "__metadata__") continue;
        const Json& e = kv.second;
        const Json* dt = e.find("dtype");
        const Json* sh = e.find("shape");
        const Json* off = e.find("data_offsets");
        if (!dt || dt->kind != Json::String || !sh || sh->kind != Json::Array || !off ||
            off->kind != Json::Array || off->arr.size() != 2)
            return bail("entry '" + kv.first + "' lacks dtype, shape or data_offsets");
        StTensor t;
        t.dtype = dtype_from_string(dt->str);
        for (const Json& d : sh->arr) {
            if (d.kind != Json::Number || !d.integral || d.i < 0)
                return bail("entry '" + kv.first + "' has a non-integer dimension");
            t.shape.push_back(d.i);
        }
        if (off->arr[0].kind != Json::Number || off->arr[1].kind != Json::Number ||
            !off->arr[0].integral || !off->arr[1].integral || off->arr[0].i < 0 ||
            off->arr[1].i < off->arr[0].i || (uint64_t)off->arr[1].i > f->data_bytes)
            return bail("entry '" + kv.first + "' has data_offsets outside the file");
        t.begin = (size_t)off->arr[0].i;
        t.end = (size_t)off->arr[1].i;
        const int es = dtype_size(t.dtype);
        const int64_t count = numel_of(t);
        if (count < 0) return bail("entry '" + kv.first + "': shape overflows");
        if (es > 0 && ((uint64_t)count > f->data_bytes || (uint64_t)count * (uint64_t)es != (uint64_t)(t.end - t.begin)))
            return bail("entry '" + kv.first + "': shape and dtype do not match its byte range");
        if (f->tensors.count(kv.first)) return bail("duplicate entry '" + kv.first + "'");
        f->names.push_back(kv.first);
        f->tensors.emplace(kv.first, std::move(t));
    }
    *out = f.release();
    return AILA_NF4_OK;
}

AILA_NF4_API void aila_st_close(AilaStFile* f) {
    if (!f) return;
    if (f->map) ::munmap(const_cast<uint8_t*>(f->map), f->map_bytes);
    if (f->fd >= 0) ::close(f->fd);
    delete f;
}

AILA_NF4_API int64_t aila_st_tensor_count(const AilaStFile* f) {
    return f ? (int64_t)f->names.size() : 0;
}

AILA_NF4_API const char* aila_st_tensor_name(const AilaStFile* f, int64_t index) {
    if (!f || index < 0 || index >= (int64_t)f->names.size()) return nullptr;
    return f->names[(size_t)index].c_str();
}

AILA_NF4_API AilaNf4Status aila_st_find(const AilaStFile* f, const char* name,
                                        AilaStTensorView* out) {
    if (!f || !name || !out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    const StTensor* t = find_tensor(f, name);
    if (!t) return fail(AILA_NF4_NOT_APPLICABLE, std::string("no tensor named ") + name);
    if (t->shape.size() > AILA_ST_MAX_RANK)
        return fail(AILA_NF4_ERR_UNSUPPORTED, std::string("tensor rank above 8: ") + name);
    std::memset(out, 0, sizeof(*out));
    out->dtype = t->dtype;
    out->rank = (int32_t)t->shape.size();
    for (size_t i = 0; i < t->shape.size(); ++i) out->shape[i] = t->shape[i];
    out->data = f->data + t->begin;
    out->nbytes = (int64_t)(t->end - t->begin);
    return AILA_NF4_OK;
}

}  // extern "C"

namespace {

// A tensor and the data section of the file that holds it.
struct Found {
    const StTensor* t = nullptr;
    const uint8_t* data = nullptr;
    const StTensor* operator->() const { return t; }
    const StTensor& operator*() const { return *t; }
    explicit operator bool() const { return t != nullptr; }
    bool operator!() const { return t == nullptr; }
    const uint8_t* bytes() const { return data + t->begin; }
};

// Same tensor names, dtype rules and size invariants as LoadBnb4BitWeightRef
// (src/utils/SafeTensors.cpp:370-489). `lookup` finds a tensor by name in one file or in the
// shards of a directory.
template <typename Lookup>
AilaNf4Status load_bnb4_weight(Lookup&& lookup, const char* name, int device, AilaNf4WeightDesc* out) {
    std::memset(out, 0, sizeof(*out));
    const std::string w = name;
    const Found packed = lookup(w);
    if (!packed)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Missing bitsandbytes packed weight tensor: " + w);
    const Found absmax = lookup(w + ".absmax");
    const Found qmap = lookup(w + ".quant_map");
    const Found state = lookup(w + ".quant_state.bitsandbytes__nf4");
    const Found nabs = lookup(w + ".nested_absmax");
    const Found nmap = lookup(w + ".nested_quant_map");
    if (!absmax || !qmap || !state)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "Missing required bitsandbytes side tensors for weight: " + w);
    if (packed->dtype != AILA_ST_U8)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes packed weight must be uint8: " + w);
    if (qmap->dtype != AILA_ST_F32)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes quant_map must be float32: " + w + ".quant_map");
    if (state->dtype != AILA_ST_U8)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes packed quant_state must be uint8: " + w);
    if (absmax->dtype != AILA_ST_U8 && absmax->dtype != AILA_ST_F32)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes absmax must be uint8 or float32: " + w + ".absmax");

    // quant_state JSON: quant_type, dtype, blocksize, shape, and for double quantisation
    // nested_blocksize, nested_dtype, nested_offset (any of the three marks the state nested)
    Json qs;
    std::string jerr;
    if (!parse_json(reinterpret_cast<const char*>(state.bytes()), state->end - state->begin, qs, jerr) ||
        qs.kind != Json::Object)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "parse bitsandbytes quant_state failed: " + jerr);
    const Json* quant_type = qs.find("quant_type");
    const Json* blocksize = qs.find("blocksize");
    const Json* shape = qs.find("shape");
    if (!blocksize || blocksize->kind != Json::Number || !blocksize->integral)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes quant_state is missing blocksize");
    if (!shape || shape->kind != Json::Array)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes quant_state is missing shape");
    std::vector<int64_t> dims;
    for (const Json& d : shape->arr) {
        if (d.kind != Json::Number || !d.integral)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes quant_state shape contains a non-integer value");
        dims.push_back(d.i);
    }
    bool nested = false;
    long long nested_blocksize = 0;
    float nested_offset = 0.0f;
    if (const Json* nb = qs.find("nested_blocksize"); nb && nb->kind == Json::Number && nb->integral) {
        nested = true;
        nested_blocksize = nb->i;
    }
    if (const Json* nd = qs.find("nested_dtype"); nd && nd->kind == Json::String && !nd->str.empty())
        nested = true;
    if (const Json* no = qs.find("nested_offset"); no && no->kind == Json::Number) {
        nested = true;
        nested_offset = (float)no->num;
    }
    if (dims.size() != 2)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Invalid bitsandbytes weight view: " + w);
    if (!quant_type || quant_type->kind != Json::String || quant_type->str != "nf4")
        return fail(AILA_NF4_ERR_UNSUPPORTED, "Only NF4 bitsandbytes weights are supported: " + w);
    if (blocksize->i <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes blocksize must be positive: " + w);
    int64_t logical = 0;
    if (dims[0] <= 0 || dims[1] <= 0 || dims[0] >= (int64_t(1) << 27) || dims[1] >= (int64_t(1) << 27) ||
        __builtin_mul_overflow(dims[0], dims[1], &logical) || logical <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes logical weight shape is invalid: " + w);
    if (numel_of(*packed) * 2 != logical)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "bitsandbytes packed weight size does not match logical shape: " + w);
    const int64_t blocks = (logical + blocksize->i - 1) / blocksize->i;
    if (numel_of(*absmax) != blocks)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "bitsandbytes absmax length does not match block count: " + w);
    if (numel_of(*qmap) < 16)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "bitsandbytes quant_map must contain at least 16 entries: " + w);
    if (nested) {
        if (!nabs || !nmap)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested quantization tensors are missing: " + w);
        if (nabs->dtype != AILA_ST_F32 || nmap->dtype != AILA_ST_F32)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes nested tensors must be float32: " + w);
        if (nested_blocksize <= 0)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes nested blocksize must be positive: " + w);
        const int64_t nblocks = (blocks + nested_blocksize - 1) / nested_blocksize;
        if (numel_of(*nabs) != nblocks)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested_absmax length does not match nested block count: " + w);
        if (absmax->dtype != AILA_ST_U8)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested absmax must be uint8 codes: " + w);
        if (numel_of(*nmap) < 256)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested_quant_map must contain at least 256 entries: " + w);
    } else if (absmax->dtype != AILA_ST_F32) {
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Non-nested bitsandbytes absmax must be float32: " + w);
    }
    out->out_features = dims[0];
    out->in_features = dims[1];
    out->blocksize = (int32_t)blocksize->i;
    out->nested = nested ? 1 : 0;
    out->nested_blocksize = (int32_t)nested_blocksize;
    out->nested_offset = nested_offset;
    out->packed_weight = packed.bytes();
    out->absmax = absmax.bytes();
    out->quant_map = reinterpret_cast<const float*>(qmap.bytes());
    out->nested_absmax = nested ? reinterpret_cast<const float*>(nabs.bytes()) : nullptr;
    out->nested_quant_map = nested ? reinterpret_cast<const float*>(nmap.bytes()) : nullptr;
    out->nested_absmax_count = nested ? numel_of(*nabs) : 0;
    out->pointers_on_device = 0;
    out->device = device;
    return AILA_NF4_OK;
}

Found find_in(const AilaStFile* f, const std::string& name) {
    Found r;
    r.t = find_tensor(f, name);
    r.data = f->data;
    return r;
}

bool file_exists(const std::string& path) {
    struct stat st;
    return ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

}  // namespace

// A model directory: model.safetensors, or the shards named by model.safetensors.index.json
// (LoadModelWeightsFromDir, src/utils/SafeTensors.cpp:491-535; parse_sharded_safetensors_index,
// :336-366). Shards are opened in sorted name order; a tensor present in several shards is taken
// from the last one, as the reference's merge does.
struct AilaStDir {
    std::vector<AilaStFile*> files;
};

extern "C" {

AILA_NF4_API AilaNf4Status aila_st_load_bnb4_weight(const AilaStFile* f, const char* name,
                                                    int device, AilaNf4WeightDesc* out) {
    if (!f || !name || !out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    return load_bnb4_weight([f](const std::string& n) { return find_in(f, n); }, name, device, out);
}

AILA_NF4_API void aila_st_dir_close(AilaStDir* d) {
    if (!d) return;
    for (AilaStFile* f : d->files) aila_st_close(f);
    delete d;
}

AILA_NF4_API AilaNf4Status aila_st_dir_open(const char* model_dir, AilaStDir** out) {
    if (!model_dir || !out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    *out = nullptr;
    const std::string dir = model_dir;
    std::vector<std::string> shards;
    if (file_exists(dir + "/model.safetensors")) {
        shards.push_back("model.safetensors");
    } else {
        const std::string index = dir + "/model.safetensors.index.json";
        if (!file_exists(index))
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "No model.safetensors or model.safetensors.index.json found in: " + dir);
        std::string text;
        {
            FILE* fp = std::fopen(index.c_str(), "rb");
            if (fp) {
                char buf[65536];
                size_t n;
                while ((n = std::fread(buf, 1, sizeof(buf), fp)) > 0) text.append(buf, n);
                std::fclose(fp);
            }
        }
        if (text.empty())
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Empty or unreadable safetensors index: " + index);
        Json root;
        std::string jerr;
        if (!parse_json(text.data(), text.size(), root, jerr) || root.kind != Json::Object)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Invalid safetensors index: " + (jerr.empty() ? "not a JSON object" : jerr));
        const Json* wm = root.find("weight_map");
        if (!wm) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Invalid safetensors index: missing weight_map");
        if (wm->kind != Json::Object)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Invalid safetensors index: weight_map is not an object");
        std::set<std::string> unique;
        for (const auto& kv : wm->obj)
            if (kv.second.kind == Json::String) unique.insert(kv.second.str);
        shards.assign(unique.begin(), unique.end());  // (a set iterates in sorted order)
        if (shards.empty()) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "No shard entries found in: " + index);
    }
    AilaStDir* d = new (std::nothrow) AilaStDir();
    if (!d) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    for (const std::string& name : shards) {
        const std::string path = dir + "/" + name;
        if (name.find("..") != std::string::npos || name.find('/') != std::string::npos || !file_exists(path)) {
            aila_st_dir_close(d);
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Missing safetensors shard: " + path);
        }
        AilaStFile* f = nullptr;
        const AilaNf4Status st = aila_st_open(path.c_str(), &f);
        if (st != AILA_NF4_OK) {
            aila_st_dir_close(d);
            return st;
        }
        d->files.push_back(f);
    }
    *out = d;
    return AILA_NF4_OK;
}

AILA_NF4_API int64_t aila_st_dir_shard_count(const AilaStDir* d) { return d ? (int64_t)d->files.size() : 0; }

AILA_NF4_API const AilaStFile* aila_st_dir_shard(const AilaStDir* d, int64_t index) {
    if (!d || index < 0 || index >= (int64_t)d->files.size()) return nullptr;
    return d->files[(size_t)index];
}

AILA_NF4_API AilaNf4Status aila_st_dir_find(const AilaStDir* d, const char* name, AilaStTensorView* out) {
    if (!d || !name || !out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    for (size_t i = d->files.size(); i-- > 0;)
        if (find_tensor(d->files[i], name)) return aila_st_find(d->files[i], name, out);
    return fail(AILA_NF4_NOT_APPLICABLE, std::string("no tensor named ") + name);
}

AILA_NF4_API AilaNf4Status aila_st_dir_load_bnb4_weight(const AilaStDir* d, const char* name, int device,
                                                        AilaNf4WeightDesc* out) {
    if (!d || !name || !out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    return load_bnb4_weight(
        [d](const std::string& n) {
            for (size_t i = d->files.size(); i-- > 0;) {
                const Found r = find_in(d->files[i], n);
                if (r) return r;
            }
            return Found();
        },
        name, device, out);
}

}  // extern "C"
