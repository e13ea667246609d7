// Checkpoint side of the quantized operators (host code only): a reader for .safetensors
// files and Hugging Face shard indexes, a writer, the host int4 quantizer, names of derived
// (packed) constants, and the builder of a packed-constant cache from a checkpoint.
//
// Reference: SafeTensorsIndex / SafeTensorsMappedFile (src/model/safetensors_index.h:13-60:
// a single file, a model.safetensors.index.json or a directory holding either; tensors are
// views into memory-mapped files), QuantizeSymmetricINT4 (src/model/weight_quantization.cpp:
// 188-270), the gpt-oss checkpoint's tensor names (xModel/gpt_oss/120b/gpt_oss_llm.py:110-115:
// <prefix>.mlp.mlp1_weight.{blocks,scales}, mlp2_weight.{blocks,scales}) and the derived-
// constant names that let a stripped engine regenerate its packed constants from the
// checkpoint (plugins/gpt_oss/include/gpt_oss_marlin_pack.h:29-44).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "layout.h"

namespace gb200 {

namespace {

// ------------------------------------------------------------------ a small JSON reader

struct Json {
    enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
    bool b = false;
    double num = 0;
    long long integer = 0;
    bool is_integer = false;
    std::string str;
    std::vector<Json> items;                              // array
    std::vector<std::pair<std::string, Json>> members;    // object, in file order
    const Json* get(const char* key) const
    {
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
};

struct JsonParser {
    const char* p;
    const char* end;
    std::string error;
    void skip()
    {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool fail_at(const char* what)
    {
        if (error.empty()) error = std::string("JSON: ") + what;
        return false;
    }
    bool parse_string(std::string& out)
    {
        if (p >= end || *p != '"') return fail_at("expected a string");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail_at("unterminated escape");
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) return fail_at("short \\u escape");
                        unsigned code = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char c = p[i];
                            code = code * 16 + unsigned(c >= '0' && c <= '9' ? c - '0' : (c | 32) >= 'a' && (c | 32) <= 'f' ? (c | 32) - 'a' + 10 : 0);
                        }
                        p += 4;
                        if (code < 0x80) out += char(code);
                        else if (code < 0x800) out += char(0xC0 | (code >> 6)), out += char(0x80 | (code & 63));
                        else out += char(0xE0 | (code >> 12)), out += char(0x80 | ((code >> 6) & 63)), out += char(0x80 | (code & 63));
                        break;
                    }
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) return fail_at("unterminated string");
        ++p;
        return true;
    }
    bool parse(Json& out, int depth = 0)
    {
        if (depth > 64) return fail_at("nesting too deep");
        skip();
        if (p >= end) return fail_at("unexpected end");
        if (*p == '{') {
            ++p;
            out.kind = Json::kObject;
            skip();
            if (p < end && *p == '}') return ++p, true;
            for (;;) {
                skip();
                std::string key;
                if (!parse_string(key)) return false;
                skip();
                if (p >= end || *p != ':') return fail_at("expected ':'");
                ++p;
                out.members.emplace_back(std::move(key), Json());
                if (!parse(out.members.back().second, depth + 1)) return false;
                skip();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') return ++p, true;
                return fail_at("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            ++p;
            out.kind = Json::kArray;
            skip();
            if (p < end && *p == ']') return ++p, true;
            for (;;) {
                out.items.emplace_back();
                if (!parse(out.items.back(), depth + 1)) return false;
                skip();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') return ++p, true;
                return fail_at("expected ',' or ']'");
            }
        }
        if (*p == '"') {
            out.kind = Json::kString;
            return parse_string(out.str);
        }
        if (end - p >= 4 && !std::strncmp(p, "true", 4)) return out.kind = Json::kBool, out.b = true, p += 4, true;
        if (end - p >= 5 && !std::strncmp(p, "false", 5)) return out.kind = Json::kBool, p += 5, true;
        if (end - p >= 4 && !std::strncmp(p, "null", 4)) return p += 4, true;
        const char* start = p;
        if (p < end && (*p == '-' || *p == '+')) ++p;
        bool integer = true;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
            if (*p == '.' || *p == 'e' || *p == 'E') integer = false;
            ++p;
        }
        if (p == start) return fail_at("unexpected character");
        const std::string text(start, p);
        out.kind = Json::kNumber;
        out.num = std::strtod(text.c_str(), nullptr);
        out.is_integer = integer;
        out.integer = integer ? std::strtoll(text.c_str(), nullptr, 10) : (long long)out.num;
        return true;
    }
};

// ------------------------------------------------------------------ the reader

struct MappedFile {
    std::string path;
    int fd = -1;
    const unsigned char* data = nullptr;
    size_t size = 0;
    ~MappedFile()
    {
        if (data) munmap(const_cast<unsigned char*>(data), size);
        if (fd >= 0) close(fd);
    }
    bool open_file(const std::string& file, std::string& error)
    {
        path = file;
        fd = ::open(file.c_str(), O_RDONLY);
        if (fd < 0) return error = "cannot open " + file, false;
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size < 8) return error = file + " is not a safetensors file (too short)", false;
        size = size_t(st.st_size);
        void* m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (m == MAP_FAILED) return error = "cannot map " + file, false;
        data = static_cast<const unsigned char*>(m);
        return true;
    }
};

struct TensorEntry {
    std::string name, dtype;
    std::vector<long long> shape;
    int file = 0;
    size_t offset = 0, bytes = 0;   // offset from the start of the file
};

int dtype_bytes(const std::string& d)
{
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "U8" || d == "I8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0") return 1;
    return 0;
}

bool is_directory(const std::string& p)
{
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
bool is_file(const std::string& p)
{
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}
std::string dir_of(const std::string& p)
{
    const size_t s = p.find_last_of('/');
    return s == std::string::npos ? std::string(".") : p.substr(0, s);
}
bool ends_with(const std::string& s, const char* tail)
{
    const size_t n = std::strlen(tail);
    return s.size() >= n && s.compare(s.size() - n, n, tail) == 0;
}

}  // namespace

struct Safetensors {
    std::vector<std::unique_ptr<MappedFile>> files;
    std::vector<TensorEntry> tensors;                 // in header order, file after file
    std::map<std::string, size_t> by_name;

    bool add_file(const std::string& path, std::string& error)
    {
        auto f = std::make_unique<MappedFile>();
        if (!f->open_file(path, error)) return false;
        unsigned long long header = 0;
        std::memcpy(&header, f->data, 8);   // little-endian length of the JSON header
        if (header > f->size - 8 || header > (1ull << 31)) return error = path + ": header length beyond the file", false;
        JsonParser jp{reinterpret_cast<const char*>(f->data + 8), reinterpret_cast<const char*>(f->data + 8 + header), {}};
        Json root;
        if (!jp.parse(root) || root.kind != Json::kObject) return error = path + ": " + (jp.error.empty() ? "header is not an object" : jp.error), false;
        const size_t data_start = 8 + size_t(header);
        const int index = int(files.size());
        for (const auto& m : root.members) {
            if (m.first == "__metadata__") continue;
            const Json* dt = m.second.get("dtype");
            const Json* sh = m.second.get("shape");
            const Json* off = m.second.get("data_offsets");
            if (!dt || dt->kind != Json::kString || !sh || sh->kind != Json::kArray || !off || off->kind != Json::kArray || off->items.size() != 2)
                return error = path + ": malformed entry for " + m.first, false;
            TensorEntry t;
            t.name = m.first;
            t.dtype = dt->str;
            size_t elements = 1;
            for (const Json& e : sh->items) {
                if (e.kind != Json::kNumber || e.integer < 0) return error = path + ": bad shape of " + m.first, false;
                t.shape.push_back(e.integer);
                elements *= size_t(e.integer);
            }
            const long long a = off->items[0].integer, b = off->items[1].integer;
            if (a < 0 || b < a || size_t(b) > f->size - data_start) return error = path + ": data of " + m.first + " lies outside the file", false;
            t.file = index;
            t.offset = data_start + size_t(a);
            t.bytes = size_t(b - a);
            const int eb = dtype_bytes(t.dtype);
            if (eb && elements * size_t(eb) != t.bytes) return error = path + ": byte count of " + m.first + " does not match its shape", false;
            if (by_name.count(t.name)) return error = "tensor " + t.name + " appears twice", false;
            by_name[t.name] = tensors.size();
            tensors.push_back(std::move(t));
        }
        files.push_back(std::move(f));
        return true;
    }

    // A single file, an index (weight_map: tensor -> shard file), or a directory with either.
    bool open_path(std::string path, std::string& error)
    {
        if (is_directory(path)) {
            if (is_file(path + "/model.safetensors.index.json")) path += "/model.safetensors.index.json";
            else if (is_file(path + "/model.safetensors")) path += "/model.safetensors";
            else return error = path + " holds neither model.safetensors.index.json nor model.safetensors", false;
        }
        if (!ends_with(path, ".json")) return add_file(path, error);
        FILE* fp = std::fopen(path.c_str(), "rb");
        if (!fp) return error = "cannot open " + path, false;
        std::string text;
        char buf[65536];
        size_t n;
        while ((n = std::fread(buf, 1, sizeof buf, fp)) > 0) text.append(buf, n);
        std::fclose(fp);
        JsonParser jp{text.data(), text.data() + text.size(), {}};
        Json root;
        if (!jp.parse(root) || root.kind != Json::kObject) return error = path + ": " + (jp.error.empty() ? "not a JSON object" : jp.error), false;
        const Json* map = root.get("weight_map");
        if (!map || map->kind != Json::kObject) return error = path + ": no weight_map", false;
        std::vector<std::string> shards;
        for (const auto& m : map->members) {
            if (m.second.kind != Json::kString) return error = path + ": weight_map entry of " + m.first + " is not a file name", false;
            if (std::find(shards.begin(), shards.end(), m.second.str) == shards.end()) shards.push_back(m.second.str);
        }
        const std::string dir = dir_of(path);
        for (const std::string& s : shards)
            if (!add_file(dir + "/" + s, error)) return false;
        for (const auto& m : map->members)
            if (!by_name.count(m.first)) return error = "tensor " + m.first + " of the index is in none of its shards", false;
        return true;
    }
};

namespace {

// ------------------------------------------------------------------ scalar conversions

float half_to_float(uint16_t h)
{
    const uint32_t sign = uint32_t(h & 0x8000u) << 16, exp = (h >> 10) & 31u, man = h & 1023u;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 1024u));
            bits = sign | uint32_t(127 - 15 - e) << 23 | (m & 1023u) << 13;
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | man << 13;
    else bits = sign | (exp + 112u) << 23 | man << 13;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// round to nearest even, as the reference's FloatToFP16 (and every hardware conversion) does
uint16_t float_to_half(float f)
{
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return uint16_t(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
    if (x >= 0x477ff000u) return uint16_t(sign | 0x7c00u);                 // rounds to infinity
    if (x < 0x33000001u) return uint16_t(sign);                             // below half of the smallest subnormal
    const int e = int(x >> 23) - 127;
    uint32_t man = (x & 0x7fffffu) | 0x800000u;
    int shift = e < -14 ? 13 + (-14 - e) : 13;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) ++half;
    if (e < -14) return uint16_t(sign | half);                              // subnormal (a carry makes it the smallest normal)
    return uint16_t(sign | (uint32_t(e + 15) << 10) + (half - 1024u));       // a carry moves into the exponent
}

float bf16_bits_to_float(uint16_t b)
{
    const uint32_t bits = uint32_t(b) << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
uint16_t float_to_bf16_bits(float f)
{
    uint32_t x;
    std::memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return uint16_t((x >> 16) | 0x40u);
    return uint16_t((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}

float read_weight(const void* w, int dtype, size_t i)
{
    if (dtype == GARNET_B200_FP32) return static_cast<const float*>(w)[i];
    const uint16_t bits = static_cast<const uint16_t*>(w)[i];
    return dtype == GARNET_B200_FP16 ? half_to_float(bits) : bf16_bits_to_float(bits);
}

}  // namespace

}  // namespace gb200

using namespace gb200;

extern "C" {

int garnet_b200_safetensors_open(const char* path, garnet_b200_safetensors_t* out)
{
    if (!out) return fail(GARNET_B200_INVALID_VALUE, "safetensors_open: null output");
    *out = nullptr;
    if (!path) return fail(GARNET_B200_INVALID_VALUE, "safetensors_open: null path");
    auto st = std::make_unique<Safetensors>();
    std::string error;
    if (!st->open_path(path, error)) return fail(GARNET_B200_INVALID_VALUE, "safetensors_open: %s", error.c_str());
    *out = reinterpret_cast<garnet_b200_safetensors_t>(st.release());
    return GARNET_B200_OK;
}

int garnet_b200_safetensors_count(garnet_b200_safetensors_t h)
{
    return h ? int(reinterpret_cast<Safetensors*>(h)->tensors.size()) : -1;
}

int garnet_b200_safetensors_entry(garnet_b200_safetensors_t h, int index, const char* name, const char** name_out,
                                  const char** dtype, int* rank, long long* shape8, const void** data, size_t* bytes)
{
    Safetensors* st = reinterpret_cast<Safetensors*>(h);
    if (!st) return fail(GARNET_B200_INVALID_VALUE, "safetensors_entry: null handle");
    size_t at;
    if (name) {
        const auto it = st->by_name.find(name);
        if (it == st->by_name.end()) return fail(GARNET_B200_INVALID_VALUE, "safetensors_entry: no tensor named %s", name);
        at = it->second;
    } else {
        if (index < 0 || size_t(index) >= st->tensors.size()) return fail(GARNET_B200_INVALID_VALUE, "safetensors_entry: index %d out of range", index);
        at = size_t(index);
    }
    const TensorEntry& t = st->tensors[at];
    if (t.shape.size() > 8) return fail(GARNET_B200_NOT_SUPPORTED, "safetensors_entry: %s has more than 8 dimensions", t.name.c_str());
    if (name_out) *name_out = t.name.c_str();
    if (dtype) *dtype = t.dtype.c_str();
    if (rank) *rank = int(t.shape.size());
    if (shape8) std::copy(t.shape.begin(), t.shape.end(), shape8);
    if (data) *data = st->files[size_t(t.file)]->data + t.offset;
    if (bytes) *bytes = t.bytes;
    return GARNET_B200_OK;
}

void garnet_b200_safetensors_close(garnet_b200_safetensors_t h) { delete reinterpret_cast<Safetensors*>(h); }

int garnet_b200_safetensors_write(const char* path, const char* const* names, const char* const* dtypes, const int* ranks,
                                  const long long* const* shapes, const void* const* datas, const size_t* bytes, int count)
{
    if (!path || count < 0 || (count && (!names || !dtypes || !ranks || !shapes || !datas || !bytes)))
        return fail(GARNET_B200_INVALID_VALUE, "safetensors_write: bad argument");
    std::string header = "{";
    size_t offset = 0;
    for (int i = 0; i < count; ++i) {
        if (!names[i] || !dtypes[i] || (!datas[i] && bytes[i])) return fail(GARNET_B200_INVALID_VALUE, "safetensors_write: null entry %d", i);
        if (i) header += ",";
        header += "\"";
        for (const char* c = names[i]; *c; ++c) {
            if (*c == '"' || *c == '\\') header += '\\';
            header += *c;
        }
        header += "\":{\"dtype\":\"" + std::string(dtypes[i]) + "\",\"shape\":[";
        for (int d = 0; d < ranks[i]; ++d) header += (d ? "," : "") + std::to_string(shapes[i][d]);
        header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + bytes[i]) + "]}";
        offset += bytes[i];
    }
    header += "}";
    while ((header.size() + 8) % 256) header += ' ';   // tensor data starts on a 256-byte boundary of the file
    FILE* fp = std::fopen(path, "wb");
    if (!fp) return fail(GARNET_B200_INVALID_VALUE, "safetensors_write: cannot create %s", path);
    const unsigned long long n = header.size();
    bool ok = std::fwrite(&n, 8, 1, fp) == 1 && std::fwrite(header.data(), 1, header.size(), fp) == header.size();
    for (int i = 0; ok && i < count; ++i) ok = bytes[i] == 0 || std::fwrite(datas[i], 1, bytes[i], fp) == bytes[i];
    ok = std::fclose(fp) == 0 && ok;
    if (!ok) return fail(GARNET_B200_INVALID_VALUE, "safetensors_write: writing %s failed", path);
    return GARNET_B200_OK;
}

int garnet_b200_int4_quantize_host(const void* w, int w_dtype, int n, int k, int group, int scale_dtype, uint8_t* nibbles,
                                   uint16_t* scales, double* max_abs_error)
{
    if (!w || !nibbles || !scales || n <= 0 || k <= 0 || group <= 0 || k % group)
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize_host: bad argument");
    if (w_dtype != GARNET_B200_FP32 && w_dtype != GARNET_B200_FP16 && w_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize_host: weight dtype must be fp32, fp16 or bf16");
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "int4_quantize_host: scale dtype must be fp16 or bf16");
    const size_t groups = size_t(k) / size_t(group);
    std::memset(nibbles, 0, (size_t(n) * k + 1) / 2);
    double worst = 0.0;
    for (size_t r = 0; r < size_t(n); ++r)
        for (size_t g = 0; g < groups; ++g) {
            const size_t start = r * k + g * group;
            float lo = 0.f, hi = 0.f;
            for (int o = 0; o < group; ++o) {
                const float v = read_weight(w, w_dtype, start + o);
                lo = std::min(lo, v);
                hi = std::max(hi, v);
            }
            float scale = std::max(-lo / 8.0f, hi / 7.0f);
            if (!std::isfinite(scale) || scale <= 0.f) scale = 1.0f;
            const uint16_t bits = scale_dtype == GARNET_B200_FP16 ? float_to_half(scale) : float_to_bf16_bits(scale);
            const float stored = scale_dtype == GARNET_B200_FP16 ? half_to_float(bits) : bf16_bits_to_float(bits);
            scales[r * groups + g] = bits;
            for (int o = 0; o < group; ++o) {
                const size_t i = start + o;
                const float v = read_weight(w, w_dtype, i);
                int q = int(std::nearbyint(v / stored));
                q = std::max(-8, std::min(7, q));
                nibbles[i >> 1] |= uint8_t((q & 15) << ((i & 1u) * 4u));
                worst = std::max(worst, double(std::fabs(v - float(q) * stored)));
            }
        }
    if (max_abs_error) *max_abs_error = worst;
    return GARNET_B200_OK;
}

// "__garnet_b200_<kind>_v1_<detail>__:<source>"; kind: w4a16 (detail g<group>_s<scale dtype>),
// mxs / mxb (streaming / block layout of MoE experts; detail u<which>_t<tp rank>of<tp world>).
int garnet_b200_packed_tensor_name(const char* source, int kind, int a, int b, int c, char* out, size_t out_bytes)
{
    if (!source || !out || kind < 0 || kind > 2) return fail(GARNET_B200_INVALID_VALUE, "packed_tensor_name: bad argument");
    char prefix[96];
    if (kind == 0) std::snprintf(prefix, sizeof prefix, "__garnet_b200_w4a16_v1_g%d_s%d__:", a, b);
    else std::snprintf(prefix, sizeof prefix, "__garnet_b200_%s_v1_u%d_t%dof%d__:", kind == 1 ? "mxs" : "mxb", a, b, c);
    const size_t need = std::strlen(prefix) + std::strlen(source) + 1;
    if (need > out_bytes) return fail(GARNET_B200_INVALID_VALUE, "packed_tensor_name: the name needs %zu bytes", need);
    std::snprintf(out, out_bytes, "%s%s", prefix, source);
    return GARNET_B200_OK;
}

int garnet_b200_packed_tensor_name_parse(const char* name, int* kind, int* a, int* b, int* c, const char** source)
{
    if (!name || !kind || !a || !b || !c || !source) return fail(GARNET_B200_INVALID_VALUE, "packed_tensor_name_parse: null pointer");
    int used = 0;
    *c = 0;
    if (std::sscanf(name, "__garnet_b200_w4a16_v1_g%d_s%d__:%n", a, b, &used) == 2 && used > 0 && name[used]) {
        *kind = 0;
        *source = name + used;
        return GARNET_B200_OK;
    }
    for (int k = 1; k <= 2; ++k) {
        const std::string fmt = std::string("__garnet_b200_") + (k == 1 ? "mxs" : "mxb") + "_v1_u%d_t%dof%d__:%n";
        used = 0;
        if (std::sscanf(name, fmt.c_str(), a, b, c, &used) == 3 && used > 0 && name[used]) {
            *kind = k;
            *source = name + used;
            return GARNET_B200_OK;
        }
    }
    return fail(GARNET_B200_INVALID_VALUE, "packed_tensor_name_parse: %s is not a derived-constant name", name);
}

// One entry of the cache being built: its header fields and how to produce its bytes.
namespace {
struct CacheEntry {
    std::string name, dtype;
    std::vector<long long> shape;
    size_t bytes = 0;
    int action = 0;              // 0 copy, 1 int4 linear, 2 MoE projection
    size_t source = 0, partner = 0;
    int which = 0, layout = 0;
};
int dtype_code(const std::string& d)
{
    return d == "F32" ? GARNET_B200_FP32 : d == "F16" ? GARNET_B200_FP16 : d == "BF16" ? GARNET_B200_BF16 : -1;
}
}  // namespace

int garnet_b200_checkpoint_build_cache(garnet_b200_safetensors_t h, const char* out_path, int group, int scale_dtype,
                                       int moe_layouts, int tp_rank, int tp_world)
{
    Safetensors* st = reinterpret_cast<Safetensors*>(h);
    if (!st || !out_path) return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: null argument");
    if (scale_dtype != GARNET_B200_FP16 && scale_dtype != GARNET_B200_BF16)
        return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: scale dtype must be fp16 or bf16");
    if (moe_layouts < 0 || moe_layouts > GARNET_B200_MOE_LAYOUT_BLOCK)
        return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: moe_layouts must be 0, 1 or 2");
    if (tp_world < 1) tp_world = 1;
    if (tp_rank < 0 || tp_rank >= tp_world) return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: bad tp rank");
    const auto moe_options = [&](const TensorEntry& blocks, int which, garnet_b200_moe_options* o) {
        // blocks: [E, rows, K/32, 16]; gate_up: rows = 2I, K = H; down: rows = H, K = I
        *o = garnet_b200_moe_options{};
        o->abi = GARNET_B200_ABI;
        o->struct_size = int(sizeof(garnet_b200_moe_options));
        const long long rows = blocks.shape[1], k = blocks.shape[2] * 32;
        o->hidden = int(which == 0 ? k : rows);
        o->intermediate = int(which == 0 ? rows / 2 : k);
        o->experts = int(blocks.shape[0]);
        o->top_k = 1;
        o->io_dtype = GARNET_B200_BF16;
        o->limit = 7.f;
        o->tp_rank = tp_rank;
        o->tp_world = tp_world > 1 ? tp_world : 0;
    };
    // ---- first pass: what the cache will hold
    std::vector<CacheEntry> entries;
    std::vector<char> consumed(st->tensors.size(), 0);
    char derived[512];
    for (size_t i = 0; i < st->tensors.size(); ++i) {
        const TensorEntry& t = st->tensors[i];
        const bool up = ends_with(t.name, ".mlp1_weight.blocks"), down = ends_with(t.name, ".mlp2_weight.blocks");
        if ((up || down) && t.dtype == "U8" && t.shape.size() == 4 && t.shape[3] == 16) {
            const std::string partner = t.name.substr(0, t.name.size() - 6) + "scales";
            const auto it = st->by_name.find(partner);
            if (it == st->by_name.end()) return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: %s has no scales tensor", t.name.c_str());
            consumed[i] = consumed[it->second] = 1;
            garnet_b200_moe_options o;
            moe_options(t, up ? 0 : 1, &o);
            for (int layout = GARNET_B200_MOE_LAYOUT_STREAM; layout <= GARNET_B200_MOE_LAYOUT_BLOCK; ++layout) {
                if (moe_layouts && moe_layouts != layout) continue;
                CacheEntry e;
                if (int rc = garnet_b200_packed_tensor_name(t.name.substr(0, t.name.size() - 7).c_str(), layout, up ? 0 : 1, tp_rank,
                                                            tp_world, derived, sizeof derived))
                    return rc;
                e.name = derived;
                e.dtype = "U8";
                if (int rc = garnet_b200_moe_packed_bytes(&o, up ? 0 : 1, layout, o.experts, &e.bytes)) return rc;
                e.shape = {(long long)e.bytes};
                e.action = 2, e.source = i, e.partner = it->second, e.which = up ? 0 : 1, e.layout = layout;
                entries.push_back(std::move(e));
            }
        }
    }
    for (size_t i = 0; i < st->tensors.size(); ++i) {
        if (consumed[i]) continue;
        const TensorEntry& t = st->tensors[i];
        CacheEntry e;
        std::vector<int64_t> shape(t.shape.begin(), t.shape.end());
        if (dtype_code(t.dtype) >= 0 && garnet_b200_is_int4_linear_weight(t.name.c_str(), t.dtype.c_str(), int(shape.size()), shape.data(), group) == 1) {
            if (int rc = garnet_b200_packed_tensor_name(t.name.c_str(), 0, group, scale_dtype, 0, derived, sizeof derived)) return rc;
            e.name = derived;
            e.dtype = "U8";
            if (int rc = garnet_b200_w4a16_packed_bytes(int(t.shape[0]), int(t.shape[1]), group, &e.bytes)) return rc;
            e.shape = {(long long)e.bytes};
            e.action = 1;
        } else {
            e.name = t.name, e.dtype = t.dtype, e.shape = t.shape, e.bytes = t.bytes;
        }
        e.source = i;
        entries.push_back(std::move(e));
    }
    // ---- header, then one blob after the other (nothing larger than one tensor is held in memory)
    std::string header = "{";
    size_t offset = 0;
    for (size_t i = 0; i < entries.size(); ++i) {
        const CacheEntry& e = entries[i];
        header += (i ? ",\"" : "\"") + e.name + "\":{\"dtype\":\"" + e.dtype + "\",\"shape\":[";
        for (size_t d = 0; d < e.shape.size(); ++d) header += (d ? "," : "") + std::to_string(e.shape[d]);
        header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + e.bytes) + "]}";
        offset += e.bytes;
    }
    header += "}";
    while ((header.size() + 8) % 256) header += ' ';
    FILE* fp = std::fopen(out_path, "wb");
    if (!fp) return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: cannot create %s", out_path);
    const unsigned long long n = header.size();
    bool ok = std::fwrite(&n, 8, 1, fp) == 1 && std::fwrite(header.data(), 1, header.size(), fp) == header.size();
    int rc = GARNET_B200_OK;
    std::vector<uint8_t> blob, nib, gathered_b, gathered_s;
    std::vector<uint16_t> sc;
    for (size_t i = 0; ok && !rc && i < entries.size(); ++i) {
        const CacheEntry& e = entries[i];
        const TensorEntry& t = st->tensors[e.source];
        const void* src = st->files[size_t(t.file)]->data + t.offset;
        if (e.action == 0) {
            ok = e.bytes == 0 || std::fwrite(src, 1, e.bytes, fp) == e.bytes;
            continue;
        }
        blob.resize(e.bytes);
        if (e.action == 1) {
            const int rows = int(t.shape[0]), cols = int(t.shape[1]);
            nib.resize(size_t(rows) * cols / 2);
            sc.resize(size_t(rows) * (cols / group));
            rc = garnet_b200_int4_quantize_host(src, dtype_code(t.dtype), rows, cols, group, scale_dtype, nib.data(), sc.data(), nullptr);
            if (!rc) rc = garnet_b200_w4a16_pack_host(nib.data(), sc.data(), scale_dtype, rows, cols, group, blob.data());
        } else {
            const TensorEntry& p = st->tensors[e.partner];
            const uint8_t* blocks = static_cast<const uint8_t*>(src);
            const uint8_t* scales = st->files[size_t(p.file)]->data + p.offset;
            garnet_b200_moe_options o;
            moe_options(t, e.which, &o);
            if (tp_world > 1) {
                // this rank's gate/up row pairs (axis 1) or down-projection K groups (axis 2)
                const int mode = e.which == 0 ? 1 : 2;
                gathered_b.resize(t.bytes / size_t(tp_world));
                gathered_s.resize(p.bytes / size_t(tp_world));
                rc = garnet_b200_moe_gather_intermediate_shard(blocks, t.bytes, t.shape.data(), 4, 1, tp_rank, tp_world, mode, gathered_b.data());
                if (!rc) rc = garnet_b200_moe_gather_intermediate_shard(scales, p.bytes, p.shape.data(), 3, 1, tp_rank, tp_world, mode, gathered_s.data());
                blocks = gathered_b.data(), scales = gathered_s.data();
            }
            if (!rc) rc = garnet_b200_moe_pack_host(&o, e.which, e.layout, blocks, scales, o.experts, blob.data());
        }
        if (!rc) ok = std::fwrite(blob.data(), 1, blob.size(), fp) == blob.size();
    }
    ok = std::fclose(fp) == 0 && ok;
    if (rc) return rc;
    if (!ok) return fail(GARNET_B200_INVALID_VALUE, "checkpoint_build_cache: writing %s failed", out_path);
    return GARNET_B200_OK;
}

}  // extern "C"
