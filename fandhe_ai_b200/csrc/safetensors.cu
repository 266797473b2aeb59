// Weight wire format: safetensors files with INT8 payloads.
//
// The reference reads safetensors through crates/onnx-interop/src/st_load.rs (layout validation
// :128-132, typed loading :433-562, "no silent skip": an unsupported dtype is an error :154-160, every missing
// key is reported at once :209-222, no renaming and no transposition) and rejects the I8 dtype today (:624).
// This file extends that contract to what the quantized decoder needs: per-output-channel int8 weights
// ("<name>.qweight" I8 [rows, cols] + "<name>.scale" F32 [rows]) next to f32 tensors ("<name>.weight" F32, quantised
// on the device as b200_decoder_load_tensor does).  The container format itself (8-byte little-endian header length,
// JSON header with dtype / shape / data_offsets per tensor, one contiguous byte buffer) is the published safetensors
// format; the parser below is a restatement of its validation rules: offsets start at 0, tensors are contiguous in
// offset order without holes or overlaps, the last offset equals the buffer length, and each tensor's byte length
// equals the product of its shape times the element width.  Host code only.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "backend.h"
#include "safetensors.h"

namespace b200 {
namespace {

struct Cursor {
    const char* p;
    const char* end;
    std::string err;
    bool fail(const std::string& m) {
        if (err.empty()) err = m;
        return false;
    }
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) { ++p; return true; }
        return false;
    }
    bool expect(char c) { return eat(c) || fail(std::string("header JSON: expected '") + c + "'"); }
    bool string(std::string* out) {
        ws();
        if (p >= end || *p != '"') return fail("header JSON: expected a string");
        ++p;
        out->clear();
        while (p < end && *p != '"') {
            char c = *p++;
            if (c == '\\') {
                if (p >= end) return fail("header JSON: unterminated escape");
                char e = *p++;
                switch (e) {
                    case '"': out->push_back('"'); break;
                    case '\\': out->push_back('\\'); break;
                    case '/': out->push_back('/'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'n': out->push_back('\n'); break;
                    case 'r': out->push_back('\r'); break;
                    case 't': out->push_back('\t'); break;
                    case 'u': {
                        if (end - p < 4) return fail("header JSON: short \\u escape");
                        unsigned v = 0;
                        for (int i = 0; i < 4; ++i) {
                            char h = *p++;
                            v <<= 4;
                            if (h >= '0' && h <= '9') v |= unsigned(h - '0');
                            else if (h >= 'a' && h <= 'f') v |= unsigned(h - 'a' + 10);
                            else if (h >= 'A' && h <= 'F') v |= unsigned(h - 'A' + 10);
                            else return fail("header JSON: bad \\u escape");
                        }
                        // UTF-8 encode the BMP code point (surrogate pairs are kept as two 3-byte sequences)
                        if (v < 0x80) out->push_back(char(v));
                        else if (v < 0x800) { out->push_back(char(0xC0 | (v >> 6))); out->push_back(char(0x80 | (v & 0x3F))); }
                        else { out->push_back(char(0xE0 | (v >> 12))); out->push_back(char(0x80 | ((v >> 6) & 0x3F))); out->push_back(char(0x80 | (v & 0x3F))); }
                        break;
                    }
                    default: return fail("header JSON: unknown escape");
                }
            } else {
                out->push_back(c);
            }
        }
        if (p >= end) return fail("header JSON: unterminated string");
        ++p;
        return true;
    }
    bool uint(uint64_t* out) {
        ws();
        if (p >= end || *p < '0' || *p > '9') return fail("header JSON: expected a non-negative integer");
        uint64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            const uint64_t d = uint64_t(*p - '0');
            if (v > (UINT64_MAX - d) / 10) return fail("header JSON: integer overflows");
            v = v * 10 + d;
            ++p;
        }
        *out = v;
        return true;
    }
    bool uint_array(std::vector<uint64_t>* out) {
        out->clear();
        if (!expect('[')) return false;
        if (eat(']')) return true;
        do {
            uint64_t v;
            if (!uint(&v)) return false;
            out->push_back(v);
        } while (eat(','));
        return expect(']');
    }
    // skips any JSON value (used for __metadata__)
    bool skip_value(int depth = 0) {
        if (depth > 16) return fail("header JSON: nesting too deep");
        ws();
        if (p >= end) return fail("header JSON: truncated");
        if (*p == '"') { std::string s; return string(&s); }
        if (*p == '{') {
            ++p;
            if (eat('}')) return true;
            do {
                std::string k;
                if (!string(&k) || !expect(':') || !skip_value(depth + 1)) return false;
            } while (eat(','));
            return expect('}');
        }
        if (*p == '[') {
            ++p;
            if (eat(']')) return true;
            do {
                if (!skip_value(depth + 1)) return false;
            } while (eat(','));
            return expect(']');
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;      // number / true / false / null
        return true;
    }
};

size_t dtype_width(const std::string& d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}

}  // namespace

bool safetensors_parse(const uint8_t* bytes, size_t len, std::vector<StTensor>* out, std::string* err) {
    out->clear();
    auto fail = [&](const std::string& m) {
        *err = "safetensors: " + m;
        return false;
    };
    if (!bytes || len < 8) return fail("file shorter than the 8-byte header length");
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | bytes[i];
    if (n > 100000000ull) return fail("header length " + std::to_string(n) + " exceeds the 100 MB limit of the format");
    if (n > len - 8) return fail("header length " + std::to_string(n) + " exceeds the file");
    const size_t data_len = len - 8 - size_t(n);
    Cursor c{reinterpret_cast<const char*>(bytes + 8), reinterpret_cast<const char*>(bytes + 8 + n), {}};
    if (!c.expect('{')) return fail(c.err);
    if (!c.eat('}')) {
        do {
            std::string name;
            if (!c.string(&name) || !c.expect(':')) return fail(c.err);
            if (name == "__metadata__") {
                if (!c.skip_value()) return fail(c.err);
                continue;
            }
            StTensor t;
            t.name = name;
            bool have_dtype = false, have_shape = false, have_off = false;
            if (!c.expect('{')) return fail(c.err);
            do {
                std::string key;
                if (!c.string(&key) || !c.expect(':')) return fail(c.err);
                if (key == "dtype") { if (!c.string(&t.dtype)) return fail(c.err); have_dtype = true; }
                else if (key == "shape") {
                    std::vector<uint64_t> s;
                    if (!c.uint_array(&s)) return fail(c.err);
                    t.shape.assign(s.begin(), s.end());
                    have_shape = true;
                } else if (key == "data_offsets") {
                    std::vector<uint64_t> o;
                    if (!c.uint_array(&o)) return fail(c.err);
                    if (o.size() != 2) return fail(name + ": data_offsets must hold two integers");
                    t.begin = o[0];
                    t.end = o[1];
                    have_off = true;
                } else if (!c.skip_value()) return fail(c.err);
            } while (c.eat(','));
            if (!c.expect('}')) return fail(c.err);
            if (!have_dtype || !have_shape || !have_off) return fail(name + ": dtype, shape and data_offsets are required");
            for (const StTensor& o : *out)
                if (o.name == name) return fail("duplicate tensor name " + name);
            out->push_back(t);
        } while (c.eat(','));
        if (!c.expect('}')) return fail(c.err);
    }
    c.ws();
    if (c.p != c.end) return fail("trailing bytes after the header JSON");
    // layout: contiguous in offset order from 0 to the end of the buffer, byte length = elements x width
    std::vector<const StTensor*> order;
    for (const StTensor& t : *out) order.push_back(&t);
    std::sort(order.begin(), order.end(), [](const StTensor* a, const StTensor* b) { return a->begin < b->begin || (a->begin == b->begin && a->end < b->end); });
    uint64_t at = 0;
    for (const StTensor* t : order) {
        const size_t w = dtype_width(t->dtype);
        if (w == 0) return fail(t->name + ": unknown dtype " + t->dtype);
        if (t->begin != at || t->end < t->begin) return fail(t->name + ": data offsets leave a hole or overlap (expected begin " + std::to_string(at) + ")");
        unsigned __int128 elems = 1;
        for (uint64_t s : t->shape) {
            elems *= s;
            if (elems > (unsigned __int128)1 << 62) return fail(t->name + ": element count overflows");
        }
        if ((unsigned __int128)(t->end - t->begin) != elems * w)
            return fail(t->name + ": byte length " + std::to_string(t->end - t->begin) + " differs from shape x dtype width " +
                        std::to_string((uint64_t)(elems * w)));
        at = t->end;
    }
    if (at != data_len) return fail("the tensors cover " + std::to_string(at) + " bytes but the buffer holds " + std::to_string(data_len));
    for (StTensor& t : *out) t.data = bytes + 8 + n + t.begin;
    return true;
}

}  // namespace b200

using namespace b200;

extern "C" {

// validate_safetensors_layout_from_bytes (crates/onnx-interop/src/st_load.rs:128-132): header and layout only, any
// dtype of the format, nothing is allocated on a device.  *n_tensors receives the number of tensors.
int32_t b200_safetensors_validate(const uint8_t* bytes, size_t len, uint64_t* n_tensors) {
    std::vector<StTensor> ts;
    std::string err;
    if (n_tensors) *n_tensors = 0;
    if (!safetensors_parse(bytes, len, &ts, &err)) return fail(B200_INVALID_ARGUMENT, err);
    if (n_tensors) *n_tensors = ts.size();
    return B200_OK;
}

}  // extern "C"
