// Safetensors reader (mmap, zero-copy) / streaming writer, and the CPU reference codecs + row quantisers
// for NVFP4 and MXFP8.  Reference counterparts: src/phaseshift/io/safetensors_{reader,writer}.cpp,
// src/phaseshift/quantization/fpx/{e4m3,ue4m3}.cpp, psq/psq.cpp (scale search), fpx/crc32.cpp.
#include "ps_io.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstring>

namespace psrt {

// ------------------------------------------------------------------------------------------------ mini JSON
namespace {
struct JParser {
    const char* p; const char* end;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    [[noreturn]] void fail(const char* m) { throw Error(StatusCode::format_error, std::string("json: ") + m); }
    JValue parse() {
        ws();
        if (p >= end) fail("unexpected end");
        JValue v;
        if (*p == '{') {
            v.kind = JValue::Object; ++p; ws();
            if (p < end && *p == '}') { ++p; return v; }
            while (true) {
                ws();
                JValue k = parse_string();
                ws();
                if (p >= end || *p != ':') fail("expected ':'");
                ++p;
                v.obj.emplace_back(k.str, parse());
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; break; }
                fail("expected ',' or '}'");
            }
            return v;
        }
        if (*p == '[') {
            v.kind = JValue::Array; ++p; ws();
            if (p < end && *p == ']') { ++p; return v; }
            while (true) {
                v.arr.push_back(parse());
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; break; }
                fail("expected ',' or ']'");
            }
            return v;
        }
        if (*p == '"') return parse_string();
        if (!strncmp(p, "true", 4)) { p += 4; v.kind = JValue::Bool; v.num = 1; return v; }
        if (!strncmp(p, "false", 5)) { p += 5; v.kind = JValue::Bool; v.num = 0; return v; }
        if (!strncmp(p, "null", 4)) { p += 4; v.kind = JValue::Null; return v; }
        char* e = nullptr;
        v.kind = JValue::Number;
        v.num = strtod(p, &e);
        if (e == p) fail("bad value");
        p = e;
        return v;
    }
    JValue parse_string() {
        if (p >= end || *p != '"') fail("expected string");
        ++p;
        JValue v; v.kind = JValue::String;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': v.str += '\n'; break; case 't': v.str += '\t'; break; case 'r': v.str += '\r'; break;
                    case 'b': v.str += '\b'; break; case 'f': v.str += '\f'; break;
                    case 'u': {   // keep BMP escapes as UTF-8
                        if (p + 4 >= end) fail("bad \\u");
                        unsigned cp = (unsigned)strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
                        p += 4;
                        if (cp < 0x80) v.str += (char)cp;
                        else if (cp < 0x800) { v.str += (char)(0xC0 | (cp >> 6)); v.str += (char)(0x80 | (cp & 0x3F)); }
                        else { v.str += (char)(0xE0 | (cp >> 12)); v.str += (char)(0x80 | ((cp >> 6) & 0x3F)); v.str += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: v.str += *p;
                }
                ++p;
            } else {
                v.str += *p++;
            }
        }
        if (p >= end) fail("unterminated string");
        ++p;
        return v;
    }
};
}  // namespace

JValue json_parse(const char* data, size_t n) {
    JParser jp{data, data + n};
    JValue v = jp.parse();
    jp.ws();
    if (jp.p != jp.end) throw Error(StatusCode::format_error, "json: trailing characters");
    return v;
}
const JValue* JValue::get(const std::string& key) const {
    for (const auto& kv : obj) if (kv.first == key) return &kv.second;
    return nullptr;
}

size_t dtype_size(const std::string& dt) {
    if (dt == "F64" || dt == "I64" || dt == "U64") return 8;
    if (dt == "F32" || dt == "I32" || dt == "U32") return 4;
    if (dt == "F16" || dt == "BF16" || dt == "I16" || dt == "U16") return 2;
    if (dt == "U8" || dt == "I8" || dt == "BOOL" || dt == "F8_E4M3" || dt == "F8_E5M2") return 1;
    throw Error(StatusCode::format_error, "unknown safetensors dtype " + dt);
}

// ------------------------------------------------------------------------------------------------ reader
SafetensorsReader::SafetensorsReader(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw Error(StatusCode::io_error, "cannot open " + path);
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 8) { ::close(fd_); throw Error(StatusCode::format_error, "file too small: " + path); }
    size_ = (size_t)st.st_size;
    base_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (base_ == MAP_FAILED) { ::close(fd_); throw Error(StatusCode::io_error, "mmap failed: " + path); }
    uint64_t hlen;
    memcpy(&hlen, base_, 8);
    if (hlen > size_ - 8) { close(); throw Error(StatusCode::format_error, "header length exceeds file"); }
    data_begin_ = 8 + (size_t)hlen;
    JValue root = json_parse((const char*)base_ + 8, (size_t)hlen);
    if (root.kind != JValue::Object) { close(); throw Error(StatusCode::format_error, "header is not an object"); }
    for (const auto& kv : root.obj) {
        if (kv.first == "__metadata__") {
            for (const auto& m : kv.second.obj) metadata_[m.first] = m.second.str;
            continue;
        }
        TensorSpec ts;
        const JValue* dt = kv.second.get("dtype");
        const JValue* sh = kv.second.get("shape");
        const JValue* off = kv.second.get("data_offsets");
        if (!dt || !sh || !off || off->arr.size() != 2) { close(); throw Error(StatusCode::format_error, "bad tensor entry " + kv.first); }
        ts.dtype = dt->str;
        uint64_t numel = 1;
        for (const auto& d : sh->arr) { ts.shape.push_back((int64_t)d.num); numel = checked_mul(numel, (uint64_t)d.num); }
        ts.begin = (uint64_t)off->arr[0].num; ts.end = (uint64_t)off->arr[1].num;
        if (ts.end < ts.begin || data_begin_ + ts.end > size_ || ts.end - ts.begin != checked_mul(numel, dtype_size(ts.dtype))) {
            close();
            throw Error(StatusCode::format_error, "tensor " + kv.first + " has inconsistent offsets");
        }
        names_.push_back(kv.first);
        specs_[kv.first] = ts;
    }
}
void SafetensorsReader::close() {
    if (base_ && base_ != MAP_FAILED) munmap((void*)base_, size_);
    base_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
}
SafetensorsReader::~SafetensorsReader() { close(); }
const TensorSpec& SafetensorsReader::spec(const std::string& name) const {
    auto it = specs_.find(name);
    if (it == specs_.end()) throw Error(StatusCode::invalid_argument, "no tensor named " + name);
    return it->second;
}
const uint8_t* SafetensorsReader::data(const std::string& name) const { return base_ + data_begin_ + spec(name).begin; }

// ------------------------------------------------------------------------------------------------ writer
SafetensorsWriter::SafetensorsWriter(const std::string& path) : path_(path) {}
SafetensorsWriter::~SafetensorsWriter() { if (fd_ >= 0) ::close(fd_); }
void SafetensorsWriter::set_metadata(const std::string& k, const std::string& v) { metadata_[k] = v; }
void SafetensorsWriter::plan_tensor(const std::string& name, const std::string& dtype, const std::vector<int64_t>& shape) {
    if (header_written_) throw Error(StatusCode::invalid_argument, "plan after header");
    if (planned_.count(name)) throw Error(StatusCode::invalid_argument, "duplicate tensor " + name);
    uint64_t numel = 1;
    for (auto d : shape) numel = checked_mul(numel, (uint64_t)d);
    Planned p;
    p.spec.dtype = dtype; p.spec.shape = shape;
    p.spec.begin = cursor_;
    p.spec.end = cursor_ + checked_mul(numel, dtype_size(dtype));
    cursor_ = p.spec.end;
    order_.push_back(name);
    planned_[name] = p;
}
static void json_escape(std::string& o, const std::string& s) {
    o += '"';
    for (char c : s) {
        if (c == '"' || c == '\\') { o += '\\'; o += c; }
        else if (c == '\n') o += "\\n";
        else o += c;
    }
    o += '"';
}
void SafetensorsWriter::write_header() {
    if (header_written_) return;
    std::string h = "{";
    bool first = true;
    if (!metadata_.empty()) {
        h += "\"__metadata__\":{";
        bool f2 = true;
        for (const auto& kv : metadata_) { if (!f2) h += ','; f2 = false; json_escape(h, kv.first); h += ':'; json_escape(h, kv.second); }
        h += '}';
        first = false;
    }
    for (const auto& n : order_) {
        const auto& p = planned_[n];
        if (!first) h += ',';
        first = false;
        json_escape(h, n);
        h += ":{\"dtype\":\"" + p.spec.dtype + "\",\"shape\":[";
        for (size_t i = 0; i < p.spec.shape.size(); ++i) { if (i) h += ','; h += std::to_string(p.spec.shape[i]); }
        h += "],\"data_offsets\":[" + std::to_string(p.spec.begin) + "," + std::to_string(p.spec.end) + "]}";
    }
    h += '}';
    while ((h.size() + 8) % 8) h += ' ';      // keep the data section 8-byte aligned
    fd_ = ::open(path_.c_str(), O_CREAT | O_TRUNC | O_WRONLY, 0644);
    if (fd_ < 0) throw Error(StatusCode::io_error, "cannot create " + path_);
    const uint64_t hlen = h.size();
    if (::write(fd_, &hlen, 8) != 8 || ::write(fd_, h.data(), h.size()) != (ssize_t)h.size())
        throw Error(StatusCode::io_error, "header write failed");
    data_begin_ = 8 + h.size();
    header_written_ = true;
}
void SafetensorsWriter::write_chunk(const std::string& name, const uint8_t* data, size_t n) {
    if (!header_written_) write_header();
    auto it = planned_.find(name);
    if (it == planned_.end()) throw Error(StatusCode::invalid_argument, "tensor was not planned: " + name);
    Planned& p = it->second;
    if (p.written + n > p.spec.end - p.spec.begin) throw Error(StatusCode::out_of_range, "chunk overruns tensor " + name);
    const off_t off = (off_t)(data_begin_ + p.spec.begin + p.written);
    size_t done = 0;
    while (done < n) {
        const ssize_t w = ::pwrite(fd_, data + done, n - done, off + (off_t)done);
        if (w <= 0) throw Error(StatusCode::io_error, "write failed for " + name);
        done += (size_t)w;
    }
    p.crc = crc32(data, n, p.crc);
    p.written += n;
}
uint32_t SafetensorsWriter::tensor_crc(const std::string& name) const { return planned_.at(name).crc; }
void SafetensorsWriter::finish() {
    if (!header_written_) write_header();
    for (const auto& n : order_) {
        const auto& p = planned_[n];
        if (p.written != p.spec.end - p.spec.begin) throw Error(StatusCode::format_error, "tensor not fully written: " + n);
    }
    if (fsync(fd_) != 0) throw Error(StatusCode::io_error, "fsync failed");
    ::close(fd_);
    fd_ = -1;
}

// ------------------------------------------------------------------------------------------------ codecs
float e4m3_decode(uint8_t b) {
    const int s = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0) v = std::ldexp((float)m, -9);                   // subnormal: m * 2^-3 * 2^-6
    else if (e == 15 && m == 7) v = NAN;
    else v = std::ldexp(1.0f + (float)m / 8.0f, e - 7);
    return s ? -v : v;
}
uint8_t e4m3_encode(float x) {      // round to nearest even, saturate to +-448
    if (std::isnan(x)) return 0x7F;
    const uint8_t sign = std::signbit(x) ? 0x80 : 0;
    float a = std::fabs(x);
    if (a >= 448.0f) return sign | 0x7E;
    if (a < std::ldexp(1.0f, -10)) return sign;                 // below half the smallest subnormal (2^-9): rounds to 0
    int e;
    std::frexp(a, &e);              // a = f * 2^e, f in [0.5,1) -> exponent of the leading bit is e-1
    int exp = e - 1;
    if (exp < -6) exp = -6;         // subnormal range shares the 2^-6 scale
    const float step = std::ldexp(1.0f, exp - 3);
    float q = a / step;             // in units of the mantissa step (8..15.x for normals, 0..7.x for subnormals)
    float r = std::nearbyint(q);    // default rounding mode = nearest even
    if (r >= 16.0f) { r = 8.0f; ++exp; }
    if (exp > 8 || (exp == 8 && r > 14.0f)) return sign | 0x7E;
    uint8_t code;
    if (r < 8.0f) code = (uint8_t)r;                            // subnormal (exp == -6)
    else code = (uint8_t)(((exp + 7) << 3) | ((int)r - 8));
    return sign | code;
}
float e2m1_decode(uint8_t nib) {
    static const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float v = lut[nib & 7];
    return (nib & 8) ? -v : v;
}
uint8_t e2m1_encode(float x) {      // nearest, midpoints to the even code, saturating; no negative zero
    static const float bounds[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    const float a = std::fabs(x);
    int idx = 0;
    while (idx < 7 && a > bounds[idx]) ++idx;
    if (idx < 7 && a == bounds[idx] && (idx & 1)) ++idx;         // a == bound: candidates idx, idx+1 -> even one
    if (idx == 0) return 0;
    return (uint8_t)(idx | (x < 0 ? 8 : 0));
}
float ue8m0_decode(uint8_t e) { return std::ldexp(1.0f, (int)e - 127); }

void quantize_row_nvfp4(const float* w, int k, int k_padded, float tensor_scale, int search, const float* importance,
                        uint8_t* codes, uint8_t* scales) {
    std::vector<float> blk(16);
    for (int b0 = 0; b0 < k_padded; b0 += 16) {
        float amax = 0.f;
        for (int i = 0; i < 16; ++i) { blk[i] = (b0 + i < k) ? w[b0 + i] : 0.f; amax = std::max(amax, std::fabs(blk[i])); }
        const int base = e4m3_encode(amax / 6.0f / tensor_scale);
        double best_err = 0; int best_sb = 0; uint8_t best_q[16];
        bool have = false;
        for (int step = -search; step <= search; ++step) {
            const int sb = std::min(0x7E, std::max(0, base + step));
            const float s = e4m3_decode((uint8_t)sb) * tensor_scale;
            const float ss = s > 0 ? s : 1.0f;
            double err = 0; uint8_t q[16];
            for (int i = 0; i < 16; ++i) {
                const float r = blk[i] / ss;
                q[i] = e2m1_encode(r);
                const float d = e2m1_decode(q[i]) * s - blk[i];
                const float wgt = (importance && b0 + i < k) ? importance[b0 + i] : 1.0f;
                err += (double)(d * d * wgt);
            }
            if (!have || err < best_err) { have = true; best_err = err; best_sb = sb; memcpy(best_q, q, 16); }
        }
        scales[b0 / 16] = (uint8_t)best_sb;
        for (int i = 0; i < 16; i += 2) codes[(b0 + i) / 2] = (uint8_t)(best_q[i] | (best_q[i + 1] << 4));
    }
}

void quantize_row_mxfp8(const float* w, int k, int k_padded, int search, const float* importance, uint8_t* codes,
                        uint8_t* scales) {
    std::vector<float> blk(32);
    for (int b0 = 0; b0 < k_padded; b0 += 32) {
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) { blk[i] = (b0 + i < k) ? w[b0 + i] : 0.f; amax = std::max(amax, std::fabs(blk[i])); }
        // ceil(log2(amax / 448)) in exact integer arithmetic (the device quantiser computes the same)
        int fe;
        const float fm = std::frexp((amax > 0 ? amax : 1.0f) / 448.0f, &fe);
        const float e0 = (float)(fm == 0.5f ? fe - 1 : fe);
        double best_err = 0; int best_e = 0; uint8_t best_c[32];
        bool have = false;
        for (int step = -search; step <= search; ++step) {
            const int e = std::min(127, std::max(-126, (int)e0 + step));
            const float s = std::ldexp(1.0f, e);
            double err = 0; uint8_t c[32];
            for (int i = 0; i < 32; ++i) {
                c[i] = e4m3_encode(blk[i] / s);
                const float d = e4m3_decode(c[i]) * s - blk[i];
                const float wgt = (importance && b0 + i < k) ? importance[b0 + i] : 1.0f;
                err += (double)(d * d * wgt);
            }
            if (!have || err < best_err) { have = true; best_err = err; best_e = e; memcpy(best_c, c, 32); }
        }
        scales[b0 / 32] = (uint8_t)(best_e + 127);
        memcpy(codes + b0, best_c, 32);
    }
}

// ---- NVFP4 key/value rows (device layout: csrc/include/kv_fp4.cuh; reference counterpart: the 4-bit KV block codec
// include/phaseshift/quantization/psq/psq4_kv.h:1-79).  Row = D/2 code bytes | D/16 UE4M3 block scales | zero padding to a
// multiple of 16 bytes; one fp32 row scale max|row| / (6 * 448) is kept beside it.  The arithmetic is the append kernel's:
// single-precision, correctly rounded multiplications and divisions, nearest-even code rounding.
int kv_nvfp4_row_bytes(int d) { return ((d / 2 + d / 16) + 15) & ~15; }

void kv_nvfp4_encode_row(const float* x, int d, uint8_t* row, float* row_scale) {
    float amax = 0.f;
    for (int i = 0; i < d; ++i) amax = std::max(amax, std::fabs(x[i]));
    const float ts = amax > 0.f ? amax * (1.0f / (6.0f * 448.0f)) : 1.0f;
    memset(row, 0, (size_t)kv_nvfp4_row_bytes(d));
    for (int b = 0; b < d / 16; ++b) {
        float bmax = 0.f;
        for (int i = 0; i < 16; ++i) bmax = std::max(bmax, std::fabs(x[16 * b + i]));
        const uint8_t sf = e4m3_encode(bmax / (6.0f * ts));
        const float sf_f = e4m3_decode(sf);
        const float inv = sf_f > 0.f ? 1.0f / (sf_f * ts) : 0.f;
        for (int i = 0; i < 16; i += 2) {
            const float a = x[16 * b + i] * inv, c = x[16 * b + i + 1] * inv;
            row[(16 * b + i) / 2] = (uint8_t)(e2m1_encode(a) | (e2m1_encode(c) << 4));
        }
        row[d / 2 + b] = sf;
    }
    *row_scale = ts;
}

void kv_nvfp4_decode_row(const uint8_t* row, float row_scale, int d, float* out) {
    for (int i = 0; i < d; ++i) {
        const uint8_t byte = row[i / 2];
        const float sf = e4m3_decode(row[d / 2 + i / 16]);
        out[i] = e2m1_decode((i & 1) ? (byte >> 4) : (byte & 0xF)) * sf * row_scale;
    }
}

}  // namespace psrt
