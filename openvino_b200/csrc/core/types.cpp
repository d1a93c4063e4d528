#include "types.hpp"

#include <mutex>

#include <cstdio>

namespace ovc {

ET et_from_name(const std::string& s) {
    for (int i = 0; i < kNumET; ++i) {
        const auto& inf = et_info(static_cast<ET>(i));
        if (s == inf.name || s == inf.precision) return static_cast<ET>(i);
    }
    std::string l;
    for (char c : s) l.push_back((char)std::tolower((unsigned char)c));
    if (l == "undefined" || l == "unspecified") return ET::dynamic;
    if (l == "bool") return ET::boolean;
    if (l == "fp32") return ET::f32;
    if (l == "fp16") return ET::f16;
    if (l == "fp64") return ET::f64;
    if (l == "bin") return ET::u1;
    for (int i = 0; i < kNumET; ++i)
        if (l == et_info(static_cast<ET>(i)).name) return static_cast<ET>(i);
    throw Error("unknown element type '" + s + "'");
}

// ------------------------------------------------------------------------------------ f16
uint16_t f32_to_f16(float f) {
    const uint32_t x = f32_bits(f);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return uint16_t(sign | 0x7e00u);                 // NaN
    if (ax >= 0x477ff000u) {                                               // rounds to >= 65520 -> inf
        return uint16_t(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) return uint16_t(sign);                           // below half of the smallest subnormal
    int exp = int(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    uint32_t out;
    if (exp < -14) {                                                       // subnormal
        const int shift = -14 - exp + 13;                                  // bits to drop
        const uint32_t rem = man & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        out = man >> shift;
        if (rem > halfway || (rem == halfway && (out & 1u))) ++out;
    } else {
        const uint32_t rem = man & 0x1fffu;
        out = (uint32_t(exp + 15) << 10) | ((man >> 13) & 0x3ffu);
        if (rem > 0x1000u || (rem == 0x1000u && (out & 1u))) ++out;        // may carry into the exponent: fine
    }
    return uint16_t(sign | out);
}

float f16_to_f32(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        int e = -1;
        do { ++e; man <<= 1; } while (!(man & 0x400u));
        return bits_f32(sign | (uint32_t(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13));
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

// Generic small-float encoder: ebits exponent bits, mbits mantissa bits, given bias; saturating
// (no infinities) when `sat` is set, with `max_code` the largest finite magnitude code.
static uint8_t encode_small(float f, int ebits, int mbits, int bias, bool has_inf, uint8_t nan_code, uint8_t max_code) {
    const uint32_t x = f32_bits(f);
    const uint8_t sign = uint8_t((x >> 31) << (ebits + mbits));
    const float a = std::fabs(f);
    if (std::isnan(f)) return uint8_t(sign | nan_code);
    const int emax_code = (1 << ebits) - 1;
    // decode helper for candidate codes
    auto decode = [&](int code) -> float {
        const int e = code >> mbits, m = code & ((1 << mbits) - 1);
        if (e == 0) return std::ldexp(float(m), 1 - bias - mbits);
        return std::ldexp(float((1 << mbits) + m), e - bias - mbits);
    };
    const float maxv = decode(max_code);
    if (std::isinf(f) || a > maxv) {
        if (has_inf) {
            // round to nearest: values beyond max + half ulp go to infinity
            const float ulp = decode(max_code) - decode(max_code - 1);
            if (std::isinf(f) || a >= maxv + ulp * 0.5f) return uint8_t(sign | (emax_code << mbits));
            return uint8_t(sign | max_code);
        }
        return uint8_t(sign | max_code);
    }
    // binary search over monotonically increasing codes 0..max_code
    int lo = 0, hi = max_code;
    while (hi - lo > 1) {
        const int mid = (lo + hi) / 2;
        if (decode(mid) <= a) lo = mid; else hi = mid;
    }
    const float dl = a - decode(lo), dh = decode(hi) - a;
    int code = lo;
    if (dh < dl || (dh == dl && (hi & 1) == 0)) code = hi;
    if (a <= 0.f) code = 0;
    return uint8_t(sign | code);
}
static float decode_small(uint8_t v, int ebits, int mbits, int bias) {
    const int code = v & ((1 << (ebits + mbits)) - 1);
    const bool neg = (v >> (ebits + mbits)) & 1;
    const int e = code >> mbits, m = code & ((1 << mbits) - 1);
    float r = (e == 0) ? std::ldexp(float(m), 1 - bias - mbits) : std::ldexp(float((1 << mbits) + m), e - bias - mbits);
    return neg ? -r : r;
}

uint8_t f32_to_f8e4m3(float f) { return encode_small(f, 4, 3, 7, false, 0x7f, 0x7e); }
float f8e4m3_to_f32(uint8_t v) {
    if ((v & 0x7f) == 0x7f) return std::numeric_limits<float>::quiet_NaN();
    return decode_small(v, 4, 3, 7);
}
uint8_t f32_to_f8e5m2(float f) { return encode_small(f, 5, 2, 15, true, 0x7f, 0x7b); }
float f8e5m2_to_f32(uint8_t v) {
    const int code = v & 0x7f;
    if (code == 0x7c) return (v & 0x80) ? -std::numeric_limits<float>::infinity() : std::numeric_limits<float>::infinity();
    if (code > 0x7c) return std::numeric_limits<float>::quiet_NaN();
    return decode_small(v, 5, 2, 15);
}
uint8_t f32_to_f8e8m0(float f) {
    if (std::isnan(f)) return 0xff;
    if (f <= 0.f) return 0;
    int e;
    const float m = std::frexp(f, &e);    // f = m * 2^e, m in [0.5, 1)
    int code = e - 1 + 127;
    if (m > 0.70710678f) ++code;          // round to the nearest power of two in the log domain
    return uint8_t(std::min(std::max(code, 0), 254));
}
float f8e8m0_to_f32(uint8_t v) {
    if (v == 0xff) return std::numeric_limits<float>::quiet_NaN();
    return std::ldexp(1.0f, int(v) - 127);
}
uint8_t f32_to_f4e2m1(float f) { return encode_small(f, 2, 1, 1, false, 0x7, 0x7) & 0xf; }
float f4e2m1_to_f32(uint8_t nib) { return decode_small(nib & 0xf, 2, 1, 1); }

static const float kNF4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                               -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                               0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                               0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
float nf4_to_f32(uint8_t nib) { return kNF4[nib & 0xf]; }
uint8_t f32_to_nf4(float f) {
    int best = 0;
    float bd = std::fabs(f - kNF4[0]);
    for (int i = 1; i < 16; ++i) {
        const float d = std::fabs(f - kNF4[i]);
        if (d < bd) { bd = d; best = i; }
    }
    return uint8_t(best);
}

// ------------------------------------------------------------------------------------ strings
std::string Dim::str() const {
    if (is_static()) return std::to_string(lo);
    if (lo > 0) return std::to_string(lo) + ".." + (hi >= 0 ? std::to_string(hi) : std::string());
    if (hi >= 0) return ".." + std::to_string(hi);
    return "?";
}

std::string PShape::str() const {
    if (rank_dynamic) return "[...]";
    return "[" + ir_str() + "]";
}
std::string PShape::ir_str() const {
    if (rank_dynamic) return "...";
    std::string s;
    for (size_t i = 0; i < dims.size(); ++i) {
        if (i) s += ",";
        s += dims[i].str();
    }
    return s;
}

static Dim parse_dim(const std::string& t0) {
    const std::string t = trim(t0);
    OVC_CHECK(!t.empty(), "empty dimension");
    if (t == "?" || t == "-1") return Dim::dynamic();
    const auto p = t.find("..");
    if (p == std::string::npos) return Dim(std::stoll(t));
    const std::string a = trim(t.substr(0, p)), b = trim(t.substr(p + 2));
    return Dim(a.empty() ? 0 : std::stoll(a), b.empty() ? -1 : std::stoll(b));
}

PShape PShape::parse(const std::string& s0) {
    std::string s = trim(s0);
    if (!s.empty() && s.front() == '[' && s.back() == ']') s = s.substr(1, s.size() - 2);
    s = trim(s);
    if (s == "...") return PShape::dynamic();
    PShape p;
    if (s.empty()) return p;
    for (auto& t : split(s, ',')) p.dims.push_back(parse_dim(t));
    return p;
}

std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    std::string cur;
    for (char c : s) {
        if (c == sep) { out.push_back(cur); cur.clear(); } else cur.push_back(c);
    }
    out.push_back(cur);
    return out;
}
std::string join(const std::vector<std::string>& v, const std::string& sep) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) { if (i) s += sep; s += v[i]; }
    return s;
}
std::string trim(const std::string& s) {
    size_t b = 0, e = s.size();
    while (b < e && std::isspace((unsigned char)s[b])) ++b;
    while (e > b && std::isspace((unsigned char)s[e - 1])) --e;
    return s.substr(b, e - b);
}

std::string format_double(double v) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "%.17g", v);
    return buf;
}

static std::string format_stream_float(double v) {
    // default ostream formatting of a float: %g with 6 significant digits
    char buf[64];
    std::snprintf(buf, sizeof(buf), "%g", v);
    return buf;
}

bool Attr::operator==(const Attr& o) const {
    if (kind != o.kind) return false;
    switch (kind) {
        case NONE: return true;
        case BOOL: case INT: return i == o.i;
        case FLOAT: return f == o.f || (std::isnan(f) && std::isnan(o.f));
        case STR: return s == o.s;
        case INTS: return is == o.is;
        case FLOATS: return fs == o.fs;
        case STRS: return ss == o.ss;
        case TYPE: return et == o.et;
        case PSHAPE: return ps == o.ps;
        case MAP: return (!map && !o.map) || (map && o.map && *map == *o.map);
    }
    return false;
}

std::string Attr::to_string() const {
    switch (kind) {
        case NONE: return "";
        case BOOL: return i ? "true" : "false";
        case INT: return std::to_string(i);
        case FLOAT: return format_double(f);
        case STR: return s;
        case INTS: {
            std::string r;
            for (size_t k = 0; k < is.size(); ++k) { if (k) r += ", "; r += std::to_string(is[k]); }
            return r;
        }
        case FLOATS: {
            std::string r;
            for (size_t k = 0; k < fs.size(); ++k) { if (k) r += ", "; r += format_stream_float(fs[k]); }
            return r;
        }
        case STRS: return join(ss, ", ");
        case TYPE: return et_name(et);
        case PSHAPE: return ps.ir_str();
        case MAP: return "";
    }
    return "";
}

Attr Attr::from_string(Kind k, const std::string& v) {
    switch (k) {
        case BOOL: {
            std::string l;
            for (char c : v) l.push_back((char)std::tolower((unsigned char)c));
            return Bool(l == "true" || l == "1");
        }
        case INT: return Int(v.empty() ? 0 : std::stoll(v));
        case FLOAT: return Float(v.empty() ? 0.0 : std::stod(v));
        case STR: return Str(v);
        case INTS: {
            std::vector<int64_t> r;
            if (!trim(v).empty()) for (auto& t : split(v, ',')) r.push_back(std::stoll(trim(t)));
            return Ints(r);
        }
        case FLOATS: {
            std::vector<double> r;
            if (!trim(v).empty()) for (auto& t : split(v, ',')) r.push_back(std::stod(trim(t)));
            return Floats(r);
        }
        case STRS: {
            std::vector<std::string> r;
            if (!trim(v).empty()) for (auto& t : split(v, ',')) r.push_back(trim(t));
            return Strs(r);
        }
        case TYPE: return Type(et_from_name(v));
        case PSHAPE: return Shape_(PShape::parse(v));
        default: return Str(v);
    }
}

// ---- symbol table: union-find over symbol ids (1-based; id 0 = no symbol)
namespace {
std::mutex g_sym_mu;
std::vector<int64_t> g_sym_parent{0};
int64_t sym_find(int64_t s) {
    while (g_sym_parent[(size_t)s] != s) {
        g_sym_parent[(size_t)s] = g_sym_parent[(size_t)g_sym_parent[(size_t)s]];
        s = g_sym_parent[(size_t)s];
    }
    return s;
}
}  // namespace

int64_t new_symbol() {
    std::lock_guard<std::mutex> lk(g_sym_mu);
    g_sym_parent.push_back((int64_t)g_sym_parent.size());
    return (int64_t)g_sym_parent.size() - 1;
}
int64_t symbol_root(int64_t sym) {
    std::lock_guard<std::mutex> lk(g_sym_mu);
    if (sym <= 0 || sym >= (int64_t)g_sym_parent.size()) return 0;
    return sym_find(sym);
}
void symbols_set_equal(int64_t a, int64_t b) {
    std::lock_guard<std::mutex> lk(g_sym_mu);
    if (a <= 0 || b <= 0 || a >= (int64_t)g_sym_parent.size() || b >= (int64_t)g_sym_parent.size()) return;
    const int64_t ra = sym_find(a), rb = sym_find(b);
    if (ra != rb) g_sym_parent[(size_t)std::max(ra, rb)] = std::min(ra, rb);
}

}  // namespace ovc
