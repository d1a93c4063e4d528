// Element types, low-precision float codecs, shapes and attribute values of the native core.
//
// Covers the roles of ov::element::Type (src/core/include/openvino/core/type/element_type.hpp:31-58),
// the scalar classes under src/core/src/type/ (float16, bfloat16, float8_e4m3, float8_e5m2, float8_e8m0,
// float4_e2m1, nf4), ov::Dimension / ov::PartialShape (src/core/src/{dimension,partial_shape}.cpp) and
// ov::Any as far as attributes go (src/core/include/openvino/core/any.hpp).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace ovc {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

#define OVC_CHECK(cond, msg)                                         \
    do {                                                             \
        if (!(cond)) {                                               \
            std::ostringstream _os;                                  \
            _os << msg;                                              \
            throw ::ovc::Error(_os.str());                           \
        }                                                            \
    } while (0)

// ------------------------------------------------------------------------------------ element types
enum class ET : uint8_t {
    dynamic, boolean, bf16, f16, f32, f64, i4, i8, i16, i32, i64, u1, u2, u3, u4, u6, u8, u16, u32, u64, nf4,
    f8e4m3, f8e5m2, string, f4e2m1, f8e8m0,
};
constexpr int kNumET = 26;

struct ETInfo {
    const char* name;       // "f32"
    const char* precision;  // IR port precision string "FP32"
    int bits;
    bool is_real, is_signed, is_quantized;
};

inline const ETInfo& et_info(ET t) {
    static const ETInfo tbl[kNumET] = {
        {"dynamic", "UNSPECIFIED", 0, false, false, false}, {"boolean", "BOOL", 8, false, true, false},
        {"bf16", "BF16", 16, true, true, false},           {"f16", "FP16", 16, true, true, false},
        {"f32", "FP32", 32, true, true, false},            {"f64", "FP64", 64, true, true, false},
        {"i4", "I4", 4, false, true, true},                {"i8", "I8", 8, false, true, true},
        {"i16", "I16", 16, false, true, false},            {"i32", "I32", 32, false, true, true},
        {"i64", "I64", 64, false, true, false},            {"u1", "BIN", 1, false, false, false},
        {"u2", "U2", 2, false, false, false},              {"u3", "U3", 3, false, false, false},
        {"u4", "U4", 4, false, false, false},              {"u6", "U6", 6, false, false, false},
        {"u8", "U8", 8, false, false, true},               {"u16", "U16", 16, false, false, false},
        {"u32", "U32", 32, false, false, false},           {"u64", "U64", 64, false, false, false},
        {"nf4", "NF4", 4, true, true, true},               {"f8e4m3", "F8E4M3", 8, true, true, true},
        {"f8e5m2", "F8E5M2", 8, true, true, true},         {"string", "STRING", 8 * (int)sizeof(std::string), false, false, false},
        {"f4e2m1", "F4E2M1", 4, true, true, true},         {"f8e8m0", "F8E8M0", 8, true, true, true},
    };
    return tbl[static_cast<int>(t)];
}
inline const char* et_name(ET t) { return et_info(t).name; }
inline int et_bits(ET t) { return et_info(t).bits; }
inline bool et_is_real(ET t) { return et_info(t).is_real; }
inline bool et_is_integral(ET t) { return !et_info(t).is_real && t != ET::dynamic && t != ET::string; }
ET et_from_name(const std::string& s);        // "f32", also the IR precision spellings ("FP32", "I64", ...)
// bytes needed for n elements (sub-byte types are packed, LSB first except u1 which is MSB first)
inline size_t et_byte_size(ET t, size_t n) {
    const int b = et_bits(t);
    if (t == ET::u3) return 3 * ((n + 7) / 8);
    if (t == ET::u6) return 3 * ((n + 3) / 4);
    return (n * (size_t)b + 7) / 8;
}

// ------------------------------------------------------------------------------------ float codecs
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);   // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);                                           // round to nearest even
    return uint16_t(u >> 16);
}
inline float bf16_to_f32(uint16_t h) { return bits_f32(uint32_t(h) << 16); }
uint16_t f32_to_f16(float f);
float f16_to_f32(uint16_t h);
uint8_t f32_to_f8e4m3(float f);
float f8e4m3_to_f32(uint8_t v);
uint8_t f32_to_f8e5m2(float f);
float f8e5m2_to_f32(uint8_t v);
uint8_t f32_to_f8e8m0(float f);
float f8e8m0_to_f32(uint8_t v);
uint8_t f32_to_f4e2m1(float f);   // returns a nibble
float f4e2m1_to_f32(uint8_t nib);
float nf4_to_f32(uint8_t nib);
uint8_t f32_to_nf4(float f);

// ------------------------------------------------------------------------------------ shapes
using Shape = std::vector<int64_t>;
inline int64_t shape_size(const Shape& s) {
    int64_t n = 1;
    for (auto d : s) n *= d;
    return n;
}

// Symbols: a dynamic dimension may carry a symbol; dimensions whose symbols are equal (same class of the table below) are
// known to have the same run-time value. Shape inference copies dimensions, so a symbol travels with its dimension; merging
// two dimensions (Concat / element-wise operands that must agree) makes their symbols equal. Role in the reference:
// ov::Symbol and ov::symbol::set_equal / are_equal, src/core/include/openvino/core/symbol.hpp.
int64_t new_symbol();
int64_t symbol_root(int64_t sym);
void symbols_set_equal(int64_t a, int64_t b);
inline bool symbols_equal(int64_t a, int64_t b) { return a != 0 && b != 0 && symbol_root(a) == symbol_root(b); }

struct Dim {
    int64_t lo = 0;
    int64_t hi = -1;   // -1: unbounded
    int64_t sym = 0;   // 0: no symbol
    Dim() = default;
    Dim(int64_t v) : lo(v < 0 ? 0 : v), hi(v < 0 ? -1 : v) {}
    Dim(int64_t l, int64_t h) : lo(l), hi(h) {}
    static Dim dynamic() { return Dim(0, -1); }
    bool is_static() const { return lo == hi; }
    bool is_dynamic() const { return !is_static(); }
    int64_t get() const { return lo; }
    bool operator==(const Dim& o) const { return lo == o.lo && hi == o.hi; }
    bool operator!=(const Dim& o) const { return !(*this == o); }
    bool compatible(const Dim& o) const {
        const int64_t l = std::max(lo, o.lo);
        const int64_t h = (hi < 0) ? o.hi : (o.hi < 0 ? hi : std::min(hi, o.hi));
        return h < 0 || l <= h;
    }
    // intersection; throws when empty
    static bool merge(Dim& dst, const Dim& a, const Dim& b) {
        const int64_t l = std::max(a.lo, b.lo);
        const int64_t h = (a.hi < 0) ? b.hi : (b.hi < 0 ? a.hi : std::min(a.hi, b.hi));
        if (h >= 0 && l > h) return false;
        const int64_t sa = a.sym, sb = b.sym;
        dst = Dim(l, h);
        if (dst.is_dynamic()) {
            dst.sym = sa ? sa : sb;
            if (sa && sb && sa != sb) symbols_set_equal(sa, sb);      // the two dimensions must agree: one class from now on
        }
        return true;
    }
    std::string str() const;   // "3", "-1" / "?" handled by callers, "1..8", "..8", "2.."
};
inline Dim operator+(const Dim& a, const Dim& b) {
    return Dim(a.lo + b.lo, (a.hi < 0 || b.hi < 0) ? -1 : a.hi + b.hi);
}
inline Dim operator*(const Dim& a, const Dim& b) {
    return Dim(a.lo * b.lo, (a.hi < 0 || b.hi < 0) ? -1 : a.hi * b.hi);
}

struct PShape {
    bool rank_dynamic = false;
    std::vector<Dim> dims;
    PShape() = default;
    PShape(const Shape& s) { for (auto d : s) dims.emplace_back(d); }
    PShape(std::vector<Dim> d) : dims(std::move(d)) {}
    PShape(std::initializer_list<Dim> d) : dims(d) {}
    static PShape dynamic() { PShape p; p.rank_dynamic = true; return p; }
    static PShape dynamic(size_t rank) { PShape p; p.dims.assign(rank, Dim::dynamic()); return p; }
    bool rank_is_static() const { return !rank_dynamic; }
    size_t rank() const { return dims.size(); }
    bool is_static() const {
        if (rank_dynamic) return false;
        for (auto& d : dims) if (!d.is_static()) return false;
        return true;
    }
    bool is_dynamic() const { return !is_static(); }
    Shape to_shape() const {
        OVC_CHECK(is_static(), "to_shape() called on a dynamic shape " << str());
        Shape s;
        for (auto& d : dims) s.push_back(d.lo);
        return s;
    }
    Shape max_shape() const { Shape s; for (auto& d : dims) s.push_back(d.hi); return s; }
    Shape min_shape() const { Shape s; for (auto& d : dims) s.push_back(d.lo); return s; }
    bool operator==(const PShape& o) const { return rank_dynamic == o.rank_dynamic && dims == o.dims; }
    bool operator!=(const PShape& o) const { return !(*this == o); }
    bool compatible(const PShape& o) const {
        if (rank_dynamic || o.rank_dynamic) return true;
        if (dims.size() != o.dims.size()) return false;
        for (size_t i = 0; i < dims.size(); ++i) if (!dims[i].compatible(o.dims[i])) return false;
        return true;
    }
    static bool merge(PShape& dst, const PShape& a, const PShape& b) {
        if (a.rank_dynamic) { dst = b; return true; }
        if (b.rank_dynamic) { dst = a; return true; }
        if (a.dims.size() != b.dims.size()) return false;
        PShape r = a;
        for (size_t i = 0; i < a.dims.size(); ++i) if (!Dim::merge(r.dims[i], a.dims[i], b.dims[i])) return false;
        dst = r;
        return true;
    }
    std::string str() const;                       // "[1,3,?,224]" / "[...]"
    std::string ir_str() const;                    // "1,3,-1,224" / "..." (IR attribute spelling)
    static PShape parse(const std::string& s);     // accepts both spellings
};

// ------------------------------------------------------------------------------------ attribute value
struct Attr;
using AttrMap = std::map<std::string, Attr>;

struct Attr {
    enum Kind : uint8_t { NONE, BOOL, INT, FLOAT, STR, INTS, FLOATS, STRS, TYPE, PSHAPE, MAP };
    Kind kind = NONE;
    int64_t i = 0;
    double f = 0;
    std::string s;
    std::vector<int64_t> is;
    std::vector<double> fs;
    std::vector<std::string> ss;
    ET et = ET::dynamic;
    PShape ps;
    std::shared_ptr<AttrMap> map;

    Attr() = default;
    static Attr Bool(bool v) { Attr a; a.kind = BOOL; a.i = v; return a; }
    static Attr Int(int64_t v) { Attr a; a.kind = INT; a.i = v; return a; }
    static Attr Float(double v) { Attr a; a.kind = FLOAT; a.f = v; return a; }
    static Attr Str(std::string v) { Attr a; a.kind = STR; a.s = std::move(v); return a; }
    static Attr Ints(std::vector<int64_t> v) { Attr a; a.kind = INTS; a.is = std::move(v); return a; }
    static Attr Floats(std::vector<double> v) { Attr a; a.kind = FLOATS; a.fs = std::move(v); return a; }
    static Attr Strs(std::vector<std::string> v) { Attr a; a.kind = STRS; a.ss = std::move(v); return a; }
    static Attr Type(ET v) { Attr a; a.kind = TYPE; a.et = v; return a; }
    static Attr Shape_(PShape v) { Attr a; a.kind = PSHAPE; a.ps = std::move(v); return a; }
    static Attr Map(AttrMap m) { Attr a; a.kind = MAP; a.map = std::make_shared<AttrMap>(std::move(m)); return a; }
    bool operator==(const Attr& o) const;
    bool operator!=(const Attr& o) const { return !(*this == o); }
    // string spelling used in IR xml attributes (ints joined with ",", floats via shortest round-trip, ...)
    std::string to_string() const;
    // parse from the xml spelling given the expected kind
    static Attr from_string(Kind k, const std::string& s);
};

std::string format_double(double v);   // the number formatting of xml attribute values
std::vector<std::string> split(const std::string& s, char sep);
std::string join(const std::vector<std::string>& v, const std::string& sep);
std::string trim(const std::string& s);

}  // namespace ovc
