#include "graph.hpp"

#include <chrono>
#include <stack>

namespace ovc {

// ------------------------------------------------------------------------------------ element access
static inline int sub_bits(ET t) { return et_bits(t); }

static uint32_t get_packed(const uint8_t* p, ET t, int64_t i) {
    switch (t) {
        case ET::u1: return (p[i >> 3] >> (7 - (i & 7))) & 1u;                 // MSB first
        case ET::u2: return (p[i >> 2] >> ((i & 3) * 2)) & 3u;                 // LSB first
        case ET::u4: case ET::i4: case ET::nf4: case ET::f4e2m1: return (p[i >> 1] >> ((i & 1) * 4)) & 0xFu;
        case ET::u3: {   // 8 values in 3 bytes: bytes 0,1 hold the two low bits of 8 values, byte 2 the high bits
            const uint8_t* g = p + (i >> 3) * 3;
            const int k = int(i & 7);
            const uint32_t lo = (g[k >> 2] >> (6 - 2 * (k & 3))) & 3u;
            const uint32_t hi = (g[2] >> (7 - k)) & 1u;
            return (hi << 2) | lo;
        }
        case ET::u6: {   // 4 values in 3 bytes: bytes 0,1 hold low nibbles, byte 2 the two high bits of each
            const uint8_t* g = p + (i >> 2) * 3;
            const int k = int(i & 3);
            const uint32_t lo = (g[k >> 1] >> (4 - 4 * (k & 1))) & 0xFu;
            const uint32_t hi = (g[2] >> (6 - 2 * k)) & 3u;
            return (hi << 4) | lo;
        }
        default: return 0;
    }
}
static void set_packed(uint8_t* p, ET t, int64_t i, uint32_t v) {
    switch (t) {
        case ET::u1: { const int sh = 7 - int(i & 7); p[i >> 3] = uint8_t((p[i >> 3] & ~(1u << sh)) | ((v & 1u) << sh)); break; }
        case ET::u2: { const int sh = int(i & 3) * 2; p[i >> 2] = uint8_t((p[i >> 2] & ~(3u << sh)) | ((v & 3u) << sh)); break; }
        case ET::u4: case ET::i4: case ET::nf4: case ET::f4e2m1: {
            const int sh = int(i & 1) * 4;
            p[i >> 1] = uint8_t((p[i >> 1] & ~(0xFu << sh)) | ((v & 0xFu) << sh));
            break;
        }
        case ET::u3: {
            uint8_t* g = p + (i >> 3) * 3;
            const int k = int(i & 7);
            const int sh = 6 - 2 * (k & 3);
            g[k >> 2] = uint8_t((g[k >> 2] & ~(3u << sh)) | ((v & 3u) << sh));
            g[2] = uint8_t((g[2] & ~(1u << (7 - k))) | (((v >> 2) & 1u) << (7 - k)));
            break;
        }
        case ET::u6: {
            uint8_t* g = p + (i >> 2) * 3;
            const int k = int(i & 3);
            const int sh = 4 - 4 * (k & 1);
            g[k >> 1] = uint8_t((g[k >> 1] & ~(0xFu << sh)) | ((v & 0xFu) << sh));
            g[2] = uint8_t((g[2] & ~(3u << (6 - 2 * k))) | (((v >> 4) & 3u) << (6 - 2 * k)));
            break;
        }
        default: break;
    }
}

double get_elem_f64(const Tensor& t, int64_t i) {
    const uint8_t* p = t.data();
    switch (t.et) {
        case ET::boolean: return p[i] ? 1.0 : 0.0;
        case ET::bf16: return bf16_to_f32(reinterpret_cast<const uint16_t*>(p)[i]);
        case ET::f16: return f16_to_f32(reinterpret_cast<const uint16_t*>(p)[i]);
        case ET::f32: return reinterpret_cast<const float*>(p)[i];
        case ET::f64: return reinterpret_cast<const double*>(p)[i];
        case ET::i8: return reinterpret_cast<const int8_t*>(p)[i];
        case ET::i16: return reinterpret_cast<const int16_t*>(p)[i];
        case ET::i32: return reinterpret_cast<const int32_t*>(p)[i];
        case ET::i64: return double(reinterpret_cast<const int64_t*>(p)[i]);
        case ET::u8: return p[i];
        case ET::u16: return reinterpret_cast<const uint16_t*>(p)[i];
        case ET::u32: return reinterpret_cast<const uint32_t*>(p)[i];
        case ET::u64: return double(reinterpret_cast<const uint64_t*>(p)[i]);
        case ET::i4: { int v = int(get_packed(p, t.et, i)); return v >= 8 ? v - 16 : v; }
        case ET::u1: case ET::u2: case ET::u3: case ET::u4: case ET::u6: return get_packed(p, t.et, i);
        case ET::nf4: return nf4_to_f32(uint8_t(get_packed(p, t.et, i)));
        case ET::f4e2m1: return f4e2m1_to_f32(uint8_t(get_packed(p, t.et, i)));
        case ET::f8e4m3: return f8e4m3_to_f32(p[i]);
        case ET::f8e5m2: return f8e5m2_to_f32(p[i]);
        case ET::f8e8m0: return f8e8m0_to_f32(p[i]);
        default: throw Error(std::string("get_elem: unsupported element type ") + et_name(t.et));
    }
}
int64_t get_elem_i64(const Tensor& t, int64_t i) {
    const uint8_t* p = t.data();
    switch (t.et) {
        case ET::i64: return reinterpret_cast<const int64_t*>(p)[i];
        case ET::u64: return int64_t(reinterpret_cast<const uint64_t*>(p)[i]);
        case ET::i32: return reinterpret_cast<const int32_t*>(p)[i];
        default: {
            const double d = get_elem_f64(t, i);
            return int64_t(d);
        }
    }
}
template <class T> static T sat_cast(double v) {
    if (std::isnan(v)) return T(0);
    const double lo = double(std::numeric_limits<T>::lowest()), hi = double(std::numeric_limits<T>::max());
    if (v <= lo) return std::numeric_limits<T>::lowest();
    if (v >= hi) return std::numeric_limits<T>::max();
    return T(v);
}
void set_elem_f64(Tensor& t, int64_t i, double v) {
    uint8_t* p = t.data();
    switch (t.et) {
        case ET::boolean: p[i] = v != 0.0; break;
        case ET::bf16: reinterpret_cast<uint16_t*>(p)[i] = f32_to_bf16(float(v)); break;
        case ET::f16: reinterpret_cast<uint16_t*>(p)[i] = f32_to_f16(float(v)); break;
        case ET::f32: reinterpret_cast<float*>(p)[i] = float(v); break;
        case ET::f64: reinterpret_cast<double*>(p)[i] = v; break;
        case ET::i8: reinterpret_cast<int8_t*>(p)[i] = sat_cast<int8_t>(v); break;
        case ET::i16: reinterpret_cast<int16_t*>(p)[i] = sat_cast<int16_t>(v); break;
        case ET::i32: reinterpret_cast<int32_t*>(p)[i] = sat_cast<int32_t>(v); break;
        case ET::i64: reinterpret_cast<int64_t*>(p)[i] = sat_cast<int64_t>(v); break;
        case ET::u8: p[i] = sat_cast<uint8_t>(v); break;
        case ET::u16: reinterpret_cast<uint16_t*>(p)[i] = sat_cast<uint16_t>(v); break;
        case ET::u32: reinterpret_cast<uint32_t*>(p)[i] = sat_cast<uint32_t>(v); break;
        case ET::u64: reinterpret_cast<uint64_t*>(p)[i] = sat_cast<uint64_t>(v); break;
        case ET::i4: set_packed(p, t.et, i, uint32_t(int(std::max(-8.0, std::min(7.0, v)))) & 0xF); break;
        case ET::u1: case ET::u2: case ET::u3: case ET::u4: case ET::u6: {
            const double mx = double((1u << sub_bits(t.et)) - 1u);
            set_packed(p, t.et, i, uint32_t(std::max(0.0, std::min(mx, v))));
            break;
        }
        case ET::nf4: set_packed(p, t.et, i, f32_to_nf4(float(v))); break;
        case ET::f4e2m1: set_packed(p, t.et, i, f32_to_f4e2m1(float(v))); break;
        case ET::f8e4m3: p[i] = f32_to_f8e4m3(float(v)); break;
        case ET::f8e5m2: p[i] = f32_to_f8e5m2(float(v)); break;
        case ET::f8e8m0: p[i] = f32_to_f8e8m0(float(v)); break;
        default: throw Error(std::string("set_elem: unsupported element type ") + et_name(t.et));
    }
}
void set_elem_i64(Tensor& t, int64_t i, int64_t v) {
    switch (t.et) {
        case ET::i64: t.ptr<int64_t>()[i] = v; break;
        case ET::u64: t.ptr<uint64_t>()[i] = uint64_t(v); break;
        case ET::i32: t.ptr<int32_t>()[i] = int32_t(v); break;
        default: set_elem_f64(t, i, double(v));
    }
}

std::vector<float> to_f32(const Tensor& t) {
    const int64_t n = t.numel();
    std::vector<float> v((size_t)n);
    if (t.et == ET::f32) { if (n) std::memcpy(v.data(), t.data(), (size_t)n * 4); return v; }
    for (int64_t i = 0; i < n; ++i) v[(size_t)i] = float(get_elem_f64(t, i));
    return v;
}
std::vector<double> to_f64(const Tensor& t) {
    const int64_t n = t.numel();
    std::vector<double> v((size_t)n);
    for (int64_t i = 0; i < n; ++i) v[(size_t)i] = get_elem_f64(t, i);
    return v;
}
std::vector<int64_t> to_i64(const Tensor& t) {
    const int64_t n = t.numel();
    std::vector<int64_t> v((size_t)n);
    for (int64_t i = 0; i < n; ++i) v[(size_t)i] = get_elem_i64(t, i);
    return v;
}
Tensor from_f32(ET et, const Shape& s, const std::vector<float>& v) {
    Tensor t(et, s);
    OVC_CHECK((int64_t)v.size() == t.numel(), "from_f32: size mismatch");
    if (et == ET::f32) { if (!v.empty()) std::memcpy(t.data(), v.data(), v.size() * 4); return t; }
    for (size_t i = 0; i < v.size(); ++i) set_elem_f64(t, (int64_t)i, v[i]);
    return t;
}
Tensor from_f64(ET et, const Shape& s, const std::vector<double>& v) {
    Tensor t(et, s);
    OVC_CHECK((int64_t)v.size() == t.numel(), "from_f64: size mismatch");
    for (size_t i = 0; i < v.size(); ++i) set_elem_f64(t, (int64_t)i, v[i]);
    return t;
}
Tensor from_i64(ET et, const Shape& s, const std::vector<int64_t>& v) {
    Tensor t(et, s);
    OVC_CHECK((int64_t)v.size() == t.numel(), "from_i64: size mismatch");
    for (size_t i = 0; i < v.size(); ++i) set_elem_i64(t, (int64_t)i, v[i]);
    return t;
}
Tensor convert_tensor(const Tensor& t, ET to) {
    if (t.et == to) return t;
    Tensor r(to, t.shape);
    const int64_t n = t.numel();
    const bool int_path = et_is_integral(t.et) && et_is_integral(to) && t.et != ET::boolean;
    if (to == ET::boolean) {
        for (int64_t i = 0; i < n; ++i) r.data()[i] = get_elem_f64(t, i) != 0.0;
    } else if (int_path) {
        // integer -> integer wraps (two's complement) like a C cast for 8..64 bit targets
        for (int64_t i = 0; i < n; ++i) {
            const int64_t v = get_elem_i64(t, i);
            switch (to) {
                case ET::i8: r.ptr<int8_t>()[i] = int8_t(v); break;
                case ET::i16: r.ptr<int16_t>()[i] = int16_t(v); break;
                case ET::i32: r.ptr<int32_t>()[i] = int32_t(v); break;
                case ET::i64: r.ptr<int64_t>()[i] = v; break;
                case ET::u8: r.ptr<uint8_t>()[i] = uint8_t(v); break;
                case ET::u16: r.ptr<uint16_t>()[i] = uint16_t(v); break;
                case ET::u32: r.ptr<uint32_t>()[i] = uint32_t(v); break;
                case ET::u64: r.ptr<uint64_t>()[i] = uint64_t(v); break;
                default: set_elem_i64(r, i, v);
            }
        }
    } else if (et_is_integral(to) && to != ET::boolean) {
        for (int64_t i = 0; i < n; ++i) set_elem_f64(r, i, std::trunc(get_elem_f64(t, i)));
    } else {
        for (int64_t i = 0; i < n; ++i) set_elem_f64(r, i, get_elem_f64(t, i));
    }
    return r;
}

// ------------------------------------------------------------------------------------ Output / Node
const PShape& Output::shape() const { return node->outs.at(index).shape; }
ET Output::et() const { return node->outs.at(index).et; }

static std::atomic<uint64_t> g_node_id{0};
uint64_t next_node_id() { return g_node_id.fetch_add(1); }

Node::Node(const OpSchema* s, std::vector<Output> inputs, std::vector<std::pair<std::string, Attr>> a)
    : schema(s), type(s->type), version(s->version), id(next_node_id()), attrs(std::move(a)), inputs_(std::move(inputs)) {
    name = type + "_" + std::to_string(id);
    input_rt.resize(inputs_.size());
    for (size_t i = 0; i < inputs_.size(); ++i) attach(i);
    outs.resize(1);
}
Node::~Node() {
    for (size_t i = 0; i < inputs_.size(); ++i) detach(i);
}
void Node::attach(size_t i) {
    auto& o = inputs_[i];
    if (o.node) o.node->outs.at(o.index).uses.push_back(Use{this, i});
}
void Node::detach(size_t i) {
    auto& o = inputs_[i];
    if (!o.node) return;
    auto& uses = o.node->outs.at(o.index).uses;
    for (size_t k = 0; k < uses.size(); ++k)
        if (uses[k].node == this && uses[k].input == i) { uses.erase(uses.begin() + (long)k); break; }
}
void Node::set_input(size_t i, const Output& src) {
    OVC_CHECK(i < inputs_.size(), "set_input: index out of range on " << name);
    detach(i);
    inputs_[i] = src;
    attach(i);
}
void Node::add_input(const Output& src) {
    inputs_.push_back(src);
    input_rt.emplace_back();
    attach(inputs_.size() - 1);
}
void Node::remove_inputs_from(size_t first) {
    while (inputs_.size() > first) {
        detach(inputs_.size() - 1);
        inputs_.pop_back();
        input_rt.pop_back();
    }
}
void Node::set_output(size_t i, ET et, const PShape& s) {
    if (outs.size() <= i) outs.resize(i + 1);
    outs[i].et = et;
    outs[i].shape = s;
}
bool Node::has_attr(const std::string& k) const {
    for (auto& kv : attrs) if (kv.first == k) return true;
    return false;
}
const Attr& Node::attr(const std::string& k) const {
    for (auto& kv : attrs) if (kv.first == k) return kv.second;
    throw Error("node " + name + " (" + type + ") has no attribute '" + k + "'");
}
Attr* Node::find_attr(const std::string& k) {
    for (auto& kv : attrs) if (kv.first == k) return &kv.second;
    return nullptr;
}
void Node::set_attr(const std::string& k, Attr v) {
    if (auto* a = find_attr(k)) { *a = std::move(v); return; }
    attrs.emplace_back(k, std::move(v));
}
int64_t Node::attr_int(const std::string& k, int64_t d) const {
    for (auto& kv : attrs) if (kv.first == k) return kv.second.kind == Attr::FLOAT ? int64_t(kv.second.f) : kv.second.i;
    return d;
}
double Node::attr_float(const std::string& k, double d) const {
    for (auto& kv : attrs) if (kv.first == k) return kv.second.kind == Attr::FLOAT ? kv.second.f : double(kv.second.i);
    return d;
}
bool Node::attr_bool(const std::string& k, bool d) const {
    for (auto& kv : attrs) if (kv.first == k) return kv.second.i != 0;
    return d;
}
std::string Node::attr_str(const std::string& k, const std::string& d) const {
    for (auto& kv : attrs) if (kv.first == k) return kv.second.kind == Attr::STR ? kv.second.s : kv.second.to_string();
    return d;
}
std::vector<int64_t> Node::attr_ints(const std::string& k) const {
    for (auto& kv : attrs) if (kv.first == k) return kv.second.is;
    return {};
}
void Node::validate_and_infer() {
    if (schema && schema->infer) {
        for (auto& o : outs) { o.lower.reset(); o.upper.reset(); }
        schema->infer(*this);
    }
}
NodePtr Node::clone_with_new_inputs(const std::vector<Output>& inputs) const {
    auto n = std::make_shared<Node>(schema, inputs, attrs);
    n->type = type;
    n->version = version;
    n->rt_info = rt_info;
    n->constant = constant;
    n->outs.resize(outs.size());
    for (auto& b : bodies) n->bodies.push_back(b ? b->clone() : nullptr);
    if (type == "Constant" || type == "Parameter") {
        for (size_t i = 0; i < outs.size(); ++i) { n->outs[i].et = outs[i].et; n->outs[i].shape = outs[i].shape; }
    }
    n->validate_and_infer();
    return n;
}
std::string Node::description() const {
    std::ostringstream os;
    os << type << "(" << version << ") '" << name << "'";
    return os.str();
}

void replace_output(const Output& from, const Output& to) {
    if (from == to) return;
    auto uses = from.node->outs.at(from.index).uses;   // copy: set_input edits the list
    for (auto& u : uses) u.node->set_input(u.input, to);
    // tensor names travel with the value
    auto& src = from.node->outs.at(from.index);
    auto& dst = to.node->outs.at(to.index);
    dst.names.insert(src.names.begin(), src.names.end());
}
void replace_node(const NodePtr& target, const NodePtr& replacement, bool copy_name) {
    OVC_CHECK(target->num_outputs() == replacement->num_outputs(),
              "replace_node: output count differs (" << target->description() << " -> " << replacement->description() << ")");
    for (size_t i = 0; i < target->num_outputs(); ++i) replace_output(Output(target, i), Output(replacement, i));
    if (copy_name) replacement->name = target->name;
}
void copy_runtime_info(const std::vector<NodePtr>& from, const std::vector<NodePtr>& to) {
    // FusedNames semantics: the union of original layer names travels to the new nodes
    std::vector<std::string> fused;
    AttrMap merged;
    for (auto& f : from) {
        auto it = f->rt_info.find("fused_names_0");
        if (it != f->rt_info.end()) {
            for (auto& s : split(it->second.s, ',')) if (!s.empty()) fused.push_back(s);
        } else {
            fused.push_back(f->name);
        }
        for (auto& kv : f->rt_info) if (kv.first != "fused_names_0") merged.insert(kv);
    }
    std::sort(fused.begin(), fused.end());
    fused.erase(std::unique(fused.begin(), fused.end()), fused.end());
    for (auto& t : to) {
        for (auto& kv : merged) t->rt_info.insert(kv);
        t->rt_info["fused_names_0"] = Attr::Str(join(fused, ","));
    }
}

// ------------------------------------------------------------------------------------ registry
OpRegistry& OpRegistry::get() {
    static OpRegistry r;
    return r;
}
void OpRegistry::add(OpSchema s) {
    auto key = std::make_pair(s.type, s.version);
    auto sp = std::make_shared<OpSchema>(std::move(s));
    if (!ops_.count(key)) versions_[sp->type].push_back(sp->version);
    ops_[key] = sp;
}
void OpRegistry::alias(const std::string& type, const std::string& version, const std::string& as_version) {
    auto it = ops_.find({type, version});
    OVC_CHECK(it != ops_.end(), "alias: unknown op " << type << ":" << version);
    ops_[{type, as_version}] = it->second;
}
const OpSchema* OpRegistry::find(const std::string& type, const std::string& version) const {
    auto it = ops_.find({type, version});
    return it == ops_.end() ? nullptr : it->second.get();
}
static int opset_number(const std::string& v) {
    if (v.rfind("opset", 0) == 0) return std::atoi(v.c_str() + 5);
    return 1000;
}
const OpSchema* OpRegistry::find_latest(const std::string& type) const {
    auto it = versions_.find(type);
    if (it == versions_.end() || it->second.empty()) return nullptr;
    std::string best = it->second.front();
    for (auto& v : it->second) if (opset_number(v) >= opset_number(best)) best = v;
    return find(type, best);
}
const OpSchema* OpRegistry::find_ci(const std::string& type, const std::string& version) const {
    if (auto* s = find(type, version)) return s;
    auto lower = [](std::string s) { for (auto& c : s) c = (char)std::tolower((unsigned char)c); return s; };
    const std::string lt = lower(type);
    const OpSchema* best = nullptr;
    for (auto& kv : ops_) {
        if (lower(kv.first.first) != lt) continue;
        if (kv.first.second == version) return kv.second.get();
        // newest version not newer than the requested opset
        if (opset_number(kv.first.second) <= opset_number(version) &&
            (!best || opset_number(kv.first.second) > opset_number(best->version)))
            best = kv.second.get();
    }
    return best;
}
std::vector<const OpSchema*> OpRegistry::all() const {
    std::vector<const OpSchema*> v;
    for (auto& kv : ops_) if (kv.first.second == kv.second->version) v.push_back(kv.second.get());
    return v;
}
std::vector<std::string> OpRegistry::types_in_opset(const std::string& opset) const {
    // an opset contains, for every type, the newest version introduced at or before it
    std::vector<std::string> out;
    const int n = opset_number(opset);
    for (auto& kv : versions_) {
        for (auto& v : kv.second) if (opset_number(v) <= n) { out.push_back(kv.first); break; }
    }
    return out;
}

NodePtr make_node(const std::string& type, const std::string& version, const std::vector<Output>& inputs,
                  const std::vector<std::pair<std::string, Attr>>& attrs, bool infer) {
    register_all_ops();
    auto& reg = OpRegistry::get();
    const OpSchema* s = version.empty() ? reg.find_latest(type) : reg.find(type, version);
    if (!s && !version.empty()) s = reg.find_ci(type, version);
    OVC_CHECK(s, "unknown operation " << type << (version.empty() ? "" : (" in " + version)));
    OVC_CHECK((int)inputs.size() >= s->min_inputs && (s->max_inputs < 0 || (int)inputs.size() <= s->max_inputs),
              type << ": expected " << s->min_inputs << ".." << s->max_inputs << " inputs, got " << inputs.size());
    for (size_t i = 0; i < inputs.size(); ++i) OVC_CHECK(inputs[i].node, type << ": input " << i << " is empty");
    std::vector<std::pair<std::string, Attr>> ordered;
    std::vector<bool> used(attrs.size(), false);
    for (auto& spec : s->attrs) {
        bool found = false;
        for (size_t k = 0; k < attrs.size(); ++k) {
            if (attrs[k].first == spec.name) {
                Attr a = attrs[k].second;
                // tolerate INT given for FLOAT and scalars given for lists
                if (spec.kind == Attr::FLOAT && a.kind == Attr::INT) a = Attr::Float(double(a.i));
                if (spec.kind == Attr::INT && a.kind == Attr::BOOL) a = Attr::Int(a.i);
                if (spec.kind == Attr::BOOL && a.kind == Attr::INT) a = Attr::Bool(a.i != 0);
                if (spec.kind == Attr::INTS && a.kind == Attr::INT) a = Attr::Ints({a.i});
                if (spec.kind == Attr::FLOATS && a.kind == Attr::FLOAT) a = Attr::Floats({a.f});
                if (spec.kind == Attr::FLOATS && a.kind == Attr::INTS) { std::vector<double> f(a.is.begin(), a.is.end()); a = Attr::Floats(f); }
                if (spec.kind == Attr::TYPE && a.kind == Attr::STR) a = Attr::Type(et_from_name(a.s));
                if (spec.kind == Attr::PSHAPE && a.kind == Attr::INTS) a = Attr::Shape_(PShape(Shape(a.is)));
                if (spec.kind == Attr::PSHAPE && a.kind == Attr::STR) a = Attr::Shape_(PShape::parse(a.s));
                if (spec.kind == Attr::FLOAT && spec.f32) a.f = double(float(a.f));
                if (spec.kind == Attr::STR && a.kind != Attr::STR) a = Attr::Str(a.to_string());
                ordered.emplace_back(spec.name, a);
                used[k] = true;
                found = true;
                break;
            }
        }
        if (!found) {
            OVC_CHECK(!spec.required, type << ": missing required attribute '" << spec.name << "'");
            ordered.emplace_back(spec.name, spec.def);
        }
    }
    for (size_t k = 0; k < attrs.size(); ++k) if (!used[k]) ordered.push_back(attrs[k]);   // extra (framework) attrs
    auto n = std::make_shared<Node>(s, inputs, std::move(ordered));
    if (infer) n->validate_and_infer();
    return n;
}

NodePtr make_constant(const Tensor& t) {
    auto n = make_node("Constant", "opset1", {}, {{"element_type", Attr::Type(t.et)}, {"shape", Attr::Shape_(PShape(t.shape))}}, false);
    n->constant = t;
    n->validate_and_infer();
    return n;
}
NodePtr make_constant_i64(const std::vector<int64_t>& v, ET et, bool scalar) {
    return make_constant(from_i64(et, scalar ? Shape{} : Shape{(int64_t)v.size()}, v));
}
NodePtr make_constant_f32(const std::vector<float>& v, const Shape& shape, ET et) {
    return make_constant(from_f32(et, shape, v));
}
NodePtr make_parameter(ET et, const PShape& shape, const std::string& name) {
    auto n = make_node("Parameter", "opset1", {}, {{"shape", Attr::Shape_(shape)}, {"element_type", Attr::Type(et)}});
    if (!name.empty()) {
        n->name = name;
        n->outs[0].names.insert(name);
    }
    return n;
}
NodePtr make_result(const Output& src) { return make_node("Result", "opset1", {src}); }

// ------------------------------------------------------------------------------------ model
std::vector<NodePtr> topological_sort(const std::vector<NodePtr>& roots) {
    // Depth-first from the roots with an explicit stack; a node is emitted once all of its inputs are.
    // The last root is visited first and inputs are pushed so that input 0 is expanded first, which is the
    // visiting order the IR layer numbering of existing IR files was produced with.
    std::vector<Node*> todo;
    std::unordered_set<Node*> done;
    std::unordered_map<Node*, int> visits;
    std::vector<NodePtr> result;
    for (auto& r : roots) todo.push_back(r.get());
    while (!todo.empty()) {
        Node* n = todo.back();
        if (done.count(n)) { todo.pop_back(); continue; }
        OVC_CHECK(++visits[n] <= 2, "loop detected during topological sort at '" << n->name << "'");
        bool ready = true;
        const size_t k = n->num_inputs();
        for (size_t i = 0; i < k; ++i) {
            Node* dep = n->input(k - i - 1).node.get();
            if (!done.count(dep)) { ready = false; todo.push_back(dep); }
        }
        if (ready) {
            result.push_back(n->shared_from_this());
            todo.pop_back();
            done.insert(n);
        }
    }
    return result;
}

Model::Model(std::vector<NodePtr> r, std::vector<NodePtr> s, std::vector<NodePtr> p, std::string n)
    : name(std::move(n)), params(std::move(p)), results(std::move(r)), sinks(std::move(s)) {
    static std::atomic<uint64_t> counter{0};
    if (name.empty()) name = "Model" + std::to_string(counter.fetch_add(1));
    for (auto& x : results) OVC_CHECK(x && x->is_result(), "Model: results must be Result nodes");
    // auto-detect parameters when none were given
    if (params.empty()) {
        for (auto& n2 : ordered_ops()) if (n2->is_parameter()) params.push_back(n2);
    } else {
        std::unordered_set<Node*> have;
        for (auto& x : params) have.insert(x.get());
        for (auto& n2 : ordered_ops())
            OVC_CHECK(!n2->is_parameter() || have.count(n2.get()), "Model references undeclared parameter '" << n2->name << "'");
    }
}
std::vector<NodePtr> Model::ordered_ops() const {
    std::vector<NodePtr> roots;
    roots.insert(roots.end(), results.begin(), results.end());
    roots.insert(roots.end(), sinks.begin(), sinks.end());
    roots.insert(roots.end(), params.begin(), params.end());
    return topological_sort(roots);
}
void Model::validate() {
    for (auto& n : ordered_ops()) n->validate_and_infer();
}
size_t Model::graph_size() const {
    size_t total = 0;
    for (auto& n : ordered_ops()) {
        total += 64;
        if (n->is_constant()) total += n->constant.byte_size();
    }
    return total;
}
bool Model::is_dynamic() const {
    for (auto& n : ordered_ops())
        for (auto& o : n->outs) if (o.shape.is_dynamic()) return true;
    return false;
}
ModelPtr Model::clone() const {
    std::unordered_map<Node*, NodePtr> map;
    for (auto& n : ordered_ops()) {
        std::vector<Output> ins;
        for (auto& i : n->inputs()) ins.emplace_back(map.at(i.node.get()), i.index);
        auto c = std::make_shared<Node>(n->schema, ins, n->attrs);
        c->type = n->type;
        c->version = n->version;
        c->name = n->name;
        c->rt_info = n->rt_info;
        c->input_rt = n->input_rt;
        c->constant = n->constant;   // buffers are shared (immutable by convention)
        c->outs.resize(n->outs.size());
        for (size_t i = 0; i < n->outs.size(); ++i) {
            c->outs[i].shape = n->outs[i].shape;
            c->outs[i].et = n->outs[i].et;
            c->outs[i].names = n->outs[i].names;
            c->outs[i].rt = n->outs[i].rt;
        }
        for (auto& b : n->bodies) c->bodies.push_back(b ? b->clone() : nullptr);
        map[n.get()] = c;
    }
    auto conv = [&](const std::vector<NodePtr>& v) {
        std::vector<NodePtr> r;
        for (auto& n : v) r.push_back(map.at(n.get()));
        return r;
    };
    auto m = std::make_shared<Model>(conv(results), conv(sinks), conv(params), name);
    m->rt_info = rt_info;
    return m;
}
void Model::reshape(const std::map<size_t, PShape>& new_shapes) {
    std::map<size_t, PShape> old;
    for (auto& kv : new_shapes) {
        OVC_CHECK(kv.first < params.size(), "reshape: no input " << kv.first);
        auto& p = params[kv.first];
        old[kv.first] = p->attr("shape").ps;
        p->set_attr("shape", Attr::Shape_(kv.second));
    }
    try {
        validate();
    } catch (...) {
        for (auto& kv : old) params[kv.first]->set_attr("shape", Attr::Shape_(kv.second));
        validate();
        throw;
    }
}
std::vector<VariableInfo> Model::variables() const {
    std::vector<VariableInfo> out;
    std::set<std::string> seen;
    for (auto& n : ordered_ops()) {
        if (n->type != "ReadValue" && n->type != "Assign") continue;
        const std::string idv = n->attr_str("variable_id");
        if (seen.count(idv)) continue;
        seen.insert(idv);
        VariableInfo vi;
        vi.id = idv;
        if (n->has_attr("variable_shape")) vi.shape = n->attr("variable_shape").ps; else vi.shape = n->outs[0].shape;
        if (n->has_attr("variable_type")) vi.et = n->attr("variable_type").et; else vi.et = n->outs[0].et;
        if (n->type == "ReadValue" && (vi.et == ET::dynamic)) { vi.et = n->outs[0].et; vi.shape = n->outs[0].shape; }
        out.push_back(vi);
    }
    return out;
}
NodePtr Model::find_node(const std::string& fname) const {
    for (auto& n : ordered_ops()) if (n->name == fname) return n;
    return nullptr;
}
void Model::add_parameters(const std::vector<NodePtr>& p) { params.insert(params.end(), p.begin(), p.end()); }
void Model::remove_parameter(const NodePtr& p) { params.erase(std::remove(params.begin(), params.end(), p), params.end()); }
void Model::add_results(const std::vector<NodePtr>& r) { results.insert(results.end(), r.begin(), r.end()); }
void Model::remove_result(const NodePtr& r) { results.erase(std::remove(results.begin(), results.end(), r), results.end()); }
void Model::add_sinks(const std::vector<NodePtr>& s) { sinks.insert(sinks.end(), s.begin(), s.end()); }
void Model::remove_sink(const NodePtr& s) { sinks.erase(std::remove(sinks.begin(), sinks.end(), s), sinks.end()); }

// ------------------------------------------------------------------------------------ evaluation
bool get_constant_ints(const Output& o, std::vector<int64_t>& v) {
    Tensor t;
    if (!try_constant_value(o, t)) return false;
    if (t.et == ET::string) return false;
    v = to_i64(t);
    return true;
}

bool try_constant_value(const Output& o, Tensor& out, int depth) {
    Node& n = *o.node;
    if (n.is_constant()) { out = n.constant; return true; }
    auto& od = n.outs.at(o.index);
    if (od.lower && od.upper && od.lower->numel() == od.upper->numel()) {
        bool same = true;
        const int64_t cnt = od.lower->numel();
        for (int64_t i = 0; i < cnt && same; ++i) same = get_elem_f64(*od.lower, i) == get_elem_f64(*od.upper, i);
        if (same) { out = *od.lower; return true; }
    }
    if (depth > 24 || !n.schema || !n.schema->eval || n.schema->has_side_effects || n.is_parameter()) return false;
    // ShapeOf of a static shape is a constant even if its producer is not
    if (n.type == "ShapeOf") {
        const PShape& s = n.in_shape(0);
        if (!s.is_static()) return false;
        out = from_i64(n.outs[0].et, Shape{(int64_t)s.rank()}, s.to_shape());
        return true;
    }
    if (n.num_inputs() == 0) return false;
    std::vector<Tensor> ins;
    int64_t total = 0;
    for (auto& i : n.inputs()) {
        Tensor t;
        if (!try_constant_value(i, t, depth + 1)) return false;
        total += t.numel();
        if (total > (1 << 16)) return false;   // value propagation is for shape arithmetic, not for weights
        ins.push_back(std::move(t));
    }
    std::vector<Tensor> outs(n.num_outputs());
    EvalContext ctx;
    ctx.num_threads = 1;
    try {
        if (!n.schema->eval(n, ins, outs, ctx)) return false;
    } catch (const Error&) {
        return false;
    }
    out = outs.at(o.index);
    return out.defined();
}

std::vector<Tensor> evaluate_model(const Model& m, const std::vector<Tensor>& inputs, EvalContext& ctx,
                                   std::vector<std::pair<std::string, double>>* per_node_us) {
    OVC_CHECK(inputs.size() == m.params.size(), "evaluate: expected " << m.params.size() << " inputs, got " << inputs.size());
    std::unordered_map<Node*, std::vector<Tensor>> values;
    for (size_t i = 0; i < m.params.size(); ++i) {
        const Tensor& t = inputs[i];
        const PShape& ps = m.params[i]->outs[0].shape;
        OVC_CHECK(ps.compatible(PShape(t.shape)), "input " << i << " ('" << m.params[i]->name << "') has shape "
                  << PShape(t.shape).str() << ", the model expects " << ps.str());
        values[m.params[i].get()] = {t};
    }
    auto order = m.ordered_ops();
    // reference counts so that intermediate tensors are released as early as possible
    std::unordered_map<Node*, int> pending;
    for (auto& n : order) for (auto& i : n->inputs()) pending[i.node.get()]++;
    std::vector<Tensor> results(m.results.size());
    for (auto& n : order) {
        if (n->is_parameter()) continue;
        if (n->is_constant()) { values[n.get()] = {n->constant}; continue; }
        std::vector<Tensor> ins;
        for (auto& i : n->inputs()) {
            auto it = values.find(i.node.get());
            OVC_CHECK(it != values.end(), "evaluate: value of '" << i.node->name << "' is missing");
            ins.push_back(it->second.at(i.index));
        }
        std::vector<Tensor> outs(n->num_outputs());
        OVC_CHECK(n->schema && n->schema->eval, "no reference implementation for " << n->description());
        const auto t0 = std::chrono::steady_clock::now();
        const bool ok = n->schema->eval(*n, ins, outs, ctx);
        OVC_CHECK(ok, "evaluation failed for " << n->description());
        if (per_node_us) {
            const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
            per_node_us->emplace_back(n->name, us);
        }
        values[n.get()] = std::move(outs);
        for (auto& i : n->inputs()) {
            if (--pending[i.node.get()] == 0 && !i.node->is_constant()) values.erase(i.node.get());
        }
    }
    for (size_t i = 0; i < m.results.size(); ++i) {
        auto it = values.find(m.results[i].get());
        OVC_CHECK(it != values.end(), "result " << i << " was not computed");
        results[i] = it->second.at(0);
    }
    return results;
}

}  // namespace ovc
