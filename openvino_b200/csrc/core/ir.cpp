// IR v10/v11 reader and IR v11 writer (.xml + .bin), the model checkpoint format.
//
// Writer layout follows src/core/src/xml_util/xml_serialize_util.cpp:932-1183 (layer order, port id
// numbering that continues from inputs into outputs, edge order, `<data>` attribute order = visitor
// order, rt_info blocks, constant de-duplication as in src/core/src/xml_util/constant_writer.cpp:25-52);
// the reader follows src/core/xml_util/src/xml_deserialize_util.cpp:926-1424.
#include "ir.hpp"

#include <cstdio>
#include <fstream>
#include <functional>

#include "xml.hpp"

namespace ovc {

namespace {

const std::map<std::string, std::string>& type_to_ir() {
    static const std::map<std::string, std::string> m = {{"Constant", "Const"}, {"PRelu", "PReLU"}, {"Relu", "ReLU"}, {"Softmax", "SoftMax"}};
    return m;
}
std::string ir_type_name(const std::string& t) {
    auto it = type_to_ir().find(t);
    return it == type_to_ir().end() ? t : it->second;
}
std::string model_type_name(const std::string& t) {
    for (auto& kv : type_to_ir()) if (kv.second == t) return kv.first;
    return t;
}

// Runtime attributes with a registered (name, version): written as <attribute name= version= [value=]/>.
// Keys in Node::rt_info are "<name>_<version>".
const std::set<std::string>& known_rt_attributes() {
    static const std::set<std::string> s = {"fused_names_0", "decompression_0", "disable_fp16_compression_0", "keep_const_precision_0",
                                            "primitives_priority_0", "old_api_map_order_0", "old_api_map_element_type_0",
                                            "dequantization_node_0", "nonconvertible_divide_0", "strides_0", "layout_0",
                                            "preprocessing_fuse_0", "dont_fuse_0", "no_transpose_sinking_0", "is_shape_subgraph_0",
                                            "original_partial_shape_0", "precise_0", "postponed_fp16_compression_0"};
    return s;
}
bool rt_has_value(const std::string& key) {
    static const std::set<std::string> with_value = {"fused_names_0", "primitives_priority_0", "old_api_map_order_0", "old_api_map_element_type_0",
                                                     "strides_0", "layout_0", "original_partial_shape_0"};
    return with_value.count(key) > 0;
}

std::string escape_delim(const std::string& name, char delim = ',') {
    std::string r;
    for (char c : name) { if (c == delim) r.push_back('\\'); r.push_back(c); }
    return r;
}
std::vector<std::string> split_names(const std::string& s) {
    // ',' separated, '\,' is an escaped comma
    std::vector<std::string> out;
    std::string cur;
    for (size_t i = 0; i < s.size(); ++i) {
        if (s[i] == '\\' && i + 1 < s.size() && s[i + 1] == ',') { cur.push_back(','); ++i; }
        else if (s[i] == ',') { out.push_back(cur); cur.clear(); }
        else cur.push_back(s[i]);
    }
    if (!cur.empty() || !s.empty()) out.push_back(cur);
    return out;
}

uint64_t hash_bytes(const uint8_t* p, size_t n) {
    uint64_t h = 1469598103934665603ull;   // FNV-1a over 8-byte words then bytes
    size_t i = 0;
    for (; i + 8 <= n; i += 8) { uint64_t w; std::memcpy(&w, p + i, 8); h = (h ^ w) * 1099511628211ull; }
    for (; i < n; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h ^ n;
}

bool is_valid_tag(const std::string& name) {
    if (name.empty()) return false;
    if (!(std::isalpha((unsigned char)name[0]) || name[0] == '_')) return false;
    for (char c : name) if (!(std::isalnum((unsigned char)c) || c == '_' || c == '-' || c == '.')) return false;
    if (name.size() >= 3 && std::tolower((unsigned char)name[0]) == 'x' && std::tolower((unsigned char)name[1]) == 'm' && std::tolower((unsigned char)name[2]) == 'l') return false;
    return true;
}

void write_model_rt_info(XmlNode* root, const std::string& name, const Attr& v) {
    XmlNode* child;
    if (is_valid_tag(name)) child = root->append_child(name);
    else { child = root->append_child("info"); child->set_attr("name", name); }
    if (v.kind == Attr::MAP && v.map) {
        for (auto& kv : *v.map) write_model_rt_info(child, kv.first, kv.second);
    } else {
        child->set_attr("value", v.kind == Attr::STR ? v.s : v.to_string());
    }
}
Attr read_model_rt_info(const XmlNode& n) {
    if (n.has_attr("value") && n.children.empty()) return Attr::Str(*n.attr("value"));
    AttrMap m;
    for (auto& c : n.children) {
        const std::string key = c->name == "info" && c->has_attr("name") ? *c->attr("name") : c->name;
        m[key] = read_model_rt_info(*c);
    }
    return Attr::Map(std::move(m));
}

void append_rt_info(XmlNode* parent, const AttrMap& rt, bool deterministic) {
    if (rt.empty()) return;
    XmlNode* rt_node = nullptr;
    auto ensure = [&] { if (!rt_node) rt_node = parent->append_child("rt_info"); return rt_node; };
    for (auto& kv : rt) {
        if (kv.first == "PrimitivesPriority" || kv.first == "alt_width") continue;   // written into <data>
        if (known_rt_attributes().count(kv.first)) {
            const size_t us = kv.first.rfind('_');
            XmlNode* a = ensure()->append_child("attribute");
            a->set_attr("name", kv.first.substr(0, us));
            a->set_attr("version", kv.first.substr(us + 1));
            if (rt_has_value(kv.first)) a->set_attr("value", kv.second.kind == Attr::STR ? kv.second.s : kv.second.to_string());
        } else if (!deterministic) {
            XmlNode* a = ensure()->append_child("user_data");
            a->set_attr("name", kv.first);
            a->set_attr("value", kv.second.kind == Attr::STR ? kv.second.s : kv.second.to_string());
            a->set_attr("version", "");
        }
    }
}
void read_rt_info(const XmlNode* rt_node, AttrMap& rt) {
    if (!rt_node) return;
    for (auto& c : rt_node->children) {
        if (c->name == "attribute" && c->has_attr("name")) {
            const std::string key = *c->attr("name") + "_" + c->attr_or("version", "0");
            if (known_rt_attributes().count(key)) rt[key] = Attr::Str(c->attr_or("value", ""));
            else if (c->has_attr("value")) rt[*c->attr("name")] = Attr::Str(*c->attr("value"));
        } else if ((c->name == "user_data" || c->name == "custom") && c->has_attr("name")) {
            rt[*c->attr("name")] = Attr::Str(c->attr_or("value", ""));
        }
    }
}

// ------------------------------------------------------------------------------------ writer
struct Writer {
    const SerializeOptions& opt;
    std::string& bin;
    std::unordered_multimap<uint64_t, std::pair<size_t, size_t>> dedup;   // hash -> (offset, size)

    size_t write_constant(const Tensor& t, size_t& size_out) {
        std::string packed;
        const uint8_t* p;
        size_t n;
        if (t.et == ET::string) {
            // header: count, the begin offset of every string, the end of the last one; then the characters
            // (src/core/src/runtime/string_aligned_buffer.cpp:19)
            const int32_t cnt = (int32_t)t.strings.size();
            std::vector<int32_t> hdr{cnt, 0};
            int32_t off = 0;
            for (auto& s : t.strings) { off += (int32_t)s.size(); hdr.push_back(off); }
            packed.assign(reinterpret_cast<const char*>(hdr.data()), hdr.size() * 4);
            for (auto& s : t.strings) packed += s;
            p = reinterpret_cast<const uint8_t*>(packed.data());
            n = packed.size();
        } else {
            p = t.data();
            n = t.byte_size();
        }
        size_out = n;
        const uint64_t h = hash_bytes(p, n);
        auto range = dedup.equal_range(h);
        for (auto it = range.first; it != range.second; ++it)
            if (it->second.second == n && std::memcmp(bin.data() + it->second.first, p, n) == 0) return it->second.first;
        const size_t off = bin.size();
        bin.append(reinterpret_cast<const char*>(p), n);
        dedup.emplace(h, std::make_pair(off, n));
        return off;
    }

    void write_ports(XmlNode* parent, const Node& n, bool inputs, int& port_id) {
        const size_t cnt = inputs ? n.num_inputs() : n.num_outputs();
        for (size_t i = 0; i < cnt; ++i) {
            XmlNode* port = parent->append_child("port");
            port->set_attr("id", std::to_string(port_id++));
            const ET et = inputs ? n.in_et(i) : n.outs[i].et;
            const PShape& s = inputs ? n.in_shape(i) : n.outs[i].shape;
            port->set_attr("precision", et_info(et).precision);
            if (!inputs && !n.outs[i].names.empty()) {
                std::vector<std::string> names(n.outs[i].names.begin(), n.outs[i].names.end());
                std::sort(names.begin(), names.end());
                std::string joined;
                for (auto& nm : names) { if (!joined.empty()) joined += ","; joined += escape_delim(nm); }
                port->set_attr("names", joined);
            }
            if (!s.rank_dynamic) for (auto& d : s.dims) port->append_child("dim")->text = d.is_static() ? std::to_string(d.lo) : "-1";
            if (opt.version >= 11) append_rt_info(port, inputs ? n.input_rt[i] : n.outs[i].rt, opt.deterministic);
        }
    }

    void write_port_map(XmlNode* layer, const Node& n, const char* map_tag, const std::vector<int64_t>& in_map,
                        const std::vector<int64_t>& out_map, const Model& body, const std::vector<NodePtr>& body_order, bool loop_like) {
        std::unordered_map<Node*, int> ids;
        for (size_t i = 0; i < body_order.size(); ++i) ids[body_order[i].get()] = (int)i;
        XmlNode* pm = layer->append_child(map_tag);
        for (size_t i = 0; i + 3 <= in_map.size(); i += 3) {
            XmlNode* e = pm->append_child("input");
            if (loop_like && in_map[i + 2] >= 0) e->set_attr("axis", std::to_string(in_map[i + 2]));
            e->set_attr("external_port_id", std::to_string(in_map[i]));
            e->set_attr("internal_layer_id", std::to_string(ids.at(body.params.at((size_t)in_map[i + 1]).get())));
        }
        const int nin = (int)n.num_inputs();
        for (size_t i = 0; i + 2 <= out_map.size(); i += 2) {
            XmlNode* e = pm->append_child("output");
            if (loop_like && out_map[i + 1] >= 0) e->set_attr("axis", std::to_string(out_map[i + 1]));
            e->set_attr("external_port_id", std::to_string(nin + (int)(i / 2)));
            e->set_attr("internal_layer_id", std::to_string(ids.at(body.results.at((size_t)out_map[i]).get())));
        }
        if (loop_like) {
            const int64_t ci = n.attr_int("current_iteration_input", -1), co = n.attr_int("body_condition_output", -1);
            if (ci >= 0) {
                XmlNode* e = pm->append_child("input");
                e->set_attr("external_port_id", "-1");
                e->set_attr("internal_layer_id", std::to_string(ids.at(body.params.at((size_t)ci).get())));
                e->set_attr("purpose", "current_iteration");
            }
            if (co >= 0) {
                XmlNode* e = pm->append_child("output");
                e->set_attr("external_port_id", "-1");
                e->set_attr("internal_layer_id", std::to_string(ids.at(body.results.at((size_t)co).get())));
                e->set_attr("purpose", "execution_condition");
            }
            const auto be = n.attr_ints("back_edges");
            XmlNode* bx = layer->append_child("back_edges");
            for (size_t i = 0; i + 2 <= be.size(); i += 2) {
                XmlNode* e = bx->append_child("edge");
                e->set_attr("from-layer", std::to_string(ids.at(body.results.at((size_t)be[i]).get())));
                e->set_attr("to-layer", std::to_string(ids.at(body.params.at((size_t)be[i + 1]).get())));
            }
        }
    }

    std::vector<NodePtr> layer_order(const Model& m) {
        std::vector<NodePtr> order;
        std::unordered_set<Node*> special;
        for (auto& p : m.params) { order.push_back(p); special.insert(p.get()); }
        for (auto& s : m.sinks) special.insert(s.get());
        for (auto& r : m.results) special.insert(r.get());
        for (auto& n : m.ordered_ops()) if (!special.count(n.get())) order.push_back(n);
        for (auto& s : m.sinks) order.push_back(s);
        for (auto& r : m.results) order.push_back(r);
        return order;
    }

    void write_model(XmlNode* net, const Model& m, bool top) {
        if (top) {
            if (!opt.deterministic) net->set_attr("name", m.name);
            net->set_attr("version", std::to_string(opt.version));
        }
        XmlNode* layers = net->append_child("layers");
        const auto order = layer_order(m);
        std::unordered_map<Node*, int> ids;
        for (size_t i = 0; i < order.size(); ++i) ids[order[i].get()] = (int)i;
        for (auto& np : order) {
            Node& n = *np;
            XmlNode* layer = layers->append_child("layer");
            layer->set_attr("id", std::to_string(ids[&n]));
            if (!opt.deterministic) layer->set_attr("name", n.name);
            layer->set_attr("type", ir_type_name(n.type));
            layer->set_attr("version", n.version);
            XmlNode* data = layer->append_child("data");
            if (opt.version >= 11) append_rt_info(layer, n.rt_info, opt.deterministic);
            int port_id = 0;
            XmlNode* input = nullptr;
            if (n.num_inputs() > 0) { input = layer->append_child("input"); write_ports(input, n, true, port_id); }
            XmlNode* output = nullptr;
            if (n.is_result()) {
                if (opt.version > 10 && !opt.deterministic && !n.outs[0].names.empty()) {
                    // only names assigned to the Result itself (not inherited from its producer)
                    std::vector<std::string> own;
                    const auto& src = n.input(0).node->outs[n.input(0).index].names;
                    for (auto& nm : n.outs[0].names) if (!src.count(nm)) own.push_back(nm);
                    if (!own.empty()) {
                        std::sort(own.begin(), own.end());
                        std::string joined;
                        for (auto& nm : own) { if (!joined.empty()) joined += ","; joined += escape_delim(nm); }
                        layer->set_attr("output_names", joined);
                    }
                }
            } else if (n.num_outputs() > 0) {
                output = layer->append_child("output");
                write_ports(output, n, false, port_id);
            }
            const bool loop_like = n.type == "TensorIterator" || n.type == "Loop";
            if (loop_like) {
                if (input) layer->move_child_to_front(input);
                if (output) layer->move_child_after(output, layer->children.front().get());
            }
            // <data> attributes
            if (n.is_constant()) {
                data->set_attr("element_type", et_name(n.constant.et));
                data->set_attr("shape", Attr::Ints(n.constant.shape).to_string());
                size_t size = 0;
                const size_t off = write_constant(n.constant, size);
                data->set_attr("offset", std::to_string(off));
                data->set_attr("size", std::to_string(size));
            } else if (!n.bodies.empty()) {
                if (n.type == "If") {
                    const char* body_tags[2] = {"then_body", "else_body"};
                    const char* map_tags[2] = {"then_port_map", "else_port_map"};
                    for (size_t b = 0; b < n.bodies.size() && b < 2; ++b) {
                        XmlNode* bx = layer->append_child(body_tags[b]);
                        write_model(bx, *n.bodies[b], false);
                        write_port_map(layer, n, map_tags[b], n.attr_ints(b == 0 ? "input_map" : "else_input_map"),
                                       n.attr_ints(b == 0 ? "output_map" : "else_output_map"), *n.bodies[b], layer_order(*n.bodies[b]), false);
                    }
                    // bodies first, then their port maps in the reference's order: then_body, else_body, then_port_map, else_port_map
                    std::vector<XmlNode*> maps;
                    for (auto& c : layer->children) if (c->name == "then_port_map" || c->name == "else_port_map") maps.push_back(c.get());
                    for (auto* mp : maps) layer->move_child_after(mp, layer->children.back().get());
                } else {
                    write_port_map(layer, n, "port_map", n.attr_ints("input_map"), n.attr_ints("output_map"), *n.bodies[0], layer_order(*n.bodies[0]), true);
                    XmlNode* bx = layer->append_child("body");
                    write_model(bx, *n.bodies[0], false);
                }
            } else {
                for (auto& kv : n.attrs) {
                    const Attr& a = kv.second;
                    if (a.kind == Attr::NONE || a.kind == Attr::MAP) continue;
                    data->set_attr(kv.first, a.to_string());
                }
            }
            for (const char* k : {"PrimitivesPriority", "alt_width"}) {
                auto it = n.rt_info.find(k);
                if (it != n.rt_info.end()) data->set_attr(k, it->second.kind == Attr::STR ? it->second.s : it->second.to_string());
            }
            if (data->attrs.empty()) layer->remove_child(data);
        }
        // edges, sorted by destination layer order (stable)
        XmlNode* edges = net->append_child("edges");
        struct E { int fl, fp, tl, tp; };
        std::vector<E> es;
        for (auto& np : order) {
            for (size_t i = 0; i < np->num_inputs(); ++i) {
                const Output& src = np->input(i);
                es.push_back({ids.at(src.node.get()), (int)(src.node->num_inputs() + src.index), ids.at(np.get()), (int)i});
            }
        }
        std::stable_sort(es.begin(), es.end(), [](const E& a, const E& b) { return a.fl < b.fl; });
        for (auto& e : es) {
            XmlNode* x = edges->append_child("edge");
            x->set_attr("from-layer", std::to_string(e.fl));
            x->set_attr("from-port", std::to_string(e.fp));
            x->set_attr("to-layer", std::to_string(e.tl));
            x->set_attr("to-port", std::to_string(e.tp));
        }
        if (top || true) {
            XmlNode* rt = net->append_child("rt_info");
            for (auto& kv : m.rt_info) {
                if (kv.first == "version" || kv.first == "__weights_path") continue;
                write_model_rt_info(rt, kv.first, kv.second);
            }
            if (!top && rt->children.empty() && false) net->remove_child(rt);
        }
    }
};

// ------------------------------------------------------------------------------------ reader
struct Reader {
    BufferPtr weights;
    int version = 11;

    Tensor read_constant(const XmlNode& data, const std::string& lname) {
        const ET et = et_from_name(data.attr_or("element_type", "f32"));
        Shape shape;
        const std::string ss = trim(data.attr_or("shape", ""));
        if (!ss.empty()) for (auto& t : split(ss, ',')) shape.push_back(std::stoll(trim(t)));
        const size_t off = (size_t)std::stoull(data.attr_or("offset", "0")), size = (size_t)std::stoull(data.attr_or("size", "0"));
        OVC_CHECK(weights || size == 0, "constant '" << lname << "' needs weights but no .bin data was given");
        OVC_CHECK(!weights || off + size <= weights->size, "constant '" << lname << "' points outside the weights (offset " << off << ", size " << size << ", file " << (weights ? weights->size : 0) << ")");
        if (et == ET::string) {
            Tensor t(et, shape);
            const uint8_t* p = weights->data + off;
            OVC_CHECK(size >= 4, "string constant '" << lname << "' is truncated");
            int32_t cnt;
            std::memcpy(&cnt, p, 4);
            const size_t hdr_bytes = (2 + (size_t)(cnt < 0 ? 0 : cnt)) * 4;   // count, cnt begin offsets, the last end
            OVC_CHECK(cnt >= 0 && hdr_bytes <= size, "string constant '" << lname << "' has a bad header");
            const char* chars = reinterpret_cast<const char*>(p) + hdr_bytes;
            const size_t chars_len = size - hdr_bytes;
            for (int32_t i = 0; i < cnt && (size_t)i < t.strings.size(); ++i) {
                int32_t b, e;
                std::memcpy(&b, p + 4 + 4 * (size_t)i, 4);
                std::memcpy(&e, p + 8 + 4 * (size_t)i, 4);
                OVC_CHECK(b >= 0 && e >= b && (size_t)e <= chars_len, "string constant '" << lname << "' has bad offsets");
                t.strings[(size_t)i].assign(chars + b, chars + e);
            }
            return t;
        }
        const size_t need = et_byte_size(et, (size_t)shape_size(shape));
        OVC_CHECK(need == size, "constant '" << lname << "': size " << size << " does not match shape " << PShape(shape).str() << " of " << et_name(et) << " (" << need << " bytes)");
        Tensor t;
        t.et = et;
        t.shape = shape;
        t.buf = std::make_shared<Buffer>(weights ? weights->data + off : nullptr, size, weights ? std::shared_ptr<void>(weights, weights.get()) : nullptr);
        if (!weights) t.buf = std::make_shared<Buffer>(0);
        return t;
    }

    struct PortInfo { int id; ET et; PShape shape; std::set<std::string> names; AttrMap rt; };
    static PortInfo read_port(const XmlNode& p) {
        PortInfo pi;
        pi.id = std::stoi(p.attr_or("id", "0"));
        pi.et = p.has_attr("precision") ? et_from_name(*p.attr("precision")) : ET::dynamic;
        for (auto& c : p.children) if (c->name == "dim") { const int64_t v = std::stoll(trim(c->text)); pi.shape.dims.push_back(v < 0 ? Dim::dynamic() : Dim(v)); }
        if (p.has_attr("names")) for (auto& nm : split_names(*p.attr("names"))) pi.names.insert(nm);
        read_rt_info(p.child("rt_info"), pi.rt);
        return pi;
    }

    ModelPtr read_model(const XmlNode& net, const std::string& default_name) {
        const XmlNode* layers = net.child("layers");
        OVC_CHECK(layers, "IR has no <layers> section");
        struct L { const XmlNode* x; int id; std::vector<PortInfo> in, out; NodePtr node; };
        std::vector<L> ls;
        std::unordered_map<int, size_t> by_id;
        for (auto& lx : layers->children) {
            if (lx->name != "layer") continue;
            L l;
            l.x = lx.get();
            OVC_CHECK(lx->has_attr("id") && lx->has_attr("type"), "<layer> without id or type");
            l.id = std::stoi(*lx->attr("id"));
            if (auto* in = lx->child("input")) for (auto& p : in->children) if (p->name == "port") l.in.push_back(read_port(*p));
            if (auto* out = lx->child("output")) for (auto& p : out->children) if (p->name == "port") l.out.push_back(read_port(*p));
            OVC_CHECK(!by_id.count(l.id), "duplicate layer id " << l.id);
            by_id[l.id] = ls.size();
            ls.push_back(std::move(l));
        }
        // edges: (to-layer, to-port) -> (from-layer, from-port)
        std::map<std::pair<int, int>, std::pair<int, int>> edge;
        if (auto* edges = net.child("edges"))
            for (auto& e : edges->children)
                if (e->name == "edge")
                    edge[{std::stoi(e->attr_or("to-layer", "-1")), std::stoi(e->attr_or("to-port", "-1"))}] = {std::stoi(e->attr_or("from-layer", "-1")), std::stoi(e->attr_or("from-port", "-1"))};

        std::vector<int> state(ls.size(), 0);
        std::function<void(size_t)> build = [&](size_t root) {
            std::vector<size_t> stack{root};
            while (!stack.empty()) {
                const size_t li = stack.back();
                L& l = ls[li];
                if (state[li] == 2) { stack.pop_back(); continue; }
                bool ready = true;
                for (auto& ip : l.in) {
                    auto it = edge.find({l.id, ip.id});
                    OVC_CHECK(it != edge.end(), "layer " << l.id << " ('" << l.x->attr_or("name", "") << "') input port " << ip.id << " is not connected");
                    auto src = by_id.find(it->second.first);
                    OVC_CHECK(src != by_id.end(), "edge refers to a missing layer " << it->second.first);
                    if (state[src->second] != 2) {
                        OVC_CHECK(state[src->second] != 1 || src->second != li, "layer " << l.id << " feeds itself");
                        ready = false;
                        stack.push_back(src->second);
                    }
                }
                if (!ready) {
                    OVC_CHECK(++state[li] < 1000000, "cycle in the IR graph");
                    state[li] = 1;
                    continue;
                }
                create_node(l, ls, by_id, edge);
                state[li] = 2;
                stack.pop_back();
            }
        };
        for (size_t i = 0; i < ls.size(); ++i) if (state[i] != 2) build(i);

        std::vector<NodePtr> params, results, sinks;
        for (auto& l : ls) {
            if (l.node->is_parameter()) params.push_back(l.node);
            else if (l.node->is_result()) results.push_back(l.node);
            else if (l.node->type == "Assign") sinks.push_back(l.node);
        }
        auto m = std::make_shared<Model>(results, sinks, params, net.attr_or("name", default_name));
        if (auto* rt = net.child("rt_info"))
            for (auto& c : rt->children) {
                const std::string key = c->name == "info" && c->has_attr("name") ? *c->attr("name") : c->name;
                m->rt_info[key] = read_model_rt_info(*c);
            }
        return m;
    }

    template <class LT>
    void create_node(LT& l, std::vector<LT>& ls, std::unordered_map<int, size_t>& by_id, std::map<std::pair<int, int>, std::pair<int, int>>& edge) {
        const XmlNode& lx = *l.x;
        const std::string type = model_type_name(*lx.attr("type"));
        const std::string ver = lx.attr_or("version", "opset1");
        const std::string lname = lx.attr_or("name", "");
        std::vector<Output> inputs;
        for (auto& ip : l.in) {
            auto e = edge.at({l.id, ip.id});
            auto& src = ls[by_id.at(e.first)];
            size_t out_index = 0;
            bool found = false;
            for (size_t k = 0; k < src.out.size(); ++k) if (src.out[k].id == e.second) { out_index = k; found = true; }
            OVC_CHECK(found, "edge into layer " << l.id << " refers to a missing output port " << e.second << " of layer " << e.first);
            inputs.emplace_back(src.node, out_index);
        }
        const XmlNode* data = lx.child("data");
        register_all_ops();
        const OpSchema* schema = OpRegistry::get().find_ci(type, ver);
        NodePtr node;
        if (type == "Constant") {
            OVC_CHECK(data, "Const layer '" << lname << "' has no <data>");
            node = make_constant(read_constant(*data, lname));
        } else if (schema) {
            std::vector<std::pair<std::string, Attr>> attrs;
            if (data) {
                for (auto& a : data->attrs) {
                    if (a.first == "PrimitivesPriority" || a.first == "alt_width") continue;
                    Attr::Kind k = Attr::STR;
                    for (auto& spec : schema->attrs) if (spec.name == a.first) k = spec.kind;
                    attrs.emplace_back(a.first, Attr::from_string(k, a.second));
                }
            }
            std::vector<ModelPtr> bodies;
            if (type == "TensorIterator" || type == "Loop" || type == "If") read_bodies(lx, type, l, attrs, bodies);
            node = make_node(schema->type, schema->version, inputs, attrs, false);
            node->version = ver;
            node->bodies = bodies;
            read_rt_info(lx.child("rt_info"), node->rt_info);
            if (schema->type == "PagedAttentionExtension" || schema->type == "Parameter") { /* shapes come from attributes */ }
            node->validate_and_infer();
        } else {
            // unknown operation: keep it as a generic framework node with the shapes recorded in the file
            OpSchema s;
            s.type = type;
            s.version = ver;
            std::vector<std::pair<ET, PShape>> outs;
            for (auto& op : l.out) outs.emplace_back(op.et, op.shape);
            s.infer = [outs](Node& n2) { n2.set_num_outputs(std::max<size_t>(outs.size(), 1)); for (size_t i = 0; i < outs.size(); ++i) n2.set_output(i, outs[i].first, outs[i].second); };
            OpRegistry::get().add(s);
            const OpSchema* fs = OpRegistry::get().find(type, ver);
            std::vector<std::pair<std::string, Attr>> attrs;
            if (data) for (auto& a : data->attrs) attrs.emplace_back(a.first, Attr::Str(a.second));
            node = std::make_shared<Node>(fs, inputs, attrs);
            node->rt_info["__framework_node"] = Attr::Bool(true);
            node->validate_and_infer();
        }
        if (!node->rt_info.count("fused_names_0") || type != "Constant") read_rt_info(lx.child("rt_info"), node->rt_info);
        if (data) for (const char* k : {"PrimitivesPriority", "alt_width"}) if (data->has_attr(k)) node->rt_info[k] = Attr::Str(*data->attr(k));
        if (!lname.empty()) node->name = lname;
        for (size_t i = 0; i < l.out.size() && i < node->num_outputs(); ++i) {
            node->outs[i].names = l.out[i].names;
            node->outs[i].rt = l.out[i].rt;
        }
        for (size_t i = 0; i < l.in.size() && i < node->input_rt.size(); ++i) node->input_rt[i] = l.in[i].rt;
        if (node->is_result()) {
            node->outs[0].names = node->input(0).node->outs[node->input(0).index].names;
            if (lx.has_attr("output_names")) for (auto& nm : split_names(*lx.attr("output_names"))) node->outs[0].names.insert(nm);
        }
        if (version <= 10 && node->is_parameter() && node->outs[0].names.empty() && !lname.empty()) node->outs[0].names.insert(lname);
        l.node = node;
    }

    template <class LT>
    void read_bodies(const XmlNode& lx, const std::string& type, LT& l, std::vector<std::pair<std::string, Attr>>& attrs, std::vector<ModelPtr>& bodies) {
        auto layer_index = [](const Model& body, const XmlNode& bx, bool params, int internal_id) -> int64_t {
            // position of the body layer with this id among the body's parameters / results
            std::vector<int> ids;
            if (auto* ly = bx.child("layers"))
                for (auto& c : ly->children) {
                    const std::string t = c->attr_or("type", "");
                    if ((params && t == "Parameter") || (!params && t == "Result")) ids.push_back(std::stoi(c->attr_or("id", "-1")));
                }
            (void)body;
            for (size_t i = 0; i < ids.size(); ++i) if (ids[i] == internal_id) return (int64_t)i;
            throw Error("port map refers to a missing body layer " + std::to_string(internal_id));
        };
        const int nin = (int)l.in.size();
        auto read_map = [&](const XmlNode* pm, const XmlNode& bx, const Model& body, std::vector<int64_t>& in_map, std::vector<int64_t>& out_map,
                            int64_t* cur_iter, int64_t* cond_out) {
            if (!pm) return;
            std::map<int, std::pair<int64_t, int64_t>> outs;   // external port -> (result index, axis)
            for (auto& e : pm->children) {
                const int ext = std::stoi(e->attr_or("external_port_id", "-1"));
                const int internal = std::stoi(e->attr_or("internal_layer_id", "-1"));
                const int64_t axis = e->has_attr("axis") ? std::stoll(*e->attr("axis")) : -1;
                const std::string purpose = e->attr_or("purpose", "");
                if (e->name == "input") {
                    const int64_t pi = layer_index(body, bx, true, internal);
                    if (purpose == "current_iteration" || ext < 0) { if (cur_iter) *cur_iter = pi; continue; }
                    in_map.push_back(ext); in_map.push_back(pi); in_map.push_back(axis);
                } else if (e->name == "output") {
                    const int64_t ri = layer_index(body, bx, false, internal);
                    if (purpose == "execution_condition" || ext < 0) { if (cond_out) *cond_out = ri; continue; }
                    outs[ext - nin] = {ri, axis};
                }
            }
            for (auto& kv : outs) { out_map.push_back(kv.second.first); out_map.push_back(kv.second.second); }
        };
        auto set = [&](const char* k, Attr v) { for (auto& a : attrs) if (a.first == k) { a.second = v; return; } attrs.emplace_back(k, v); };
        if (type == "If") {
            const char* body_tags[2] = {"then_body", "else_body"};
            const char* map_tags[2] = {"then_port_map", "else_port_map"};
            for (int b = 0; b < 2; ++b) {
                const XmlNode* bx = lx.child(body_tags[b]);
                OVC_CHECK(bx, "If layer without " << body_tags[b]);
                auto body = read_model(*bx, body_tags[b]);
                std::vector<int64_t> im, om;
                read_map(lx.child(map_tags[b]), *bx, *body, im, om, nullptr, nullptr);
                set(b == 0 ? "input_map" : "else_input_map", Attr::Ints(im));
                set(b == 0 ? "output_map" : "else_output_map", Attr::Ints(om));
                bodies.push_back(body);
            }
        } else {
            const XmlNode* bx = lx.child("body");
            OVC_CHECK(bx, type << " layer without <body>");
            auto body = read_model(*bx, "body");
            std::vector<int64_t> im, om, be;
            int64_t ci = -1, co = -1;
            read_map(lx.child("port_map"), *bx, *body, im, om, &ci, &co);
            if (auto* bex = lx.child("back_edges"))
                for (auto& e : bex->children) {
                    be.push_back(layer_index(*body, *bx, false, std::stoi(e->attr_or("from-layer", "-1"))));
                    be.push_back(layer_index(*body, *bx, true, std::stoi(e->attr_or("to-layer", "-1"))));
                }
            set("input_map", Attr::Ints(im));
            set("output_map", Attr::Ints(om));
            set("back_edges", Attr::Ints(be));
            set("current_iteration_input", Attr::Int(ci));
            set("body_condition_output", Attr::Int(co));
            bodies.push_back(body);
        }
    }
};

}  // namespace

void serialize_model(const Model& m, std::string& xml, std::string& bin, const SerializeOptions& opt) {
    XmlDocument doc;
    doc.root.reset(new XmlNode());
    doc.root->name = "net";
    bin.clear();
    Writer w{opt, bin, {}};
    w.write_model(doc.root.get(), m, true);
    xml = doc.to_string();
}

ModelPtr deserialize_model(const std::string& xml, BufferPtr weights) {
    XmlDocument doc = XmlDocument::parse(xml);
    OVC_CHECK(doc.root && doc.root->name == "net", "not an IR file: the root element is not <net>");
    Reader r;
    r.weights = std::move(weights);
    r.version = std::stoi(doc.root->attr_or("version", "11"));
    OVC_CHECK(r.version >= 10 && r.version <= 11, "unsupported IR version " << r.version);
    auto m = r.read_model(*doc.root, "Model");
    m->rt_info.erase("version");
    return m;
}

static bool read_file(const std::string& path, std::string& out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    f.seekg(0, std::ios::end);
    const std::streamoff n = f.tellg();
    f.seekg(0);
    out.resize((size_t)n);
    if (n) f.read(&out[0], n);
    return bool(f);
}

ModelPtr read_model_files(const std::string& xml_path, const std::string& bin_path_in) {
    std::string xml;
    OVC_CHECK(read_file(xml_path, xml), "cannot read '" << xml_path << "'");
    std::string bin_path = bin_path_in;
    if (bin_path.empty()) {
        bin_path = xml_path;
        const size_t dot = bin_path.rfind('.');
        if (dot != std::string::npos) bin_path = bin_path.substr(0, dot);
        bin_path += ".bin";
    }
    BufferPtr weights;
    std::string bin;
    if (read_file(bin_path, bin)) {
        weights = std::make_shared<Buffer>(bin.size());
        if (!bin.empty()) std::memcpy(weights->data, bin.data(), bin.size());
    } else {
        OVC_CHECK(bin_path_in.empty(), "cannot read weights file '" << bin_path << "'");
    }
    return deserialize_model(xml, weights);
}

void save_model_files(const Model& m, const std::string& xml_path, const std::string& bin_path_in, const SerializeOptions& opt) {
    std::string xml, bin;
    serialize_model(m, xml, bin, opt);
    std::string bin_path = bin_path_in;
    if (bin_path.empty()) {
        bin_path = xml_path;
        const size_t dot = bin_path.rfind('.');
        if (dot != std::string::npos) bin_path = bin_path.substr(0, dot);
        bin_path += ".bin";
    }
    {
        std::ofstream f(xml_path, std::ios::binary);
        OVC_CHECK(bool(f), "cannot write '" << xml_path << "'");
        f.write(xml.data(), (std::streamsize)xml.size());
    }
    {
        std::ofstream f(bin_path, std::ios::binary);
        OVC_CHECK(bool(f), "cannot write '" << bin_path << "'");
        f.write(bin.data(), (std::streamsize)bin.size());
    }
}

uint64_t model_hash(const Model& m) {
    SerializeOptions opt;
    opt.deterministic = true;
    std::string xml, bin;
    serialize_model(m, xml, bin, opt);
    return hash_bytes(reinterpret_cast<const uint8_t*>(xml.data()), xml.size()) * 1099511628211ull ^
           hash_bytes(reinterpret_cast<const uint8_t*>(bin.data()), bin.size());
}

}  // namespace ovc
