// pybind11 surface of the native core (module openvino_b200._ovcore). The Python package wraps these
// low-level objects into the openvino-compatible API (Model, Node, Output, Tensor, Core, ...).
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "ir.hpp"
#include "pass.hpp"
#include "runtime.hpp"
#include "sysconf.hpp"
#include "sched.hpp"

namespace py = pybind11;
using namespace ovc;

namespace {

// ---- Attr <-> python
py::object attr_to_py(const Attr& a) {
    switch (a.kind) {
        case Attr::NONE: return py::none();
        case Attr::BOOL: return py::bool_(a.i != 0);
        case Attr::INT: return py::int_(a.i);
        case Attr::FLOAT: return py::float_(a.f);
        case Attr::STR: return py::str(a.s);
        case Attr::INTS: return py::cast(a.is);
        case Attr::FLOATS: return py::cast(a.fs);
        case Attr::STRS: return py::cast(a.ss);
        case Attr::TYPE: return py::make_tuple(py::str("__type__"), py::str(et_name(a.et)));
        case Attr::PSHAPE: {
            if (a.ps.rank_dynamic) return py::make_tuple(py::str("__pshape__"), py::none());
            py::list l;
            for (auto& d : a.ps.dims) l.append(py::make_tuple(d.lo, d.hi));
            return py::make_tuple(py::str("__pshape__"), l);
        }
        case Attr::MAP: {
            py::dict d;
            if (a.map) for (auto& kv : *a.map) d[py::str(kv.first)] = attr_to_py(kv.second);
            return std::move(d);
        }
    }
    return py::none();
}

PShape pshape_from_py(const py::handle& h) {
    if (h.is_none()) return PShape::dynamic();
    PShape p;
    for (auto item : h) {
        if (py::isinstance<py::tuple>(item) || py::isinstance<py::list>(item)) {
            auto t = py::cast<std::vector<int64_t>>(item);
            p.dims.emplace_back(t.at(0), t.at(1));
            if (t.size() > 2 && p.dims.back().is_dynamic()) p.dims.back().sym = t[2];
        } else {
            p.dims.emplace_back(py::cast<int64_t>(item));
        }
    }
    return p;
}
py::object pshape_to_py(const PShape& s) {
    if (s.rank_dynamic) return py::none();
    py::list l;
    for (auto& d : s.dims) {
        if (d.sym) l.append(py::make_tuple(d.lo, d.hi, d.sym));
        else l.append(py::make_tuple(d.lo, d.hi));
    }
    return std::move(l);
}

Attr py_to_attr(const py::handle& h) {
    if (h.is_none()) return Attr();
    if (py::isinstance<py::bool_>(h)) return Attr::Bool(py::cast<bool>(h));
    if (py::isinstance<py::int_>(h)) return Attr::Int(py::cast<int64_t>(h));
    if (py::isinstance<py::float_>(h)) return Attr::Float(py::cast<double>(h));
    if (py::isinstance<py::str>(h)) return Attr::Str(py::cast<std::string>(h));
    if (py::isinstance<py::dict>(h)) {
        AttrMap m;
        for (auto kv : py::cast<py::dict>(h)) m[py::cast<std::string>(py::str(kv.first))] = py_to_attr(kv.second);
        return Attr::Map(std::move(m));
    }
    if (py::isinstance<py::tuple>(h)) {
        auto t = py::cast<py::tuple>(h);
        if (t.size() == 2 && py::isinstance<py::str>(t[0])) {
            const std::string tag = py::cast<std::string>(t[0]);
            if (tag == "__type__") return Attr::Type(et_from_name(py::cast<std::string>(t[1])));
            if (tag == "__pshape__") return Attr::Shape_(pshape_from_py(t[1]));
        }
    }
    if (py::isinstance<py::sequence>(h)) {
        auto seq = py::cast<py::sequence>(h);
        if (seq.size() == 0) return Attr::Ints({});
        bool all_int = true, all_num = true, all_str = true;
        for (auto item : seq) {
            if (!(py::isinstance<py::int_>(item) || py::isinstance<py::bool_>(item))) all_int = false;
            if (!(py::isinstance<py::int_>(item) || py::isinstance<py::float_>(item))) all_num = false;
            if (!py::isinstance<py::str>(item)) all_str = false;
        }
        if (all_int) return Attr::Ints(py::cast<std::vector<int64_t>>(seq));
        if (all_num) return Attr::Floats(py::cast<std::vector<double>>(seq));
        if (all_str) return Attr::Strs(py::cast<std::vector<std::string>>(seq));
    }
    // numpy scalars and other number-likes
    try { return Attr::Float(py::cast<double>(h)); } catch (...) {}
    return Attr::Str(py::cast<std::string>(py::str(h)));
}

py::dict attrmap_to_py(const AttrMap& m) {
    py::dict d;
    for (auto& kv : m) d[py::str(kv.first)] = attr_to_py(kv.second);
    return d;
}

// ---- Tensor <-> numpy
const char* numpy_dtype_of(ET t) {
    switch (t) {
        case ET::boolean: return "bool";
        case ET::f16: return "float16";
        case ET::f32: return "float32";
        case ET::f64: return "float64";
        case ET::i8: return "int8";
        case ET::i16: return "int16";
        case ET::i32: return "int32";
        case ET::i64: return "int64";
        case ET::u8: return "uint8";
        case ET::u16: return "uint16";
        case ET::u32: return "uint32";
        case ET::u64: return "uint64";
        case ET::bf16: return "uint16";   // raw bits
        default: return "uint8";          // packed / 8-bit float types: raw bytes
    }
}

struct GilDeleter {
    void operator()(py::object* o) const {
        py::gil_scoped_acquire g;
        delete o;
    }
};

// View over a numpy array's memory (no copy); `et` reinterprets the bytes.
Tensor tensor_from_array(py::array arr, const std::string& et_name_, std::vector<int64_t> shape, bool share) {
    const ET et = et_from_name(et_name_);
    if (!(arr.flags() & py::array::c_style)) arr = py::array::ensure(arr, py::array::c_style | py::array::forcecast);
    Tensor t;
    t.et = et;
    t.shape = std::move(shape);
    const size_t need = et_byte_size(et, (size_t)shape_size(t.shape));
    OVC_CHECK((size_t)arr.nbytes() >= need, "array of " << arr.nbytes() << " bytes is too small for " << PShape(t.shape).str() << " of " << et_name(et));
    if (share) {
        std::shared_ptr<py::object> keep(new py::object(arr), GilDeleter());
        t.buf = std::make_shared<Buffer>(static_cast<uint8_t*>(arr.mutable_data()), need, std::shared_ptr<void>(keep, keep.get()));
    } else {
        t.buf = std::make_shared<Buffer>(need);
        if (need) std::memcpy(t.buf->data, arr.data(), need);
    }
    return t;
}

// numpy view of a tensor's memory (zero copy; the Buffer stays alive through the array's base object)
py::object tensor_to_array(const Tensor& t) {
    if (t.et == ET::string) {
        py::list l;
        for (auto& s : t.strings) l.append(py::bytes(s));
        return std::move(l);
    }
    const ET et = t.et;
    const int bits = et_bits(et);
    py::dtype dt(numpy_dtype_of(et));
    std::vector<py::ssize_t> shape;
    if (bits % 8 == 0 && bits >= 8 && et != ET::dynamic) for (auto d : t.shape) shape.push_back((py::ssize_t)d);
    else shape = {(py::ssize_t)t.byte_size()};
    auto* holder = new BufferPtr(t.buf);
    py::capsule base(holder, [](void* p) { delete static_cast<BufferPtr*>(p); });
    return py::array(dt, shape, t.data(), base);
}

struct PyTensor {   // what crosses the boundary: (array, element type name, logical shape)
    static py::tuple pack(const Tensor& t) { return py::make_tuple(tensor_to_array(t), py::str(et_name(t.et)), py::cast(t.shape)); }
};

Output out_from_py(const py::handle& h) {
    if (py::isinstance<py::tuple>(h)) {
        auto t = py::cast<py::tuple>(h);
        return Output(py::cast<NodePtr>(t[0]), py::cast<size_t>(t[1]));
    }
    return Output(py::cast<NodePtr>(h), 0);
}
std::vector<Output> outs_from_py(const py::iterable& it) {
    std::vector<Output> v;
    for (auto h : it) v.push_back(out_from_py(h));
    return v;
}

// A ModelPass implemented in Python
class PyModelPass : public ModelPass {
public:
    py::object fn;
    bool run_on_model(const ModelPtr& m) override {
        py::gil_scoped_acquire g;
        return py::cast<bool>(fn(m));
    }
};

}  // namespace

PYBIND11_MODULE(_ovcore, mod) {
    mod.doc() = "native core of openvino_b200: graph IR, IR v11 reader/writer, passes, reference executor, runtime, scheduler";
    register_all_ops();

    py::register_exception<Error>(mod, "CoreError", PyExc_RuntimeError);
    static py::exception<BusyError> busy_exc(mod, "BusyError", PyExc_RuntimeError);
    static py::exception<CancelledError> cancelled_exc(mod, "CancelledError", PyExc_RuntimeError);
    py::register_exception_translator([](std::exception_ptr p) {
        try { if (p) std::rethrow_exception(p); }
        catch (const BusyError& e) { busy_exc(e.what()); }
        catch (const CancelledError& e) { cancelled_exc(e.what()); }
    });

    // ------------------------------------------------------------------ element types
    mod.def("type_names", [] { std::vector<std::string> v; for (int i = 0; i < kNumET; ++i) v.push_back(et_name((ET)i)); return v; });
    mod.def("type_info", [](const std::string& n) {
        const auto& i = et_info(et_from_name(n));
        return py::make_tuple(i.name, i.precision, i.bits, i.is_real, i.is_signed, i.is_quantized);
    });
    mod.def("type_numpy_dtype", [](const std::string& n) { return std::string(numpy_dtype_of(et_from_name(n))); });
    mod.def("type_byte_size", [](const std::string& n, int64_t count) { return et_byte_size(et_from_name(n), (size_t)count); });
    mod.def("convert_bytes", [](py::array arr, const std::string& from, const std::string& to, std::vector<int64_t> shape) {
        Tensor t = tensor_from_array(arr, from, shape, true);
        return PyTensor::pack(convert_tensor(t, et_from_name(to)));
    });
    mod.def("pshape_to_string", [](const py::object& s) { return pshape_from_py(s).str(); });
    mod.def("new_symbol", &new_symbol);
    mod.def("symbol_root", &symbol_root);
    mod.def("symbols_set_equal", &symbols_set_equal);
    mod.def("pshape_parse", [](const std::string& s) { return pshape_to_py(PShape::parse(s)); });

    // ------------------------------------------------------------------ Node
    py::class_<Node, NodePtr>(mod, "Node")
        .def_readonly("type", &Node::type)
        .def_readwrite("version", &Node::version)
        .def_readwrite("name", &Node::name)
        .def_readonly("id", &Node::id)
        .def("num_inputs", &Node::num_inputs)
        .def("num_outputs", &Node::num_outputs)
        .def("input_source", [](Node& n, size_t i) { const Output& o = n.input(i); return py::make_tuple(o.node, o.index); })
        .def("set_input", [](Node& n, size_t i, const py::object& src) { n.set_input(i, out_from_py(src)); })
        .def("add_input", [](Node& n, const py::object& src) { n.add_input(out_from_py(src)); })
        .def("output_shape", [](Node& n, size_t i) { return pshape_to_py(n.outs.at(i).shape); })
        .def("output_type", [](Node& n, size_t i) { return std::string(et_name(n.outs.at(i).et)); })
        .def("output_names", [](Node& n, size_t i) { return n.outs.at(i).names; })
        .def("set_output_names", [](Node& n, size_t i, std::set<std::string> names) { n.outs.at(i).names = std::move(names); })
        .def("output_rt_info", [](Node& n, size_t i) { return attrmap_to_py(n.outs.at(i).rt); })
        .def("set_output_rt_info", [](Node& n, size_t i, const std::string& k, const py::object& v) { n.outs.at(i).rt[k] = py_to_attr(v); })
        .def("output_users", [](Node& n, size_t i) {
            py::list l;
            for (auto& u : n.outs.at(i).uses) l.append(py::make_tuple(u.node->shared_from_this(), u.input));
            return l;
        })
        .def("attrs", [](Node& n) { py::dict d; for (auto& kv : n.attrs) d[py::str(kv.first)] = attr_to_py(kv.second); return d; })
        .def("attr_names", [](Node& n) { std::vector<std::string> v; for (auto& kv : n.attrs) v.push_back(kv.first); return v; })
        .def("has_attr", &Node::has_attr)
        .def("get_attr", [](Node& n, const std::string& k) { return attr_to_py(n.attr(k)); })
        .def("set_attr", [](Node& n, const std::string& k, const py::object& v) {
            Attr a = py_to_attr(v);
            if (n.schema) for (auto& spec : n.schema->attrs) if (spec.name == k) {
                if (spec.kind == Attr::FLOAT && a.kind == Attr::INT) a = Attr::Float((double)a.i);
                if (spec.kind == Attr::TYPE && a.kind == Attr::STR) a = Attr::Type(et_from_name(a.s));
                if (spec.kind == Attr::PSHAPE && a.kind == Attr::INTS) a = Attr::Shape_(PShape(Shape(a.is)));
                if (spec.kind == Attr::FLOAT && spec.f32) a.f = double(float(a.f));
            }
            n.set_attr(k, a);
        })
        .def("rt_info", [](Node& n) { return attrmap_to_py(n.rt_info); })
        .def("set_rt_info", [](Node& n, const std::string& k, const py::object& v) { n.rt_info[k] = py_to_attr(v); })
        .def("erase_rt_info", [](Node& n, const std::string& k) { n.rt_info.erase(k); })
        .def("validate", &Node::validate_and_infer)
        .def("constant_data", [](Node& n) { OVC_CHECK(n.is_constant(), "not a Constant"); return PyTensor::pack(n.constant); })
        .def("bodies", [](Node& n) { return n.bodies; })
        .def("set_bodies", [](Node& n, std::vector<ModelPtr> b) { n.bodies = std::move(b); })
        .def("clone_with_new_inputs", [](Node& n, const py::iterable& ins) { return n.clone_with_new_inputs(outs_from_py(ins)); })
        .def("has_evaluate", [](Node& n) { return n.schema && bool(n.schema->eval); })
        .def("__repr__", [](Node& n) { return "<Node " + n.description() + ">"; });

    mod.def("make_node", [](const std::string& type, const std::string& version, const py::iterable& inputs, const py::dict& attrs, bool infer) {
        std::vector<std::pair<std::string, Attr>> a;
        for (auto kv : attrs) a.emplace_back(py::cast<std::string>(py::str(kv.first)), py_to_attr(kv.second));
        return make_node(type, version, outs_from_py(inputs), a, infer);
    }, py::arg("type"), py::arg("version"), py::arg("inputs"), py::arg("attrs") = py::dict(), py::arg("infer") = true);
    // Operations defined in Python: `infer(node) -> [(element type name, partial shape), ...]` and, optionally,
    // `evaluate(node, [(array, type, shape), ...]) -> [(array, type name), ...]`. The callables live for the whole process.
    mod.def("register_custom_op", [](const std::string& type, const std::string& version, py::object infer, py::object eval, const py::dict& attrs) {
        auto* infer_p = new py::object(std::move(infer));
        auto* eval_p = eval.is_none() ? nullptr : new py::object(std::move(eval));
        OpSchema s;
        s.type = type;
        s.version = version;
        for (auto kv : attrs) {      // name -> default value: gives the IR reader the kind of every attribute
            AttrSpec a;
            a.name = py::cast<std::string>(py::str(kv.first));
            a.def = py_to_attr(kv.second);
            a.kind = a.def.kind;
            s.attrs.push_back(a);
        }
        s.infer = [infer_p](Node& n) {
            py::gil_scoped_acquire g;
            py::list outs = py::cast<py::list>((*infer_p)(n.shared_from_this()));
            n.set_num_outputs(outs.size());
            size_t i = 0;
            for (auto o : outs) {
                auto t = py::cast<py::tuple>(o);
                n.set_output(i++, et_from_name(py::cast<std::string>(t[0])), pshape_from_py(t[1]));
            }
        };
        if (eval_p)
            s.eval = [eval_p](const Node& n, const std::vector<Tensor>& in, std::vector<Tensor>& out, EvalContext&) {
                py::gil_scoped_acquire g;
                py::list pin;
                for (auto& t : in) pin.append(PyTensor::pack(t));
                py::object r = (*eval_p)(const_cast<Node&>(n).shared_from_this(), pin);
                if (r.is_none()) return false;
                out.clear();
                for (auto o : py::cast<py::list>(r)) {
                    auto t = py::cast<py::tuple>(o);
                    py::array arr = py::cast<py::array>(t[0]);
                    std::vector<int64_t> shape(arr.shape(), arr.shape() + arr.ndim());
                    out.push_back(tensor_from_array(arr, py::cast<std::string>(t[1]), shape, false));
                }
                return true;
            };
        OpRegistry::get().add(std::move(s));
    }, py::arg("type"), py::arg("version"), py::arg("infer"), py::arg("evaluate") = py::none(), py::arg("attrs") = py::dict());
    mod.def("make_constant", [](py::array arr, const std::string& et, std::vector<int64_t> shape, bool share) {
        return make_constant(tensor_from_array(arr, et, shape, share));
    }, py::arg("array"), py::arg("element_type"), py::arg("shape"), py::arg("share") = false);
    mod.def("make_string_constant", [](std::vector<std::string> values, std::vector<int64_t> shape) {
        Tensor t(ET::string, shape);
        OVC_CHECK((int64_t)values.size() == t.numel(), "string constant: value count does not match the shape");
        t.strings = std::move(values);
        return make_constant(t);
    });
    mod.def("make_parameter", [](const std::string& et, const py::object& shape, const std::string& name) {
        return make_parameter(et_from_name(et), pshape_from_py(shape), name);
    });
    mod.def("make_result", [](const py::object& src) { return make_result(out_from_py(src)); });
    mod.def("replace_output", [](const py::object& from, const py::object& to) { replace_output(out_from_py(from), out_from_py(to)); });
    mod.def("replace_node", [](const NodePtr& a, const NodePtr& b) { replace_node(a, b); });
    mod.def("copy_runtime_info", [](std::vector<NodePtr> from, std::vector<NodePtr> to) { copy_runtime_info(from, to); });
    mod.def("op_schemas", [] {
        py::list l;
        for (auto* s : OpRegistry::get().all()) {
            py::list attrs;
            for (auto& a : s->attrs) attrs.append(py::make_tuple(a.name, (int)a.kind, attr_to_py(a.def)));
            l.append(py::make_tuple(s->type, s->version, attrs, s->min_inputs, s->max_inputs, bool(s->eval)));
        }
        return l;
    });
    mod.def("types_in_opset", [](const std::string& o) { return OpRegistry::get().types_in_opset(o); });

    // ------------------------------------------------------------------ Model
    py::class_<Model, ModelPtr>(mod, "Model")
        .def(py::init([](std::vector<NodePtr> results, std::vector<NodePtr> sinks, std::vector<NodePtr> params, const std::string& name) {
            return std::make_shared<Model>(std::move(results), std::move(sinks), std::move(params), name);
        }))
        .def_readwrite("name", &Model::name)
        .def_readwrite("params", &Model::params)
        .def_readwrite("results", &Model::results)
        .def_readwrite("sinks", &Model::sinks)
        .def("ordered_ops", &Model::ordered_ops)
        .def("validate", &Model::validate)
        .def("clone", &Model::clone)
        .def("is_dynamic", &Model::is_dynamic)
        .def("reshape", [](Model& m, const py::dict& shapes) {
            std::map<size_t, PShape> s;
            for (auto kv : shapes) s[py::cast<size_t>(kv.first)] = pshape_from_py(kv.second);
            m.reshape(s);
        })
        .def("variables", [](Model& m) {
            py::list l;
            for (auto& v : m.variables()) l.append(py::make_tuple(v.id, pshape_to_py(v.shape), std::string(et_name(v.et))));
            return l;
        })
        .def("rt_info", [](Model& m) { return attrmap_to_py(m.rt_info); })
        .def("set_rt_info", [](Model& m, const std::string& k, const py::object& v) { m.rt_info[k] = py_to_attr(v); })
        .def("erase_rt_info", [](Model& m, const std::string& k) { m.rt_info.erase(k); })
        .def("add_parameters", &Model::add_parameters)
        .def("remove_parameter", &Model::remove_parameter)
        .def("add_results", &Model::add_results)
        .def("remove_result", &Model::remove_result)
        .def("add_sinks", &Model::add_sinks)
        .def("remove_sink", &Model::remove_sink)
        .def("graph_size", &Model::graph_size);

    // ------------------------------------------------------------------ IR
    mod.def("serialize", [](const Model& m, int version, bool deterministic) {
        SerializeOptions o;
        o.version = version;
        o.deterministic = deterministic;
        std::string xml, bin;
        {
            py::gil_scoped_release r;
            serialize_model(m, xml, bin, o);
        }
        return py::make_tuple(py::bytes(xml), py::bytes(bin));
    }, py::arg("model"), py::arg("version") = 11, py::arg("deterministic") = false);
    mod.def("deserialize", [](const std::string& xml, const py::object& weights) {
        BufferPtr w;
        if (!weights.is_none()) {
            py::buffer b = py::cast<py::buffer>(weights);
            py::buffer_info info = b.request();
            const size_t n = (size_t)info.size * (size_t)info.itemsize;
            std::shared_ptr<py::object> keep(new py::object(weights), GilDeleter());
            w = std::make_shared<Buffer>(static_cast<uint8_t*>(info.ptr), n, std::shared_ptr<void>(keep, keep.get()));
        }
        return deserialize_model(xml, w);
    }, py::arg("xml"), py::arg("weights") = py::none());
    mod.def("read_model_files", [](const std::string& x, const std::string& b) { py::gil_scoped_release r; return read_model_files(x, b); },
            py::arg("xml_path"), py::arg("bin_path") = "");
    mod.def("save_model_files", [](const Model& m, const std::string& x, const std::string& b, int version) {
        SerializeOptions o;
        o.version = version;
        py::gil_scoped_release r;
        save_model_files(m, x, b, o);
    }, py::arg("model"), py::arg("xml_path"), py::arg("bin_path") = "", py::arg("version") = 11);
    mod.def("model_hash", [](const Model& m) { return model_hash(m); });

    // ------------------------------------------------------------------ evaluation
    py::class_<VariableStore, std::shared_ptr<VariableStore>>(mod, "VariableStore")
        .def(py::init<>())
        .def("reset", &VariableStore::reset)
        .def("names", [](VariableStore& s) { std::vector<std::string> v; for (auto& kv : s.values) v.push_back(kv.first); return v; })
        .def("get", [](VariableStore& s, const std::string& k) -> py::object { auto it = s.values.find(k); if (it == s.values.end()) return py::none(); return PyTensor::pack(it->second); })
        .def("set", [](VariableStore& s, const std::string& k, py::array a, const std::string& et, std::vector<int64_t> shape) { s.values[k] = tensor_from_array(a, et, shape, false); })
        .def("erase", [](VariableStore& s, const std::string& k) { s.values.erase(k); });

    mod.def("evaluate", [](const Model& m, const py::list& inputs, std::shared_ptr<VariableStore> vars, int threads, bool profile) {
        std::vector<Tensor> ins;
        for (auto h : inputs) {
            auto t = py::cast<py::tuple>(h);
            if (py::isinstance<py::list>(t[0])) {   // string tensor
                Tensor st(ET::string, py::cast<std::vector<int64_t>>(t[2]));
                size_t i = 0;
                for (auto s : py::cast<py::list>(t[0])) st.strings.at(i++) = py::cast<std::string>(s);
                ins.push_back(st);
            } else {
                ins.push_back(tensor_from_array(py::cast<py::array>(t[0]), py::cast<std::string>(t[1]), py::cast<std::vector<int64_t>>(t[2]), true));
            }
        }
        std::vector<Tensor> outs;
        std::vector<std::pair<std::string, double>> prof;
        {
            py::gil_scoped_release r;
            EvalContext ctx;
            ctx.variables = vars.get();
            ctx.num_threads = threads;
            outs = evaluate_model(m, ins, ctx, profile ? &prof : nullptr);
        }
        py::list res;
        for (auto& t : outs) res.append(PyTensor::pack(t));
        return py::make_tuple(res, prof);
    }, py::arg("model"), py::arg("inputs"), py::arg("variables") = nullptr, py::arg("threads") = 0, py::arg("profile") = false);
    mod.def("constant_value", [](const py::object& o) -> py::object {
        Tensor t;
        if (!try_constant_value(out_from_py(o), t)) return py::none();
        return PyTensor::pack(t);
    });

    // ------------------------------------------------------------------ passes and patterns
    py::class_<PatternNode, PatternPtr>(mod, "PatternNode")
        .def_readwrite("name", &PatternNode::name)
        .def_readwrite("output_index", &PatternNode::output_index);
    auto wrap_pred = [](const py::object& pred) -> ValuePredicate {
        if (pred.is_none()) return nullptr;
        py::object p = pred;
        return [p](const Output& o) { py::gil_scoped_acquire g; return py::cast<bool>(p(py::make_tuple(o.node, o.index))); };
    };
    mod.def("pattern_any", [wrap_pred](const py::object& pred) { return pattern::any_input(wrap_pred(pred)); }, py::arg("pred") = py::none());
    mod.def("pattern_type", [wrap_pred](std::vector<std::string> types, std::vector<PatternPtr> inputs, const py::object& pred) {
        return pattern::wrap_type(std::move(types), std::move(inputs), wrap_pred(pred));
    }, py::arg("types"), py::arg("inputs") = std::vector<PatternPtr>(), py::arg("pred") = py::none());
    mod.def("pattern_optional", [wrap_pred](std::vector<std::string> types, std::vector<PatternPtr> inputs, const py::object& pred) {
        return pattern::optional(std::move(types), std::move(inputs), wrap_pred(pred));
    }, py::arg("types"), py::arg("inputs"), py::arg("pred") = py::none());
    mod.def("pattern_or", [](std::vector<PatternPtr> alts) { return pattern::any_of(std::move(alts)); });

    py::class_<Matcher, std::shared_ptr<Matcher>>(mod, "Matcher")
        .def(py::init([](PatternPtr root, const std::string& name) { return std::make_shared<Matcher>(root, name); }), py::arg("root"), py::arg("name") = "")
        .def("match", [](Matcher& m, const py::object& v) { return m.match(out_from_py(v)); })
        .def("get_match_root", &Matcher::match_root)
        .def("get_match_value", [](Matcher& m) { auto o = m.match_value(); return py::make_tuple(o.node, o.index); })
        .def("get_matched_nodes", &Matcher::matched_nodes)
        .def("has", [](Matcher& m, const PatternPtr& p) { return m.has(p); })
        .def("at", [](Matcher& m, const PatternPtr& p) { auto o = m.at(p); return py::make_tuple(o.node, o.index); })
        .def_property_readonly("name", &Matcher::name);

    py::class_<ModelPass, std::shared_ptr<ModelPass>>(mod, "ModelPass")
        .def_readwrite("name", &ModelPass::name)
        .def("run_on_model", [](ModelPass& p, const ModelPtr& m) { return p.run_on_model(m); });
    mod.def("make_pass", [](const std::string& name, const py::dict& options) {
        AttrMap o;
        for (auto kv : options) o[py::cast<std::string>(py::str(kv.first))] = py_to_attr(kv.second);
        return make_pass(name, o);
    }, py::arg("name"), py::arg("options") = py::dict());
    mod.def("make_python_pass", [](const std::string& name, py::object fn) {
        auto p = std::make_shared<PyModelPass>();
        p->name = name;
        p->fn = std::move(fn);
        return std::static_pointer_cast<ModelPass>(p);
    });
    mod.def("make_matcher_pass", [](const std::string& name, PatternPtr root, py::object callback) {
        auto mp = std::make_shared<MatcherPass>(name, root, [callback](Matcher& m) {
            py::gil_scoped_acquire g;
            return py::cast<bool>(callback(py::cast(&m, py::return_value_policy::reference)));
        });
        auto gr = std::make_shared<GraphRewrite>();
        gr->name = name;
        gr->add(mp);
        return std::static_pointer_cast<ModelPass>(gr);
    });
    mod.def("available_passes", &available_passes);
    py::class_<PassManager>(mod, "PassManager")
        .def(py::init<>())
        .def("add", &PassManager::add)
        .def("disable", &PassManager::disable)
        .def("enable", &PassManager::enable)
        .def_readwrite("validate_after_each", &PassManager::validate_after_each)
        .def("run", &PassManager::run)
        .def("timings", [](PassManager& pm) { py::list l; for (auto& t : pm.timings()) l.append(py::make_tuple(t.name, t.ms, t.changed)); return l; });
    mod.def("run_moc_transformations", &run_moc_transformations, py::arg("model"), py::arg("constant_folding") = true);
    mod.def("run_llm_fusions", &run_llm_fusions);
    mod.def("sdpa_to_paged_attention", [](const ModelPtr& m, const py::dict& options) {
        AttrMap o;
        for (auto kv : options) o[py::cast<std::string>(py::str(kv.first))] = py_to_attr(kv.second);
        return sdpa_to_paged_attention(m, o);
    }, py::arg("model"), py::arg("options") = py::dict());
    mod.def("make_stateful", &make_stateful);
    mod.def("stateful_to_stateless", &stateful_to_stateless);

    // ------------------------------------------------------------------ host topology
    py::class_<CpuTopology>(mod, "CpuTopology")
        .def_readonly("sockets", &CpuTopology::sockets)
        .def_readonly("numa_nodes", &CpuTopology::numa_nodes)
        .def_readonly("cores", &CpuTopology::cores)
        .def_readonly("processors", &CpuTopology::processors)
        .def_readonly("proc_type_table", &CpuTopology::proc_type_table)
        .def_readonly("cpu_mapping_table", &CpuTopology::cpu_mapping_table)
        .def_readonly("flags", &CpuTopology::flags)
        .def("has", &CpuTopology::has);
    mod.def("read_cpu_topology", &read_cpu_topology, py::arg("root") = "/");
    mod.def("host_cpu_topology", []() { return host_cpu_topology(); });
    mod.def("parse_cpu_list", &parse_cpu_list);
    mod.def("plan_streams", [](const CpuTopology& t, const std::string& hint, int streams, int threads) {
        const StreamsPlan p = plan_streams(t, hint, streams, threads);
        return py::make_tuple(p.num_streams, p.threads_per_stream);
    }, py::arg("topology"), py::arg("hint") = "LATENCY", py::arg("num_streams") = 0, py::arg("num_threads") = 0);
    mod.def("compress_weights", &compress_weights, py::arg("model"), py::arg("mode") = "int4_asym", py::arg("group_size") = 128,
            py::arg("ratio") = 1.0, py::arg("all_layers") = false);
    mod.def("compress_model_to_f16", &compress_model_to_f16);

    // ------------------------------------------------------------------ runtime
    py::class_<TaskExecutor, std::shared_ptr<TaskExecutor>>(mod, "TaskExecutor")
        .def(py::init<int, std::string>(), py::arg("num_threads"), py::arg("name") = "executor")
        .def("num_threads", &TaskExecutor::num_threads)
        .def("run", [](TaskExecutor& e, py::object fn) {
            auto held = std::shared_ptr<py::object>(new py::object(std::move(fn)), GilDeleter());
            e.run([held] { py::gil_scoped_acquire g; (*held)(); });
        });

    py::class_<AsyncRequest, std::shared_ptr<AsyncRequest>>(mod, "AsyncRequest")
        .def(py::init([] { return std::make_shared<AsyncRequest>(); }))
        .def("set_pipeline", [](AsyncRequest& r, const py::list& stages) {
            std::vector<AsyncRequest::Stage> st;
            for (auto h : stages) {
                auto t = py::cast<py::tuple>(h);
                std::shared_ptr<TaskExecutor> ex = t[0].is_none() ? nullptr : py::cast<std::shared_ptr<TaskExecutor>>(t[0]);
                auto held = std::shared_ptr<py::object>(new py::object(py::reinterpret_borrow<py::object>(t[1])), GilDeleter());
                st.emplace_back(ex, [held] { py::gil_scoped_acquire g; (*held)(); });
            }
            r.set_pipeline(std::move(st));
        })
        .def("set_callback", [](AsyncRequest& r, const py::object& cb) {
            if (cb.is_none()) { r.set_callback(nullptr); return; }
            auto held = std::shared_ptr<py::object>(new py::object(cb), GilDeleter());
            r.set_callback([held](std::exception_ptr e) {
                py::gil_scoped_acquire g;
                py::object err = py::none();
                if (e) {
                    try { std::rethrow_exception(e); }
                    catch (py::error_already_set& pe) { err = pe.value(); }
                    catch (const std::exception& se) { err = py::str(se.what()); }
                }
                (*held)(err);
            });
        })
        .def("set_cancel_hook", [](AsyncRequest& r, py::object fn) {
            auto held = std::shared_ptr<py::object>(new py::object(std::move(fn)), GilDeleter());
            r.set_cancel_hook([held] { py::gil_scoped_acquire g; (*held)(); });
        })
        .def("infer", [](AsyncRequest& r) { py::gil_scoped_release g; r.infer(); })
        .def("start_async", [](AsyncRequest& r) { py::gil_scoped_release g; r.start_async(); })
        .def("wait", [](AsyncRequest& r) { py::gil_scoped_release g; r.wait(); })
        .def("wait_for", [](AsyncRequest& r, int64_t ms) { py::gil_scoped_release g; return r.wait_for(ms); })
        .def("cancel", [](AsyncRequest& r) { py::gil_scoped_release g; r.cancel(); })
        .def("state", [](AsyncRequest& r) { return (int)r.state(); })
        .def("latency_ms", &AsyncRequest::last_latency_ms);

    py::class_<IdleQueue, std::shared_ptr<IdleQueue>>(mod, "IdleQueue")
        .def(py::init<size_t>())
        .def("size", &IdleQueue::size)
        .def("is_ready", &IdleQueue::is_ready)
        .def("get_idle", [](IdleQueue& q) { py::gil_scoped_release g; return q.get_idle(); })
        .def("acquire", [](IdleQueue& q) { py::gil_scoped_release g; return q.acquire(); })
        .def("release", &IdleQueue::release)
        .def("wait_all", [](IdleQueue& q) { py::gil_scoped_release g; q.wait_all(); })
        .def("set_error", [](IdleQueue& q, const std::string& msg) { q.set_error(std::make_exception_ptr(Error(msg))); });

    // ------------------------------------------------------------------ scheduler
    py::class_<SchedulerConfig>(mod, "SchedulerConfig")
        .def(py::init<>())
        .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
        .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
        .def_readwrite("num_kv_blocks", &SchedulerConfig::num_kv_blocks)
        .def_readwrite("block_size", &SchedulerConfig::block_size)
        .def_readwrite("dynamic_split_fuse", &SchedulerConfig::dynamic_split_fuse)
        .def_readwrite("enable_prefix_caching", &SchedulerConfig::enable_prefix_caching);
    py::class_<SeqState, SeqPtr>(mod, "SeqState")
        .def_readonly("request_id", &SeqState::request_id)
        .def_readonly("generated", &SeqState::generated)
        .def_readonly("num_computed", &SeqState::num_computed)
        .def_readonly("finished", &SeqState::finished)
        .def_readonly("slot", &SeqState::slot)
        .def_readonly("blocks", &SeqState::blocks)
        .def_readonly("num_cached_tokens", &SeqState::num_cached_tokens)
        .def("num_generated", [](SeqState& s) { return s.generated.size(); })
        .def("generated_at", [](SeqState& s, size_t i) { return s.generated.at(i); })
        .def("prompt_len", [](SeqState& s) { return s.prompt.size(); })
        .def("total_len", &SeqState::total_len);
    py::class_<DescLayout>(mod, "DescLayout")
        .def(py::init<>())
        .def_readwrite("ids", &DescLayout::ids).def_readwrite("positions", &DescLayout::positions).def_readwrite("slot_map", &DescLayout::slot_map)
        .def_readwrite("tok_src", &DescLayout::tok_src).def_readwrite("tok_dst", &DescLayout::tok_dst).def_readwrite("logit_idx", &DescLayout::logit_idx)
        .def_readwrite("past_lens", &DescLayout::past_lens).def_readwrite("subsequence_begins", &DescLayout::subsequence_begins)
        .def_readwrite("block_indices_begins", &DescLayout::block_indices_begins).def_readwrite("block_indices", &DescLayout::block_indices)
        .def_readwrite("Tcap", &DescLayout::Tcap).def_readwrite("Bcap", &DescLayout::Bcap).def_readwrite("blocks_cap", &DescLayout::blocks_cap);
    py::class_<ScheduledStep>(mod, "ScheduledStep")
        .def_readonly("seqs", &ScheduledStep::seqs)
        .def_readonly("num_new", &ScheduledStep::num_new)
        .def_readonly("T", &ScheduledStep::T)
        .def_readonly("max_q_len", &ScheduledStep::max_q_len)
        .def_readonly("max_ctx", &ScheduledStep::max_ctx);
    py::class_<Produced>(mod, "Produced")
        .def_readonly("seq", &Produced::seq)
        .def_readonly("gen_index", &Produced::gen_index)
        .def_readonly("row", &Produced::row);
    py::class_<Scheduler>(mod, "Scheduler")
        .def(py::init<const SchedulerConfig&>())
        .def("add", [](Scheduler& s, int64_t rid, std::vector<int32_t> prompt, int64_t max_new, int32_t eos, bool ignore_eos) {
            return s.add(rid, std::move(prompt), max_new, eos, ignore_eos);
        })
        .def("has_unfinished", &Scheduler::has_unfinished)
        .def("schedule", [](Scheduler& s) -> py::object { ScheduledStep st; if (!s.schedule(st)) return py::none(); return py::cast(st); })
        .def("fill", [](Scheduler& s, const ScheduledStep& st, py::array_t<int32_t> desc, const DescLayout& lay, bool host_ids) {
            s.fill(st, desc.mutable_data(), lay, host_ids);
        }, py::arg("step"), py::arg("desc"), py::arg("layout"), py::arg("host_ids_for_generated") = false)
        .def("commit", [](Scheduler& s, const ScheduledStep& st, const py::object& tokens) {
            if (tokens.is_none()) return s.commit(st, nullptr);
            auto a = py::cast<py::array_t<int32_t>>(tokens);
            return s.commit(st, a.data());
        }, py::arg("step"), py::arg("tokens") = py::none())
        .def("patch", [](Scheduler& s, const std::vector<Produced>& p, py::array_t<int32_t> tokens) { s.patch(p, tokens.data()); })
        .def("num_free_blocks", &Scheduler::num_free_blocks)
        .def("num_cached_blocks", &Scheduler::num_cached_blocks)
        .def("prefix_hit_tokens", &Scheduler::prefix_hit_tokens)
        .def("num_preemptions", &Scheduler::num_preemptions)
        .def("num_running", &Scheduler::num_running)
        .def("num_waiting", &Scheduler::num_waiting);
}
