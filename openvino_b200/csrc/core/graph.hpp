// Graph IR of the native core: tensors, nodes, models, the table-driven operation registry.
//
// Roles covered (reference: ov::Model src/core/include/openvino/core/model.hpp:96-515, ov::Node
// src/core/include/openvino/core/node.hpp:188-437, Output/Input handles, ov::Tensor
// src/core/include/openvino/runtime/tensor.hpp:55-242, the opset tables under
// src/core/include/openvino/opsets/). Unlike the reference's class-per-op design every operation
// here is a row in a registry: attribute schema (in serialisation order), shape/type inference
// function and reference evaluation function. One Node class carries any operation.
#pragma once
#include <atomic>
#include <functional>
#include <mutex>
#include <unordered_map>
#include <unordered_set>

#include "types.hpp"

namespace ovc {

// ------------------------------------------------------------------------------------ tensors
struct Buffer {
    uint8_t* data = nullptr;
    size_t size = 0;
    std::vector<uint8_t> owned;
    std::shared_ptr<void> keeper;   // keeps external memory (numpy array, mmap) alive
    Buffer() = default;
    explicit Buffer(size_t n) : size(n), owned(n ? n : 1) { data = owned.data(); }
    Buffer(uint8_t* p, size_t n, std::shared_ptr<void> k) : data(p), size(n), keeper(std::move(k)) {}
};
using BufferPtr = std::shared_ptr<Buffer>;

struct Tensor {
    ET et = ET::dynamic;
    Shape shape;
    BufferPtr buf;
    std::vector<std::string> strings;   // payload of ET::string tensors
    Tensor() = default;
    Tensor(ET t, Shape s) : et(t), shape(std::move(s)) {
        if (t != ET::string) buf = std::make_shared<Buffer>(et_byte_size(t, (size_t)shape_size(shape)));
        else strings.resize((size_t)shape_size(shape));
    }
    Tensor(ET t, Shape s, BufferPtr b) : et(t), shape(std::move(s)), buf(std::move(b)) {}
    int64_t numel() const { return shape_size(shape); }
    size_t byte_size() const { return et_byte_size(et, (size_t)numel()); }
    uint8_t* data() const { return buf ? buf->data : nullptr; }
    template <class T> T* ptr() const { return reinterpret_cast<T*>(data()); }
    bool defined() const { return et != ET::dynamic; }
};

// Element access through a common compute type (float for reals, int64 for integers).
double get_elem_f64(const Tensor& t, int64_t i);
int64_t get_elem_i64(const Tensor& t, int64_t i);
void set_elem_f64(Tensor& t, int64_t i, double v);
void set_elem_i64(Tensor& t, int64_t i, int64_t v);
std::vector<float> to_f32(const Tensor& t);
std::vector<double> to_f64(const Tensor& t);
std::vector<int64_t> to_i64(const Tensor& t);
Tensor from_f32(ET et, const Shape& s, const std::vector<float>& v);
Tensor from_f64(ET et, const Shape& s, const std::vector<double>& v);
Tensor from_i64(ET et, const Shape& s, const std::vector<int64_t>& v);
Tensor convert_tensor(const Tensor& t, ET to);

// ------------------------------------------------------------------------------------ graph
class Node;
class Model;
using NodePtr = std::shared_ptr<Node>;
using ModelPtr = std::shared_ptr<Model>;

struct Output {
    NodePtr node;
    size_t index = 0;
    Output() = default;
    Output(NodePtr n, size_t i = 0) : node(std::move(n)), index(i) {}
    bool operator==(const Output& o) const { return node == o.node && index == o.index; }
    bool operator!=(const Output& o) const { return !(*this == o); }
    bool operator<(const Output& o) const { return node.get() < o.node.get() || (node == o.node && index < o.index); }
    const PShape& shape() const;
    ET et() const;
    explicit operator bool() const { return node != nullptr; }
};

struct Use {           // one consumer of an output
    Node* node;
    size_t input;
};

struct OutDesc {
    PShape shape = PShape::dynamic();
    ET et = ET::dynamic;
    std::set<std::string> names;
    AttrMap rt;
    std::vector<Use> uses;
    // bound evaluation cache (value known at shape-inference time, e.g. ShapeOf -> Gather chains)
    std::shared_ptr<Tensor> lower, upper;
};

struct EvalContext;
struct OpSchema;

class Node : public std::enable_shared_from_this<Node> {
public:
    Node(const OpSchema* schema, std::vector<Output> inputs, std::vector<std::pair<std::string, Attr>> attrs);
    ~Node();
    Node(const Node&) = delete;

    const OpSchema* schema;
    std::string type;        // "MatMul"
    std::string version;     // "opset1"
    std::string name;        // friendly name
    uint64_t id;             // creation sequence number
    std::vector<std::pair<std::string, Attr>> attrs;   // in schema (serialisation) order; extra attrs appended
    AttrMap rt_info;
    std::vector<AttrMap> input_rt;                      // per input port
    std::vector<OutDesc> outs;
    Tensor constant;                                    // payload of Constant nodes
    std::vector<ModelPtr> bodies;                       // sub-graphs (If / Loop / TensorIterator)

    // inputs
    size_t num_inputs() const { return inputs_.size(); }
    const Output& input(size_t i) const { return inputs_.at(i); }
    const std::vector<Output>& inputs() const { return inputs_; }
    void set_input(size_t i, const Output& src);
    void add_input(const Output& src);
    void remove_inputs_from(size_t first);
    NodePtr input_node(size_t i) const { return inputs_.at(i).node; }
    const PShape& in_shape(size_t i) const { return inputs_.at(i).shape(); }
    ET in_et(size_t i) const { return inputs_.at(i).et(); }

    // outputs
    size_t num_outputs() const { return outs.size(); }
    Output output(size_t i = 0) { return Output(shared_from_this(), i); }
    void set_output(size_t i, ET et, const PShape& s);
    void set_num_outputs(size_t n) { outs.resize(n); }

    // attributes
    bool has_attr(const std::string& k) const;
    const Attr& attr(const std::string& k) const;
    Attr* find_attr(const std::string& k);
    void set_attr(const std::string& k, Attr v);
    int64_t attr_int(const std::string& k, int64_t d = 0) const;
    double attr_float(const std::string& k, double d = 0) const;
    bool attr_bool(const std::string& k, bool d = false) const;
    std::string attr_str(const std::string& k, const std::string& d = "") const;
    std::vector<int64_t> attr_ints(const std::string& k) const;

    bool is(const char* t) const { return type == t; }
    bool is_constant() const { return type == "Constant"; }
    bool is_parameter() const { return type == "Parameter"; }
    bool is_result() const { return type == "Result"; }

    void validate_and_infer();      // runs the schema's inference function
    NodePtr clone_with_new_inputs(const std::vector<Output>& inputs) const;
    std::string description() const;

private:
    std::vector<Output> inputs_;
    void attach(size_t i);
    void detach(size_t i);
};

// Replace every use of `from` by `to`.
void replace_output(const Output& from, const Output& to);
// Replace all outputs of `target` by the outputs of `replacement` (friendly name is carried over when asked).
void replace_node(const NodePtr& target, const NodePtr& replacement, bool copy_name = true);
void copy_runtime_info(const std::vector<NodePtr>& from, const std::vector<NodePtr>& to);

// ------------------------------------------------------------------------------------ op registry
struct AttrSpec {
    std::string name;
    Attr::Kind kind;
    Attr def;
    bool required = false;
    bool f32 = false;          // FLOAT stored as float in the reference: values are rounded through float
    bool optional_in_ir = false;   // not written when equal to the default (visitor skips it)
};

using InferFn = std::function<void(Node&)>;
using EvalFn = std::function<bool(const Node&, const std::vector<Tensor>&, std::vector<Tensor>&, EvalContext&)>;

struct OpSchema {
    std::string type;
    std::string version;
    std::vector<AttrSpec> attrs;
    InferFn infer;
    EvalFn eval;
    int min_inputs = 0;
    int max_inputs = -1;
    bool commutative = false;
    bool has_side_effects = false;   // Assign, ReadValue, Result ...: never folded / removed
};

class OpRegistry {
public:
    static OpRegistry& get();
    void add(OpSchema s);
    void alias(const std::string& type, const std::string& version, const std::string& as_version);
    const OpSchema* find(const std::string& type, const std::string& version) const;   // exact
    const OpSchema* find_latest(const std::string& type) const;                        // newest registered version
    const OpSchema* find_ci(const std::string& type, const std::string& version) const; // case-insensitive type (IR reader)
    std::vector<const OpSchema*> all() const;
    std::vector<std::string> types_in_opset(const std::string& opset) const;
private:
    std::map<std::pair<std::string, std::string>, std::shared_ptr<OpSchema>> ops_;
    std::map<std::string, std::vector<std::string>> versions_;   // type -> versions in registration order
};

void register_all_ops();   // idempotent

// Node factory: schema lookup (version "" = newest), defaults for missing attributes, inference.
NodePtr make_node(const std::string& type, const std::string& version, const std::vector<Output>& inputs,
                  const std::vector<std::pair<std::string, Attr>>& attrs = {}, bool infer = true);
NodePtr make_constant(const Tensor& t);
NodePtr make_constant_i64(const std::vector<int64_t>& v, ET et = ET::i64, bool scalar = false);
NodePtr make_constant_f32(const std::vector<float>& v, const Shape& shape, ET et = ET::f32);
NodePtr make_parameter(ET et, const PShape& shape, const std::string& name = "");
NodePtr make_result(const Output& src);

// ------------------------------------------------------------------------------------ model
struct VariableInfo {
    std::string id;
    PShape shape;
    ET et = ET::dynamic;
};

class Model : public std::enable_shared_from_this<Model> {
public:
    Model(std::vector<NodePtr> results, std::vector<NodePtr> sinks, std::vector<NodePtr> params, std::string name = "");
    std::string name;
    std::vector<NodePtr> params, results, sinks;
    AttrMap rt_info;

    std::vector<NodePtr> ordered_ops() const;      // topological order (inputs before users)
    std::vector<NodePtr> ops() const { return ordered_ops(); }
    void validate();                               // re-run inference over the whole graph
    ModelPtr clone() const;
    void reshape(const std::map<size_t, PShape>& new_shapes);
    bool is_dynamic() const;
    std::vector<VariableInfo> variables() const;
    Output input(size_t i) const { return Output(params.at(i), 0); }
    Output output(size_t i) const { return Output(results.at(i), 0); }
    NodePtr find_node(const std::string& friendly_name) const;
    void add_parameters(const std::vector<NodePtr>& p);
    void remove_parameter(const NodePtr& p);
    void add_results(const std::vector<NodePtr>& r);
    void remove_result(const NodePtr& r);
    void add_sinks(const std::vector<NodePtr>& s);
    void remove_sink(const NodePtr& s);
    size_t graph_size() const;
};

std::vector<NodePtr> topological_sort(const std::vector<NodePtr>& roots);
uint64_t next_node_id();

// ------------------------------------------------------------------------------------ evaluation
struct VariableStore {
    std::map<std::string, Tensor> values;
    void reset() { values.clear(); }
};

struct EvalContext {
    VariableStore* variables = nullptr;
    int num_threads = 0;                       // 0 = hardware concurrency
    std::map<std::string, Attr> properties;    // device configuration visible to kernels
    void* user = nullptr;                      // plugin-specific (paged cache manager ...)
};

// Evaluate a whole model on host tensors with the reference kernels (the numerical oracle).
std::vector<Tensor> evaluate_model(const Model& m, const std::vector<Tensor>& inputs, EvalContext& ctx,
                                   std::vector<std::pair<std::string, double>>* per_node_us = nullptr);
// Try to compute the value of an output from constants only (used by shape inference and folding).
bool try_constant_value(const Output& o, Tensor& out, int depth = 0);
bool get_constant_ints(const Output& o, std::vector<int64_t>& v);

}  // namespace ovc
