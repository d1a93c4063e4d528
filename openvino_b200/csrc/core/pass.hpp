// Pass infrastructure and declarative pattern matcher of the native graph compiler.
//
// Roles covered: ov::pass::{PassBase, ModelPass, MatcherPass, GraphRewrite, Manager, PassConfig}
// (src/core/include/openvino/pass/*.hpp, src/core/src/pass/manager.cpp:150-383) and the pattern
// language of src/core/src/pattern/ (wrap_type, any_input, optional, Or, predicates, commutative
// permutation matching, src/core/src/pattern/matcher.cpp:130-192).
#pragma once
#include <chrono>

#include "graph.hpp"

namespace ovc {

// ------------------------------------------------------------------------------------ patterns
struct PatternNode;
using PatternPtr = std::shared_ptr<PatternNode>;
using ValuePredicate = std::function<bool(const Output&)>;

struct PatternNode {
    enum Kind { ANY, TYPE, OR, OPTIONAL } kind = ANY;
    std::vector<std::string> types;        // TYPE / OPTIONAL: accepted op types ("Add" or "Add:opset1")
    std::vector<PatternPtr> inputs;        // TYPE / OPTIONAL: input patterns (empty = do not look at the inputs)
    std::vector<PatternPtr> alternatives;  // OR
    ValuePredicate pred;
    std::string name;                      // optional label for debugging
    int output_index = -1;                 // match only this output of a multi-output node (-1: any)
};

namespace pattern {
PatternPtr any_input(ValuePredicate pred = nullptr);
PatternPtr wrap_type(std::vector<std::string> types, std::vector<PatternPtr> inputs = {}, ValuePredicate pred = nullptr);
PatternPtr optional(std::vector<std::string> types, PatternPtr input, ValuePredicate pred = nullptr);
PatternPtr optional(std::vector<std::string> types, std::vector<PatternPtr> inputs, ValuePredicate pred = nullptr);
PatternPtr any_of(std::vector<PatternPtr> alternatives);
PatternPtr wrap_const(ValuePredicate pred = nullptr);
// predicates
ValuePredicate consumers_count(size_t n);
ValuePredicate has_static_rank();
ValuePredicate has_static_shape();
ValuePredicate rank_equals(size_t r);
ValuePredicate type_matches_any(std::vector<ET> types);
ValuePredicate all_of(std::vector<ValuePredicate> preds);
}  // namespace pattern

class Matcher {
public:
    explicit Matcher(PatternPtr root, std::string name = "") : root_(std::move(root)), name_(std::move(name)) {}
    bool match(const Output& value);
    const std::map<const PatternNode*, Output>& pattern_map() const { return map_; }
    bool has(const PatternPtr& p) const { return map_.count(p.get()) > 0; }
    Output at(const PatternPtr& p) const;
    NodePtr node(const PatternPtr& p) const { return at(p).node; }
    Output match_value() const { return root_value_; }
    NodePtr match_root() const { return root_value_.node; }
    std::vector<NodePtr> matched_nodes() const { return matched_; }
    const std::string& name() const { return name_; }
    PatternPtr root() const { return root_; }
private:
    bool match_value(const PatternPtr& p, const Output& v);
    bool match_inputs(const PatternPtr& p, const NodePtr& n);
    PatternPtr root_;
    std::string name_;
    Output root_value_;
    std::map<const PatternNode*, Output> map_;
    std::vector<NodePtr> matched_;
};

// ------------------------------------------------------------------------------------ passes
class PassBase {
public:
    virtual ~PassBase() = default;
    std::string name;
    bool enabled = true;
};

class ModelPass : public PassBase {
public:
    virtual bool run_on_model(const ModelPtr& m) = 0;
};

using MatcherCallback = std::function<bool(Matcher&)>;

class MatcherPass : public PassBase {
public:
    MatcherPass() = default;
    MatcherPass(std::string n, PatternPtr root, MatcherCallback cb) { name = std::move(n); matcher = std::make_shared<Matcher>(std::move(root), name); callback = std::move(cb); }
    std::shared_ptr<Matcher> matcher;
    MatcherCallback callback;
    bool apply(const NodePtr& node);   // try to match at every output of the node
};

class GraphRewrite : public ModelPass {
public:
    std::vector<std::shared_ptr<MatcherPass>> matchers;
    void add(std::shared_ptr<MatcherPass> m) { matchers.push_back(std::move(m)); }
    bool run_on_model(const ModelPtr& m) override;
};

// Wraps a callable as a ModelPass
class LambdaPass : public ModelPass {
public:
    LambdaPass(std::string n, std::function<bool(const ModelPtr&)> f) : fn(std::move(f)) { name = std::move(n); }
    std::function<bool(const ModelPtr&)> fn;
    bool run_on_model(const ModelPtr& m) override { return fn(m); }
};

struct PassTiming {
    std::string name;
    double ms;
    bool changed;
};

class PassManager {
public:
    void add(std::shared_ptr<ModelPass> p) { passes_.push_back(std::move(p)); }
    void add_matcher(std::shared_ptr<MatcherPass> p);   // wrapped into its own GraphRewrite
    void disable(const std::string& pass_name) { disabled_.insert(pass_name); }
    void enable(const std::string& pass_name) { disabled_.erase(pass_name); }
    bool run(const ModelPtr& m);
    bool validate_after_each = true;
    const std::vector<PassTiming>& timings() const { return timings_; }
private:
    std::vector<std::shared_ptr<ModelPass>> passes_;
    std::set<std::string> disabled_;
    std::vector<PassTiming> timings_;
};

// ------------------------------------------------------------------------------------ pass library
// Every factory returns a ready-to-run pass; the names are the reference's pass names.
std::shared_ptr<ModelPass> make_pass(const std::string& name, const AttrMap& options = {});
std::vector<std::string> available_passes();

// pipelines
void run_moc_transformations(const ModelPtr& m, bool constant_folding = true);
void run_llm_fusions(const ModelPtr& m);                              // RMS, RoPE, GLU, FC, compressed FC
bool sdpa_to_paged_attention(const ModelPtr& m, const AttrMap& options = {});
bool make_stateful(const ModelPtr& m, const std::vector<std::pair<std::string, std::string>>& param_result_names);
bool stateful_to_stateless(const ModelPtr& m);
bool compress_weights(const ModelPtr& m, const std::string& mode, int64_t group_size, double ratio, bool all_layers);
bool compress_model_to_f16(const ModelPtr& m);

}  // namespace ovc
