#include "pass.hpp"

#include <cstdlib>
#include <iostream>

namespace ovc {

// ------------------------------------------------------------------------------------ pattern builders
namespace pattern {
PatternPtr any_input(ValuePredicate pred) {
    auto p = std::make_shared<PatternNode>();
    p->kind = PatternNode::ANY;
    p->pred = std::move(pred);
    return p;
}
PatternPtr wrap_type(std::vector<std::string> types, std::vector<PatternPtr> inputs, ValuePredicate pred) {
    auto p = std::make_shared<PatternNode>();
    p->kind = PatternNode::TYPE;
    p->types = std::move(types);
    p->inputs = std::move(inputs);
    p->pred = std::move(pred);
    return p;
}
PatternPtr optional(std::vector<std::string> types, PatternPtr input, ValuePredicate pred) {
    return optional(std::move(types), std::vector<PatternPtr>{std::move(input)}, std::move(pred));
}
PatternPtr optional(std::vector<std::string> types, std::vector<PatternPtr> inputs, ValuePredicate pred) {
    auto p = std::make_shared<PatternNode>();
    p->kind = PatternNode::OPTIONAL;
    p->types = std::move(types);
    p->inputs = std::move(inputs);
    p->pred = std::move(pred);
    return p;
}
PatternPtr any_of(std::vector<PatternPtr> alternatives) {
    auto p = std::make_shared<PatternNode>();
    p->kind = PatternNode::OR;
    p->alternatives = std::move(alternatives);
    return p;
}
PatternPtr wrap_const(ValuePredicate pred) { return wrap_type({"Constant"}, {}, std::move(pred)); }

ValuePredicate consumers_count(size_t n) {
    return [n](const Output& o) { return o.node->outs[o.index].uses.size() == n; };
}
ValuePredicate has_static_rank() { return [](const Output& o) { return o.shape().rank_is_static(); }; }
ValuePredicate has_static_shape() { return [](const Output& o) { return o.shape().is_static(); }; }
ValuePredicate rank_equals(size_t r) { return [r](const Output& o) { return o.shape().rank_is_static() && o.shape().rank() == r; }; }
ValuePredicate type_matches_any(std::vector<ET> types) {
    return [types](const Output& o) { return std::find(types.begin(), types.end(), o.et()) != types.end(); };
}
ValuePredicate all_of(std::vector<ValuePredicate> preds) {
    return [preds](const Output& o) { for (auto& p : preds) if (p && !p(o)) return false; return true; };
}
}  // namespace pattern

// ------------------------------------------------------------------------------------ matcher
static bool type_accepts(const std::vector<std::string>& types, const Node& n) {
    for (auto& t : types) {
        const size_t c = t.find(':');
        if (c == std::string::npos) { if (t == n.type) return true; }
        else if (t.substr(0, c) == n.type && t.substr(c + 1) == n.version) return true;
    }
    return false;
}

Output Matcher::at(const PatternPtr& p) const {
    auto it = map_.find(p.get());
    OVC_CHECK(it != map_.end(), "pattern node '" << p->name << "' did not take part in the match");
    return it->second;
}

bool Matcher::match(const Output& value) {
    map_.clear();
    matched_.clear();
    root_value_ = value;
    return match_value(root_, value);
}

bool Matcher::match_inputs(const PatternPtr& p, const NodePtr& n) {
    if (p->inputs.empty()) return true;
    if (p->inputs.size() != n->num_inputs()) return false;
    auto try_order = [&](const std::vector<size_t>& order) {
        const auto saved_map = map_;
        const auto saved_nodes = matched_;
        for (size_t i = 0; i < order.size(); ++i) {
            if (!match_value(p->inputs[i], n->input(order[i]))) { map_ = saved_map; matched_ = saved_nodes; return false; }
        }
        return true;
    };
    std::vector<size_t> order(n->num_inputs());
    for (size_t i = 0; i < order.size(); ++i) order[i] = i;
    if (try_order(order)) return true;
    if (n->schema && n->schema->commutative && order.size() == 2) {
        std::swap(order[0], order[1]);
        if (try_order(order)) return true;
    }
    return false;
}

bool Matcher::match_value(const PatternPtr& p, const Output& v) {
    // a pattern node that is reachable twice must bind to the same value both times
    auto it = map_.find(p.get());
    if (it != map_.end()) return it->second == v;
    switch (p->kind) {
        case PatternNode::ANY:
            if (p->pred && !p->pred(v)) return false;
            map_[p.get()] = v;
            return true;
        case PatternNode::TYPE: {
            if (!type_accepts(p->types, *v.node)) return false;
            if (p->output_index >= 0 && (size_t)p->output_index != v.index) return false;
            if (p->pred && !p->pred(v)) return false;
            const auto saved_map = map_;
            const auto saved_nodes = matched_;
            map_[p.get()] = v;
            if (!match_inputs(p, v.node)) { map_ = saved_map; matched_ = saved_nodes; return false; }
            matched_.push_back(v.node);
            return true;
        }
        case PatternNode::OPTIONAL: {
            if (type_accepts(p->types, *v.node) && (!p->pred || p->pred(v))) {
                const auto saved_map = map_;
                const auto saved_nodes = matched_;
                map_[p.get()] = v;
                if (match_inputs(p, v.node)) { matched_.push_back(v.node); return true; }
                map_ = saved_map;
                matched_ = saved_nodes;
            }
            // the optional node is absent: its first input pattern must match the value itself
            if (p->inputs.empty()) return false;
            return match_value(p->inputs[0], v);
        }
        case PatternNode::OR: {
            for (auto& alt : p->alternatives) {
                const auto saved_map = map_;
                const auto saved_nodes = matched_;
                if (match_value(alt, v)) { map_[p.get()] = v; return true; }
                map_ = saved_map;
                matched_ = saved_nodes;
            }
            return false;
        }
    }
    return false;
}

// ------------------------------------------------------------------------------------ passes
bool MatcherPass::apply(const NodePtr& node) {
    for (size_t i = 0; i < node->num_outputs(); ++i) {
        if (matcher->match(Output(node, i))) {
            if (callback(*matcher)) return true;
        }
        if (matcher->root()->kind == PatternNode::TYPE && matcher->root()->output_index < 0) break;   // node-level pattern
    }
    return false;
}

bool GraphRewrite::run_on_model(const ModelPtr& m) {
    bool changed = false;
    // nodes created by a callback are visited too (they may enable further matches)
    std::unordered_set<Node*> seen;
    for (int round = 0; round < 8; ++round) {
        bool round_changed = false;
        auto order = m->ordered_ops();
        for (auto& n : order) {
            if (round > 0 && seen.count(n.get())) continue;
            seen.insert(n.get());
            // skip nodes that a previous callback detached from the graph
            if (!n->is_result() && n->type != "Assign") {
                bool used = false;
                for (auto& o : n->outs) if (!o.uses.empty()) used = true;
                if (!used) continue;
            }
            for (auto& mp : matchers) {
                if (!mp->enabled) continue;
                if (mp->apply(n)) { round_changed = true; break; }
            }
        }
        changed |= round_changed;
        if (!round_changed) break;
    }
    return changed;
}

void PassManager::add_matcher(std::shared_ptr<MatcherPass> p) {
    auto gr = std::make_shared<GraphRewrite>();
    gr->name = p->name;
    gr->add(std::move(p));
    passes_.push_back(gr);
}

bool PassManager::run(const ModelPtr& m) {
    bool changed = false;
    timings_.clear();
    const bool profile = std::getenv("OV_ENABLE_PROFILE_PASS") != nullptr;
    for (auto& p : passes_) {
        if (!p->enabled || disabled_.count(p->name)) continue;
        const auto t0 = std::chrono::steady_clock::now();
        const bool c = p->run_on_model(m);
        if (c && validate_after_each) m->validate();
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        timings_.push_back({p->name, ms, c});
        if (profile) std::cerr << "[pass] " << p->name << " " << ms << " ms" << (c ? " (changed)" : "") << "\n";
        changed |= c;
    }
    return changed;
}

}  // namespace ovc
