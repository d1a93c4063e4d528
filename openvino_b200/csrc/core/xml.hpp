// Minimal XML DOM with a writer whose output is byte-compatible with the formatting IR files use
// (declaration `<?xml version="1.0"?>`, one TAB per depth, attributes in insertion order, self-closing
// elements written as `<tag a="b" />`, text-only elements on one line, trailing newline) and a parser
// for the subset IR files need (elements, attributes, text, comments, the five named entities and
// numeric character references).
#pragma once
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace ovc {

struct XmlNode {
    std::string name;
    std::vector<std::pair<std::string, std::string>> attrs;
    std::vector<std::unique_ptr<XmlNode>> children;
    std::string text;   // PCDATA (only kept for elements without child elements)
    XmlNode* parent = nullptr;

    XmlNode* append_child(const std::string& n);
    XmlNode* prepend_child(const std::string& n);
    void remove_child(XmlNode* c);
    XmlNode* child(const std::string& n) const;
    std::vector<XmlNode*> children_named(const std::string& n) const;
    void set_attr(const std::string& k, const std::string& v);     // appends or overwrites
    const std::string* attr(const std::string& k) const;
    std::string attr_or(const std::string& k, const std::string& d) const;
    bool has_attr(const std::string& k) const { return attr(k) != nullptr; }
    void remove_attr(const std::string& k);
    void move_child_to_front(XmlNode* c);
    void move_child_after(XmlNode* c, XmlNode* after);
};

struct XmlDocument {
    std::unique_ptr<XmlNode> root;
    std::string to_string() const;
    static XmlDocument parse(const std::string& text);
};

}  // namespace ovc
