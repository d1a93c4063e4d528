#include "xml.hpp"

#include <algorithm>
#include <cstring>

#include "types.hpp"

namespace ovc {

XmlNode* XmlNode::append_child(const std::string& n) {
    children.emplace_back(new XmlNode());
    children.back()->name = n;
    children.back()->parent = this;
    return children.back().get();
}
XmlNode* XmlNode::prepend_child(const std::string& n) {
    children.emplace(children.begin(), new XmlNode());
    children.front()->name = n;
    children.front()->parent = this;
    return children.front().get();
}
void XmlNode::remove_child(XmlNode* c) {
    children.erase(std::remove_if(children.begin(), children.end(), [&](const std::unique_ptr<XmlNode>& p) { return p.get() == c; }),
                   children.end());
}
XmlNode* XmlNode::child(const std::string& n) const {
    for (auto& c : children) if (c->name == n) return c.get();
    return nullptr;
}
std::vector<XmlNode*> XmlNode::children_named(const std::string& n) const {
    std::vector<XmlNode*> v;
    for (auto& c : children) if (c->name == n) v.push_back(c.get());
    return v;
}
void XmlNode::set_attr(const std::string& k, const std::string& v) {
    for (auto& a : attrs) if (a.first == k) { a.second = v; return; }
    attrs.emplace_back(k, v);
}
const std::string* XmlNode::attr(const std::string& k) const {
    for (auto& a : attrs) if (a.first == k) return &a.second;
    return nullptr;
}
std::string XmlNode::attr_or(const std::string& k, const std::string& d) const {
    auto* p = attr(k);
    return p ? *p : d;
}
void XmlNode::remove_attr(const std::string& k) {
    attrs.erase(std::remove_if(attrs.begin(), attrs.end(), [&](const std::pair<std::string, std::string>& a) { return a.first == k; }), attrs.end());
}
void XmlNode::move_child_to_front(XmlNode* c) {
    for (size_t i = 0; i < children.size(); ++i) {
        if (children[i].get() == c) {
            auto p = std::move(children[i]);
            children.erase(children.begin() + (long)i);
            children.insert(children.begin(), std::move(p));
            return;
        }
    }
}
void XmlNode::move_child_after(XmlNode* c, XmlNode* after) {
    std::unique_ptr<XmlNode> p;
    for (size_t i = 0; i < children.size(); ++i) if (children[i].get() == c) { p = std::move(children[i]); children.erase(children.begin() + (long)i); break; }
    if (!p) return;
    for (size_t i = 0; i < children.size(); ++i) if (children[i].get() == after) { children.insert(children.begin() + (long)i + 1, std::move(p)); return; }
    children.push_back(std::move(p));
}

// ------------------------------------------------------------------------------------ writer
static void escape_into(std::string& out, const std::string& s, bool attribute) {
    for (unsigned char c : s) {
        switch (c) {
            case '&': out += "&amp;"; break;
            case '<': out += "&lt;"; break;
            case '>': out += "&gt;"; break;
            case '"': if (attribute) out += "&quot;"; else out.push_back('"'); break;
            default:
                if (c < 32 && (attribute ? c != '\t' : (c != '\n' && c != '\t' && c != '\r'))) {
                    out += "&#";
                    out.push_back(char('0' + c / 10));
                    out.push_back(char('0' + c % 10));
                    out.push_back(';');
                } else {
                    out.push_back((char)c);
                }
        }
    }
}

static void write_node(std::string& out, const XmlNode& n, int depth) {
    out.append((size_t)depth, '\t');
    out.push_back('<');
    out += n.name;
    for (auto& a : n.attrs) {
        out.push_back(' ');
        out += a.first;
        out += "=\"";
        escape_into(out, a.second, true);
        out.push_back('"');
    }
    if (n.children.empty() && n.text.empty()) {
        out += " />\n";
        return;
    }
    out.push_back('>');
    if (n.children.empty()) {
        escape_into(out, n.text, false);
    } else {
        out.push_back('\n');
        for (auto& c : n.children) write_node(out, *c, depth + 1);
        out.append((size_t)depth, '\t');
    }
    out += "</";
    out += n.name;
    out += ">\n";
}

std::string XmlDocument::to_string() const {
    std::string out = "<?xml version=\"1.0\"?>\n";
    if (root) write_node(out, *root, 0);
    return out;
}

// ------------------------------------------------------------------------------------ parser
namespace {
struct Parser {
    const std::string& s;
    size_t p = 0;
    explicit Parser(const std::string& t) : s(t) {}
    [[noreturn]] void fail(const std::string& m) const { throw Error("XML parse error at offset " + std::to_string(p) + ": " + m); }
    bool starts(const char* t) const { return s.compare(p, std::strlen(t), t) == 0; }
    void skip_ws() { while (p < s.size() && std::isspace((unsigned char)s[p])) ++p; }
    void skip_misc() {
        for (;;) {
            skip_ws();
            if (starts("<?")) { const size_t e = s.find("?>", p); if (e == std::string::npos) fail("unterminated declaration"); p = e + 2; }
            else if (starts("<!--")) { const size_t e = s.find("-->", p); if (e == std::string::npos) fail("unterminated comment"); p = e + 3; }
            else if (starts("<!DOCTYPE")) { const size_t e = s.find('>', p); if (e == std::string::npos) fail("unterminated doctype"); p = e + 1; }
            else break;
        }
    }
    std::string name() {
        const size_t b = p;
        while (p < s.size() && (std::isalnum((unsigned char)s[p]) || s[p] == '_' || s[p] == '-' || s[p] == '.' || s[p] == ':')) ++p;
        if (p == b) fail("expected a name");
        return s.substr(b, p - b);
    }
    std::string unescape(const std::string& t) const {
        if (t.find('&') == std::string::npos) return t;
        std::string o;
        for (size_t i = 0; i < t.size(); ++i) {
            if (t[i] != '&') { o.push_back(t[i]); continue; }
            const size_t e = t.find(';', i);
            if (e == std::string::npos) { o.push_back('&'); continue; }
            const std::string ent = t.substr(i + 1, e - i - 1);
            if (ent == "amp") o.push_back('&');
            else if (ent == "lt") o.push_back('<');
            else if (ent == "gt") o.push_back('>');
            else if (ent == "quot") o.push_back('"');
            else if (ent == "apos") o.push_back('\'');
            else if (!ent.empty() && ent[0] == '#') {
                unsigned long cp = ent.size() > 1 && (ent[1] == 'x' || ent[1] == 'X') ? std::strtoul(ent.c_str() + 2, nullptr, 16) : std::strtoul(ent.c_str() + 1, nullptr, 10);
                if (cp < 0x80) o.push_back((char)cp);
                else if (cp < 0x800) { o.push_back((char)(0xC0 | (cp >> 6))); o.push_back((char)(0x80 | (cp & 0x3F))); }
                else if (cp < 0x10000) { o.push_back((char)(0xE0 | (cp >> 12))); o.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); o.push_back((char)(0x80 | (cp & 0x3F))); }
                else { o.push_back((char)(0xF0 | (cp >> 18))); o.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); o.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); o.push_back((char)(0x80 | (cp & 0x3F))); }
            } else { o += t.substr(i, e - i + 1); }
            i = e;
        }
        return o;
    }
    std::unique_ptr<XmlNode> element(int depth) {
        if (depth > 256) fail("nesting too deep");
        if (p >= s.size() || s[p] != '<') fail("expected '<'");
        ++p;
        std::unique_ptr<XmlNode> n(new XmlNode());
        n->name = name();
        for (;;) {
            skip_ws();
            if (p >= s.size()) fail("unterminated tag");
            if (s[p] == '/') { if (p + 1 >= s.size() || s[p + 1] != '>') fail("expected '/>'"); p += 2; return n; }
            if (s[p] == '>') { ++p; break; }
            const std::string k = name();
            skip_ws();
            if (p >= s.size() || s[p] != '=') fail("expected '=' after attribute name");
            ++p;
            skip_ws();
            if (p >= s.size() || (s[p] != '"' && s[p] != '\'')) fail("expected a quoted attribute value");
            const char q = s[p++];
            const size_t e = s.find(q, p);
            if (e == std::string::npos) fail("unterminated attribute value");
            n->attrs.emplace_back(k, unescape(s.substr(p, e - p)));
            p = e + 1;
        }
        std::string text;
        for (;;) {
            if (p >= s.size()) fail("unterminated element <" + n->name + ">");
            if (s[p] != '<') { const size_t e = s.find('<', p); if (e == std::string::npos) fail("unterminated element"); text += s.substr(p, e - p); p = e; continue; }
            if (starts("</")) {
                p += 2;
                const std::string c = name();
                if (c != n->name) fail("mismatched closing tag </" + c + "> for <" + n->name + ">");
                skip_ws();
                if (p >= s.size() || s[p] != '>') fail("expected '>'");
                ++p;
                break;
            }
            if (starts("<!--")) { const size_t e = s.find("-->", p); if (e == std::string::npos) fail("unterminated comment"); p = e + 3; continue; }
            if (starts("<![CDATA[")) { const size_t e = s.find("]]>", p); if (e == std::string::npos) fail("unterminated CDATA"); text += s.substr(p + 9, e - p - 9); p = e + 3; continue; }
            if (starts("<?")) { const size_t e = s.find("?>", p); if (e == std::string::npos) fail("unterminated PI"); p = e + 2; continue; }
            auto c = element(depth + 1);
            c->parent = n.get();
            n->children.push_back(std::move(c));
        }
        if (n->children.empty()) n->text = unescape(text);
        return n;
    }
};
}  // namespace

XmlDocument XmlDocument::parse(const std::string& text) {
    Parser ps(text);
    ps.skip_misc();
    XmlDocument d;
    d.root = ps.element(0);
    return d;
}

}  // namespace ovc
