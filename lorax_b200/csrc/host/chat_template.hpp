// Chat templates rendered in the router: an interpreter for the part of Jinja2 that chat templates are written in, so that a chat
// request does not cost a round trip to a shard before it can be validated.  The reference router renders them with minijinja
// (router/src/infer.rs:40-147: `messages`, `bos_token`, `eos_token`, `add_generation_prompt`, `tools`, `raise_exception`); no
// template engine exists for C++ here.  Implemented: text, `{{ }}`, `{% if / elif / else %}`, `{% for [a, b] in ... [if ...] %}` with
// `loop`, `{% set %}` (names and namespace attributes), comments, whitespace control (`-`, and the `trim_blocks` / `lstrip_blocks`
// settings chat templates are rendered with), `{% generation %}` markers; expressions with literals, lists, dicts, attribute /
// item access, slices, calls, filters, tests, comparisons, `in`, boolean operators, arithmetic, `~` and `a if c else b`.
// Macros are callable (`{{ f(x) }}`).  Anything else (`call`, `filter` blocks, an unknown filter or test ...) makes `compile` or `render` throw `Unsupported`, and
// the router asks shard 0 (which runs Jinja2) for that template or request.
#pragma once
#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.hpp"
#include "unicode.hpp"

namespace lx {
namespace jinja {

struct TemplateError : std::runtime_error { using std::runtime_error::runtime_error; };      // raise_exception, type errors
struct Unsupported : std::runtime_error { using std::runtime_error::runtime_error; };        // outside the implemented subset

struct Val;
using List = std::vector<Val>;
using Dict = std::vector<std::pair<std::string, Val>>;

struct Val {
  enum Kind { Undefined, None, Bool, Int, Float, Str, ListK, DictK } kind = Undefined;
  bool b = false;
  long long i = 0;
  double f = 0;
  std::string s;
  std::shared_ptr<List> list;
  std::shared_ptr<Dict> dict;       // shared: a namespace() is mutated through every copy
  bool is_namespace = false;

  Val() = default;
  static Val none() { Val v; v.kind = None; return v; }
  static Val boolean(bool x) { Val v; v.kind = Bool; v.b = x; return v; }
  static Val integer(long long x) { Val v; v.kind = Int; v.i = x; return v; }
  static Val real(double x) { Val v; v.kind = Float; v.f = x; return v; }
  static Val str(std::string x) { Val v; v.kind = Str; v.s = std::move(x); return v; }
  static Val make_list(List l = {}) { Val v; v.kind = ListK; v.list = std::make_shared<List>(std::move(l)); return v; }
  static Val make_dict(Dict d = {}) { Val v; v.kind = DictK; v.dict = std::make_shared<Dict>(std::move(d)); return v; }

  bool is_number() const { return kind == Int || kind == Float || kind == Bool; }
  double num() const { return kind == Float ? f : kind == Bool ? (b ? 1.0 : 0.0) : (double)i; }
  bool truthy() const {
    switch (kind) {
      case Undefined: case None: return false;
      case Bool: return b;
      case Int: return i != 0;
      case Float: return f != 0;
      case Str: return !s.empty();
      case ListK: return !list->empty();
      case DictK: return !dict->empty();
    }
    return false;
  }
  const Val* find(const std::string& key) const {
    if (kind != DictK) return nullptr;
    for (auto& kv : *dict) if (kv.first == key) return &kv.second;
    return nullptr;
  }
  void set(const std::string& key, Val v) {
    for (auto& kv : *dict) if (kv.first == key) { kv.second = std::move(v); return; }
    dict->emplace_back(key, std::move(v));
  }
};

inline Val from_json(const json::Value& j) {
  switch (j.type()) {
    case json::Value::Null: return Val::none();
    case json::Value::Bool: return Val::boolean(j.as_bool());
    case json::Value::Number: {
      const double d = j.as_double();
      if (d == std::floor(d) && std::fabs(d) < 9e15 && j.dump().find_first_of(".eE") == std::string::npos) return Val::integer((long long)d);
      return Val::real(d);
    }
    case json::Value::String: return Val::str(j.as_string());
    case json::Value::Arr: { List l; for (auto& e : j.items()) l.push_back(from_json(e)); return Val::make_list(std::move(l)); }
    case json::Value::Obj: { Dict d; for (auto& kv : j.members()) d.emplace_back(kv.first, from_json(kv.second)); return Val::make_dict(std::move(d)); }
  }
  return Val();
}

inline std::string float_repr(double f) {
  if (f == std::floor(f) && std::fabs(f) < 1e16) { char buf[64]; std::snprintf(buf, sizeof buf, "%.1f", f); return buf; }
  char buf[64];
  for (int prec = 1; prec <= 17; ++prec) {
    std::snprintf(buf, sizeof buf, "%.*g", prec, f);
    if (std::strtod(buf, nullptr) == f) break;
  }
  return buf;
}
inline std::string py_repr(const Val& v);
// str(value), what `{{ value }}` prints
inline std::string to_text(const Val& v) {
  switch (v.kind) {
    case Val::Undefined: return "";
    case Val::None: return "None";
    case Val::Bool: return v.b ? "True" : "False";
    case Val::Int: return std::to_string(v.i);
    case Val::Float: return float_repr(v.f);
    case Val::Str: return v.s;
    default: return py_repr(v);
  }
}
inline std::string py_repr(const Val& v) {
  switch (v.kind) {
    case Val::Str: {
      const bool dq = v.s.find('\'') != std::string::npos && v.s.find('"') == std::string::npos;
      std::string o(1, dq ? '"' : '\'');
      for (char c : v.s) {
        if (c == '\\') o += "\\\\";
        else if (c == '\n') o += "\\n";
        else if (c == '\t') o += "\\t";
        else if (c == '\r') o += "\\r";
        else if (c == '\'' && !dq) o += "\\'";
        else o.push_back(c);
      }
      o.push_back(dq ? '"' : '\'');
      return o;
    }
    case Val::ListK: {
      std::string o = "[";
      for (size_t k = 0; k < v.list->size(); ++k) { if (k) o += ", "; o += py_repr((*v.list)[k]); }
      return o + "]";
    }
    case Val::DictK: {
      std::string o = "{";
      for (size_t k = 0; k < v.dict->size(); ++k) { if (k) o += ", "; o += py_repr(Val::str((*v.dict)[k].first)) + ": " + py_repr((*v.dict)[k].second); }
      return o + "}";
    }
    default: return to_text(v);
  }
}

// json.dumps the way Jinja2's `tojson` does it: keys sorted, ASCII only, and < > & ' written as \u escapes.
struct JsonStyle { bool sort_keys = true, html_safe = true, compact = false; };
inline void json_dump(const Val& v, std::string& o, int indent, int depth, const JsonStyle& st = JsonStyle()) {
  auto nl = [&](int d) { if (indent >= 0) { o.push_back('\n'); o.append((size_t)(indent * d), ' '); } };
  switch (v.kind) {
    case Val::Undefined: throw TemplateError("Undefined is not JSON serializable");
    case Val::None: o += "null"; return;
    case Val::Bool: o += v.b ? "true" : "false"; return;
    case Val::Int: o += std::to_string(v.i); return;
    case Val::Float: o += float_repr(v.f); return;
    case Val::Str: {
      o.push_back('"');
      for (uint32_t c : uni::from_utf8(v.s)) {
        char buf[16];
        if (c == '"') o += "\\\"";
        else if (c == '\\') o += "\\\\";
        else if (c == '\n') o += "\\n";
        else if (c == '\r') o += "\\r";
        else if (c == '\t') o += "\\t";
        else if (c == '\b') o += "\\b";
        else if (c == '\f') o += "\\f";
        else if (c < 0x20 || (st.html_safe && (c == '<' || c == '>' || c == '&' || c == '\'')) || (c >= 0x7F && c < 0x10000)) { std::snprintf(buf, sizeof buf, "\\u%04x", c); o += buf; }
        else if (c >= 0x10000) { const uint32_t x = c - 0x10000; std::snprintf(buf, sizeof buf, "\\u%04x\\u%04x", 0xD800 + (x >> 10), 0xDC00 + (x & 0x3FF)); o += buf; }
        else o.push_back((char)c);
      }
      o.push_back('"');
      return;
    }
    case Val::ListK: {
      if (v.list->empty()) { o += "[]"; return; }
      o.push_back('[');
      for (size_t k = 0; k < v.list->size(); ++k) {
        if (k) o += (indent >= 0 || st.compact) ? "," : ", ";
        nl(depth + 1);
        json_dump((*v.list)[k], o, indent, depth + 1, st);
      }
      nl(depth);
      o.push_back(']');
      return;
    }
    case Val::DictK: {
      if (v.dict->empty()) { o += "{}"; return; }
      std::vector<const std::pair<std::string, Val>*> items;
      for (auto& kv : *v.dict) items.push_back(&kv);
      if (st.sort_keys) std::stable_sort(items.begin(), items.end(), [](auto* a, auto* b) { return a->first < b->first; });
      o.push_back('{');
      for (size_t k = 0; k < items.size(); ++k) {
        if (k) o += (indent >= 0 || st.compact) ? "," : ", ";
        nl(depth + 1);
        json_dump(Val::str(items[k]->first), o, indent, depth + 1, st);
        o += st.compact ? ":" : ": ";
        json_dump(items[k]->second, o, indent, depth + 1, st);
      }
      nl(depth);
      o.push_back('}');
      return;
    }
  }
}

inline bool equal(const Val& a, const Val& b) {
  if (a.is_number() && b.is_number()) return a.num() == b.num();
  if (a.kind != b.kind) return false;
  switch (a.kind) {
    case Val::Undefined: case Val::None: return true;
    case Val::Str: return a.s == b.s;
    case Val::ListK:
      if (a.list->size() != b.list->size()) return false;
      for (size_t k = 0; k < a.list->size(); ++k) if (!equal((*a.list)[k], (*b.list)[k])) return false;
      return true;
    case Val::DictK:
      if (a.dict->size() != b.dict->size()) return false;
      for (auto& kv : *a.dict) { const Val* o = b.find(kv.first); if (!o || !equal(kv.second, *o)) return false; }
      return true;
    default: return false;
  }
}

// ------------------------------------------------------------------------------------------------ expressions
struct Context;
struct Expr {
  virtual ~Expr() = default;
  virtual Val eval(Context& c) const = 0;
};
using ExprP = std::unique_ptr<Expr>;

struct MacroDef;
struct Context {
  std::vector<std::map<std::string, Val>> scopes;
  std::map<std::string, const MacroDef*> macros;
  int depth = 0;
  Val lookup(const std::string& name) const {
    for (size_t k = scopes.size(); k-- > 0;) { auto it = scopes[k].find(name); if (it != scopes[k].end()) return it->second; }
    return Val();
  }
  void assign(const std::string& name, Val v) { scopes.back()[name] = std::move(v); }
};

struct Lit : Expr { Val v; explicit Lit(Val x) : v(std::move(x)) {} Val eval(Context&) const override { return v; } };
struct Name : Expr { std::string n; explicit Name(std::string x) : n(std::move(x)) {} Val eval(Context& c) const override { return c.lookup(n); } };
struct ListLit : Expr {
  std::vector<ExprP> items;
  Val eval(Context& c) const override { List l; for (auto& e : items) l.push_back(e->eval(c)); return Val::make_list(std::move(l)); }
};
struct DictLit : Expr {
  std::vector<std::pair<ExprP, ExprP>> items;
  Val eval(Context& c) const override {
    Val d = Val::make_dict();
    for (auto& kv : items) d.set(to_text(kv.first->eval(c)), kv.second->eval(c));
    return d;
  }
};

inline Val get_attr(const Val& o, const std::string& key) {
  if (o.kind == Val::DictK) { const Val* v = o.find(key); return v ? *v : Val(); }
  if (o.kind == Val::Undefined) throw TemplateError("'" + key + "' is looked up on an undefined value");
  return Val();
}
inline Val get_item(const Val& o, const Val& idx) {
  if (o.kind == Val::DictK) return get_attr(o, to_text(idx));
  if (o.kind == Val::ListK || o.kind == Val::Str) {
    if (idx.kind != Val::Int) return Val();
    if (o.kind == Val::ListK) {
      long long k = idx.i < 0 ? idx.i + (long long)o.list->size() : idx.i;
      return (k >= 0 && k < (long long)o.list->size()) ? (*o.list)[(size_t)k] : Val();
    }
    const uni::Text t = uni::from_utf8(o.s);
    long long k = idx.i < 0 ? idx.i + (long long)t.size() : idx.i;
    return (k >= 0 && k < (long long)t.size()) ? Val::str(uni::to_utf8(&t[(size_t)k], 1)) : Val();
  }
  if (o.kind == Val::Undefined) throw TemplateError("an undefined value is indexed");
  return Val();
}

struct Attr : Expr {
  ExprP obj; std::string key;
  Val eval(Context& c) const override { return get_attr(obj->eval(c), key); }
};
struct Item : Expr {
  ExprP obj, idx;
  Val eval(Context& c) const override { return get_item(obj->eval(c), idx->eval(c)); }
};
struct Slice : Expr {
  ExprP obj, lo, hi;
  Val eval(Context& c) const override {
    const Val o = obj->eval(c);
    const bool is_list = o.kind == Val::ListK;
    if (!is_list && o.kind != Val::Str) throw TemplateError("only lists and strings are sliced");
    const uni::Text t = is_list ? uni::Text() : uni::from_utf8(o.s);
    const long long n = is_list ? (long long)o.list->size() : (long long)t.size();
    auto clamp = [&](const ExprP& e, long long dflt) {
      if (!e) return dflt;
      const Val v = e->eval(c);
      if (v.kind == Val::None) return dflt;
      if (v.kind != Val::Int) throw TemplateError("slice bounds are integers");
      long long k = v.i < 0 ? v.i + n : v.i;
      return std::max(0ll, std::min(n, k));
    };
    const long long a = clamp(lo, 0), b = clamp(hi, n);
    if (is_list) return Val::make_list(a < b ? List(o.list->begin() + a, o.list->begin() + b) : List());
    return Val::str(a < b ? uni::to_utf8(&t[(size_t)a], (size_t)(b - a)) : std::string());
  }
};

inline std::string strip_text(const std::string& s, bool left, bool right, const std::string& chars = "") {
  uni::Text t = uni::from_utf8(s);
  const uni::Text cs = uni::from_utf8(chars);
  auto drop = [&](uint32_t ch) { return cs.empty() ? uni::is_space(ch) : std::find(cs.begin(), cs.end(), ch) != cs.end(); };
  size_t b = 0, e = t.size();
  if (left) while (b < e && drop(t[b])) ++b;
  if (right) while (e > b && drop(t[e - 1])) --e;
  return uni::to_utf8(t.data() + b, e - b);
}
inline std::string map_case(const std::string& s, int mode) {       // 0 lower, 1 upper, 2 capitalize, 3 title
  std::string o = s;
  bool start = true;
  for (size_t k = 0; k < o.size(); ++k) {
    unsigned char ch = (unsigned char)o[k];
    if (ch >= 0x80) { if (mode < 2) throw Unsupported("case mapping of non-ASCII text"); start = false; continue; }
    const bool alpha = (ch | 32) >= 'a' && (ch | 32) <= 'z';
    const bool up = mode == 1 || (mode == 2 && k == 0) || (mode == 3 && start);
    if (alpha) o[k] = (char)(up ? (ch & ~32) : (ch | 32));
    start = !alpha && !(ch >= '0' && ch <= '9') && ch != '\'';
  }
  return o;
}
inline std::string replace_all(std::string s, const std::string& a, const std::string& b) {
  if (a.empty()) return s;
  for (size_t p = 0; (p = s.find(a, p)) != std::string::npos; p += b.size()) s.replace(p, a.size(), b);
  return s;
}

struct Arg { std::string name; ExprP value; };

inline bool apply_test(const std::string& t, const Val& x, const std::vector<Val>& args);
inline Val get_attr(const Val& o, const std::string& key);
// "a.b.c" looked up step by step (the attribute arguments of selectattr / map)
inline Val get_path(const Val& o, const std::string& path) {
  Val cur = o;
  size_t p = 0;
  while (true) {
    const size_t q = path.find('.', p);
    const std::string key = path.substr(p, q == std::string::npos ? std::string::npos : q - p);
    if (cur.kind == Val::ListK && !key.empty() && std::isdigit((unsigned char)key[0])) {
      const size_t k = (size_t)std::strtoul(key.c_str(), nullptr, 10);
      cur = k < cur.list->size() ? (*cur.list)[k] : Val();
    } else {
      cur = cur.kind == Val::Undefined ? Val() : get_attr(cur, key);
    }
    if (q == std::string::npos) return cur;
    p = q + 1;
  }
}

inline Val apply_filter(const std::string& f, const Val& x, const std::vector<std::pair<std::string, Val>>& args) {
  auto arg = [&](size_t pos, const char* name) -> const Val* {
    for (auto& a : args) if (a.first == name) return &a.second;
    size_t k = 0;
    for (auto& a : args) if (a.first.empty()) { if (k == pos) return &a.second; ++k; }
    return nullptr;
  };
  if (f == "trim" || f == "strip") { const Val* cs = arg(0, "chars"); return Val::str(strip_text(to_text(x), true, true, cs ? to_text(*cs) : "")); }
  if (f == "length" || f == "count") {
    if (x.kind == Val::Str) return Val::integer((long long)uni::from_utf8(x.s).size());
    if (x.kind == Val::ListK) return Val::integer((long long)x.list->size());
    if (x.kind == Val::DictK) return Val::integer((long long)x.dict->size());
    throw TemplateError("object has no length");
  }
  if (f == "upper") return Val::str(map_case(to_text(x), 1));
  if (f == "lower") return Val::str(map_case(to_text(x), 0));
  if (f == "capitalize") return Val::str(map_case(map_case(to_text(x), 0), 2));
  if (f == "title") return Val::str(map_case(map_case(to_text(x), 0), 3));
  if (f == "string") return Val::str(to_text(x));
  if (f == "safe") return x;
  if (f == "int") {
    if (x.kind == Val::Int) return x;
    if (x.is_number()) return Val::integer((long long)x.num());
    if (x.kind == Val::Str) { char* end = nullptr; const long long v = std::strtoll(x.s.c_str(), &end, 10); return Val::integer(end && *end == 0 && !x.s.empty() ? v : 0); }
    return Val::integer(0);
  }
  if (f == "float") {
    if (x.is_number()) return Val::real(x.num());
    if (x.kind == Val::Str) { char* end = nullptr; const double v = std::strtod(x.s.c_str(), &end); return Val::real(end && *end == 0 && !x.s.empty() ? v : 0.0); }
    return Val::real(0.0);
  }
  if (f == "default" || f == "d") {
    const Val* d = arg(0, "default_value");
    const Val* boolean = arg(1, "boolean");
    const bool use = x.kind == Val::Undefined || (boolean && boolean->truthy() && !x.truthy());
    return use ? (d ? *d : Val::str("")) : x;
  }
  if (f == "first" || f == "last") {
    if (x.kind == Val::ListK) return x.list->empty() ? Val() : (f == "first" ? x.list->front() : x.list->back());
    if (x.kind == Val::Str) { const uni::Text t = uni::from_utf8(x.s); return t.empty() ? Val() : Val::str(uni::to_utf8(f == "first" ? &t.front() : &t.back(), 1)); }
    throw TemplateError(f + " of something that is no sequence");
  }
  if (f == "join") {
    const Val* sep = arg(0, "d");
    if (arg(1, "attribute")) throw Unsupported("join with an attribute");
    if (x.kind != Val::ListK) throw TemplateError("join of something that is no list");
    std::string o;
    for (size_t k = 0; k < x.list->size(); ++k) { if (k && sep) o += to_text(*sep); o += to_text((*x.list)[k]); }
    return Val::str(o);
  }
  if (f == "list") {
    if (x.kind == Val::ListK) return x;
    if (x.kind == Val::Str) { List l; for (uint32_t ch : uni::from_utf8(x.s)) l.push_back(Val::str(uni::to_utf8(&ch, 1))); return Val::make_list(std::move(l)); }
    if (x.kind == Val::DictK) { List l; for (auto& kv : *x.dict) l.push_back(Val::str(kv.first)); return Val::make_list(std::move(l)); }
    throw TemplateError("list of something that cannot be iterated");
  }
  if (f == "items" || f == "dictitems") {
    if (x.kind == Val::Undefined) return Val::make_list();
    if (x.kind != Val::DictK) throw TemplateError("items of something that is no mapping");
    List l;
    for (auto& kv : *x.dict) l.push_back(Val::make_list({Val::str(kv.first), kv.second}));
    return Val::make_list(std::move(l));
  }
  if (f == "replace") {
    const Val *a = arg(0, "old"), *b = arg(1, "new");
    if (!a || !b || arg(2, "count")) throw Unsupported("replace with a count");
    return Val::str(replace_all(to_text(x), to_text(*a), to_text(*b)));
  }
  if (f == "tojson") {
    const Val* ind = arg(0, "indent");
    std::string o;
    json_dump(x, o, ind && ind->kind == Val::Int ? (int)ind->i : -1, 0);
    return Val::str(o);
  }
  if (f == "reverse") {
    if (x.kind == Val::ListK) return Val::make_list(List(x.list->rbegin(), x.list->rend()));
    throw Unsupported("reverse of something that is no list");
  }
  if (f == "selectattr" || f == "rejectattr" || f == "select" || f == "reject") {
    if (x.kind != Val::ListK) throw TemplateError(f + " of something that is no list");
    const bool by_attr = f == "selectattr" || f == "rejectattr";
    const bool keep_if = f == "selectattr" || f == "select";
    std::vector<Val> pos;
    for (auto& a : args) if (a.first.empty()) pos.push_back(a.second);
    if (by_attr && pos.empty()) throw TemplateError(f + " needs an attribute");
    const size_t t0 = by_attr ? 1 : 0;
    List out;
    for (auto& item : *x.list) {
      const Val v = by_attr ? get_path(item, to_text(pos[0])) : item;
      bool hit;
      if (pos.size() > t0) hit = apply_test(to_text(pos[t0]), v, std::vector<Val>(pos.begin() + (long)t0 + 1, pos.end()));
      else hit = v.truthy();
      if (hit == keep_if) out.push_back(item);
    }
    return Val::make_list(std::move(out));
  }
  if (f == "map") {
    if (x.kind != Val::ListK) throw TemplateError("map of something that is no list");
    const Val* attribute = nullptr;
    const Val* dflt = nullptr;
    std::vector<std::pair<std::string, Val>> rest;
    const Val* fname = nullptr;
    for (auto& a : args) {
      if (a.first == "attribute") attribute = &a.second;
      else if (a.first == "default") dflt = &a.second;
      else if (a.first.empty() && !fname && !attribute) fname = &a.second;
      else rest.push_back(a);
    }
    List out;
    for (auto& item : *x.list) {
      if (attribute) { Val v = get_path(item, to_text(*attribute)); out.push_back(v.kind == Val::Undefined && dflt ? *dflt : v); }
      else if (fname) out.push_back(apply_filter(to_text(*fname), item, rest));
      else throw TemplateError("map needs a filter or an attribute");
    }
    return Val::make_list(std::move(out));
  }
  if (f == "sum") {
    if (x.kind != Val::ListK) throw TemplateError("sum of something that is no list");
    bool fl = false;
    double acc = 0;
    for (auto& e : *x.list) { if (!e.is_number()) throw TemplateError("sum of something that is no number"); fl = fl || e.kind == Val::Float; acc += e.num(); }
    return fl ? Val::real(acc) : Val::integer((long long)acc);
  }
  if (f == "min" || f == "max") {
    if (x.kind != Val::ListK || x.list->empty()) return Val();
    const Val* best = &(*x.list)[0];
    for (auto& e : *x.list) {
      bool less;
      if (e.is_number() && best->is_number()) less = e.num() < best->num();
      else if (e.kind == Val::Str && best->kind == Val::Str) less = e.s < best->s;
      else throw TemplateError("values of these types are not ordered");
      if (less == (f == "min") && !equal(e, *best)) best = &e;
    }
    return *best;
  }
  if (f == "dictsort") {
    if (x.kind != Val::DictK) throw TemplateError("dictsort of something that is no mapping");
    if (!args.empty()) throw Unsupported("dictsort with arguments");
    std::vector<std::pair<std::string, Val>> items(x.dict->begin(), x.dict->end());
    auto lower = [](std::string v) { for (auto& ch : v) if (ch >= 'A' && ch <= 'Z') ch = (char)(ch + 32); return v; };
    std::stable_sort(items.begin(), items.end(), [&](auto& a, auto& b) { return lower(a.first) < lower(b.first); });
    List l;
    for (auto& kv : items) l.push_back(Val::make_list({Val::str(kv.first), kv.second}));
    return Val::make_list(std::move(l));
  }
  if (f == "unique") {
    if (x.kind != Val::ListK) throw TemplateError("unique of something that is no list");
    List out;
    for (auto& e : *x.list) { bool seen = false; for (auto& o : out) if (equal(o, e)) { seen = true; break; } if (!seen) out.push_back(e); }
    return Val::make_list(std::move(out));
  }
  if (f == "abs" && x.is_number()) return x.kind == Val::Float ? Val::real(std::fabs(x.f)) : Val::integer(std::llabs((long long)x.num()));
  if (f == "indent") {
    const Val* w = nullptr;
    bool first = false;
    size_t k = 0;
    for (auto& a : args) {
      if (a.first == "width" || (a.first.empty() && k == 0)) w = &a.second;
      else if (a.first == "first" || (a.first.empty() && k == 1)) first = a.second.truthy();
      else throw Unsupported("indent with this argument");
      if (a.first.empty()) ++k;
    }
    const std::string pad = w && w->kind == Val::Str ? w->s : std::string((size_t)(w && w->kind == Val::Int ? w->i : 4), ' ');
    const std::string src = to_text(x);
    std::string o;
    size_t p = 0;
    bool line0 = true;
    while (p <= src.size()) {
      const size_t q = src.find('\n', p);
      const std::string line = src.substr(p, q == std::string::npos ? std::string::npos : q - p);
      if (!line.empty() && (!line0 || first)) o += pad;
      o += line;
      if (q == std::string::npos) break;
      o.push_back('\n');
      p = q + 1;
      line0 = false;
    }
    return Val::str(o);
  }
  throw Unsupported("filter " + f);
}

inline bool apply_test(const std::string& t, const Val& x, const std::vector<Val>& args) {
  if (t == "defined") return x.kind != Val::Undefined;
  if (t == "undefined") return x.kind == Val::Undefined;
  if (t == "none") return x.kind == Val::None;
  if (t == "string") return x.kind == Val::Str;
  if (t == "mapping") return x.kind == Val::DictK;
  if (t == "iterable") return x.kind == Val::Str || x.kind == Val::ListK || x.kind == Val::DictK;
  if (t == "sequence") return x.kind == Val::Str || x.kind == Val::ListK || x.kind == Val::DictK;
  if (t == "number") return x.kind == Val::Int || x.kind == Val::Float || x.kind == Val::Bool;
  if (t == "integer") return x.kind == Val::Int;
  if (t == "float") return x.kind == Val::Float;
  if (t == "boolean") return x.kind == Val::Bool;
  if (t == "true") return x.kind == Val::Bool && x.b;
  if (t == "false") return x.kind == Val::Bool && !x.b;
  if (t == "odd") return x.kind == Val::Int && (x.i % 2) != 0;
  if (t == "even") return x.kind == Val::Int && (x.i % 2) == 0;
  if ((t == "equalto" || t == "eq" || t == "==") && args.size() == 1) return equal(x, args[0]);
  if ((t == "ne" || t == "!=") && args.size() == 1) return !equal(x, args[0]);
  if (t == "in" && args.size() == 1) {
    const Val& h = args[0];
    if (h.kind == Val::ListK) { for (auto& e : *h.list) if (equal(e, x)) return true; return false; }
    if (h.kind == Val::Str) return x.kind == Val::Str && h.s.find(x.s) != std::string::npos;
    if (h.kind == Val::DictK) return h.find(to_text(x)) != nullptr;
    return false;
  }
  throw Unsupported("test " + t);
}

struct Filter : Expr {
  ExprP obj; std::string name; std::vector<Arg> args;
  Val eval(Context& c) const override {
    std::vector<std::pair<std::string, Val>> av;
    for (auto& a : args) av.emplace_back(a.name, a.value->eval(c));
    return apply_filter(name, obj->eval(c), av);
  }
};
struct Test : Expr {
  ExprP obj; std::string name; std::vector<ExprP> args; bool negated = false;
  Val eval(Context& c) const override {
    std::vector<Val> av;
    for (auto& a : args) av.push_back(a->eval(c));
    return Val::boolean(apply_test(name, obj->eval(c), av) != negated);
  }
};

Val call_macro(const MacroDef& m, const std::vector<std::pair<std::string, Val>>& args, Context& c);
// Calls: macros, global functions, and the methods of strings / dicts / lists that templates use.
struct Call : Expr {
  ExprP callee;                    // Name (function) or Attr (method)
  std::vector<Arg> args;
  Val eval(Context& c) const override {
    std::vector<std::pair<std::string, Val>> av;
    for (auto& a : args) av.emplace_back(a.name, a.value->eval(c));
    auto pos = [&](size_t k) -> const Val* { size_t n = 0; for (auto& a : av) if (a.first.empty()) { if (n == k) return &a.second; ++n; } return nullptr; };
    if (auto* nm = dynamic_cast<const Name*>(callee.get())) {
      const std::string& fn = nm->n;
      auto mi = c.macros.find(fn);
      if (mi != c.macros.end()) return call_macro(*mi->second, av, c);
      if (fn == "raise_exception") throw TemplateError(pos(0) ? to_text(*pos(0)) : "template error");
      if (fn == "namespace") { Val ns = Val::make_dict(); ns.is_namespace = true; for (auto& a : av) if (!a.first.empty()) ns.set(a.first, a.second); return ns; }
      if (fn == "dict") { Val d = Val::make_dict(); for (auto& a : av) if (!a.first.empty()) d.set(a.first, a.second); return d; }
      if (fn == "range") {
        long long lo = 0, hi = 0, st = 1;
        if (pos(1)) { lo = pos(0)->i; hi = pos(1)->i; if (pos(2)) st = pos(2)->i; } else if (pos(0)) hi = pos(0)->i;
        if (st == 0 || (hi - lo) / st > 100000) throw TemplateError("range too large");
        List l;
        for (long long k = lo; st > 0 ? k < hi : k > hi; k += st) l.push_back(Val::integer(k));
        return Val::make_list(std::move(l));
      }
      if (fn == "strftime_now") {
        char buf[256];
        const std::time_t now = std::time(nullptr);
        std::tm tmv;
        localtime_r(&now, &tmv);
        const size_t n = std::strftime(buf, sizeof buf, pos(0) ? to_text(*pos(0)).c_str() : "%Y-%m-%d", &tmv);
        return Val::str(std::string(buf, n));
      }
      throw Unsupported("function " + fn);
    }
    auto* at = dynamic_cast<const Attr*>(callee.get());
    if (!at) throw Unsupported("call of an expression");
    const Val o = at->obj->eval(c);
    const std::string& m = at->key;
    if (o.kind == Val::Str) {
      if (m == "strip" || m == "lstrip" || m == "rstrip") return Val::str(strip_text(o.s, m != "rstrip", m != "lstrip", pos(0) ? to_text(*pos(0)) : ""));
      if (m == "upper") return Val::str(map_case(o.s, 1));
      if (m == "lower") return Val::str(map_case(o.s, 0));
      if (m == "title") return Val::str(map_case(map_case(o.s, 0), 3));
      if (m == "capitalize") return Val::str(map_case(map_case(o.s, 0), 2));
      if (m == "startswith" && pos(0)) return Val::boolean(o.s.rfind(to_text(*pos(0)), 0) == 0);
      if (m == "endswith" && pos(0)) { const std::string t = to_text(*pos(0)); return Val::boolean(o.s.size() >= t.size() && o.s.compare(o.s.size() - t.size(), t.size(), t) == 0); }
      if (m == "replace" && pos(0) && pos(1) && !pos(2)) return Val::str(replace_all(o.s, to_text(*pos(0)), to_text(*pos(1))));
      if (m == "split" && !pos(1)) {
        List l;
        if (!pos(0) || pos(0)->kind == Val::None) {
          std::string w;
          for (uint32_t ch : uni::from_utf8(o.s)) { if (uni::is_space(ch)) { if (!w.empty()) l.push_back(Val::str(w)); w.clear(); } else uni::append_utf8(w, ch); }
          if (!w.empty()) l.push_back(Val::str(w));
        } else {
          const std::string sep = to_text(*pos(0));
          if (sep.empty()) throw TemplateError("empty separator");
          size_t p = 0, q;
          while ((q = o.s.find(sep, p)) != std::string::npos) { l.push_back(Val::str(o.s.substr(p, q - p))); p = q + sep.size(); }
          l.push_back(Val::str(o.s.substr(p)));
        }
        return Val::make_list(std::move(l));
      }
      throw Unsupported("string method " + m);
    }
    if (o.kind == Val::DictK) {
      if (m == "items") { List l; for (auto& kv : *o.dict) l.push_back(Val::make_list({Val::str(kv.first), kv.second})); return Val::make_list(std::move(l)); }
      if (m == "keys") { List l; for (auto& kv : *o.dict) l.push_back(Val::str(kv.first)); return Val::make_list(std::move(l)); }
      if (m == "values") { List l; for (auto& kv : *o.dict) l.push_back(kv.second); return Val::make_list(std::move(l)); }
      if (m == "cycle" && o.find("index0") && o.find("revindex0") && pos(0)) {       // loop.cycle('a', 'b', ...)
        size_t n = 0;
        while (pos(n)) ++n;
        return *pos((size_t)o.find("index0")->i % n);
      }
      if (m == "get" && pos(0)) { const Val* v = o.find(to_text(*pos(0))); return v ? *v : (pos(1) ? *pos(1) : Val::none()); }
      throw Unsupported("mapping method " + m);
    }
    if (o.kind == Val::ListK && m == "append" && pos(0)) { o.list->push_back(*pos(0)); return Val::none(); }
    if (o.kind == Val::Undefined) throw TemplateError("'" + m + "' is called on an undefined value");
    throw Unsupported("method " + m);
  }
};

struct Unary : Expr {
  char op; ExprP x;       // '!' not, '-' minus, '+'
  Val eval(Context& c) const override {
    const Val v = x->eval(c);
    if (op == '!') return Val::boolean(!v.truthy());
    if (!v.is_number()) throw TemplateError("sign of something that is no number");
    if (v.kind == Val::Float) return Val::real(op == '-' ? -v.f : v.f);
    return Val::integer(op == '-' ? -(long long)v.num() : (long long)v.num());
  }
};
struct Binary : Expr {
  std::string op; ExprP a, b;
  Val eval(Context& c) const override {
    if (op == "and") { const Val x = a->eval(c); return x.truthy() ? b->eval(c) : x; }
    if (op == "or") { const Val x = a->eval(c); return x.truthy() ? x : b->eval(c); }
    const Val x = a->eval(c), y = b->eval(c);
    if (op == "==") return Val::boolean(equal(x, y));
    if (op == "!=") return Val::boolean(!equal(x, y));
    if (op == "in" || op == "not in") return Val::boolean(apply_test("in", x, {y}) == (op == "in"));
    if (op == "~") return Val::str(to_text(x) + to_text(y));
    if (op == "<" || op == ">" || op == "<=" || op == ">=") {
      int cmp;
      if (x.is_number() && y.is_number()) cmp = x.num() < y.num() ? -1 : x.num() > y.num() ? 1 : 0;
      else if (x.kind == Val::Str && y.kind == Val::Str) cmp = x.s.compare(y.s) < 0 ? -1 : x.s == y.s ? 0 : 1;
      else throw TemplateError("values of these types are not ordered");
      return Val::boolean(op == "<" ? cmp < 0 : op == ">" ? cmp > 0 : op == "<=" ? cmp <= 0 : cmp >= 0);
    }
    if (op == "+") {
      if (x.kind == Val::Str && y.kind == Val::Str) return Val::str(x.s + y.s);
      if (x.kind == Val::ListK && y.kind == Val::ListK) { List l = *x.list; l.insert(l.end(), y.list->begin(), y.list->end()); return Val::make_list(std::move(l)); }
      if (x.is_number() && y.is_number()) {
        if (x.kind == Val::Float || y.kind == Val::Float) return Val::real(x.num() + y.num());
        return Val::integer((long long)x.num() + (long long)y.num());
      }
      throw TemplateError(std::string("can only concatenate str (not \"") + (y.kind == Val::Str ? "str" : y.kind == Val::None ? "NoneType" : y.kind == Val::Undefined ? "Undefined" : "object") + "\") to str");
    }
    if (op == "*" && x.kind == Val::Str && y.kind == Val::Int) { std::string o; for (long long k = 0; k < y.i && o.size() < (1u << 20); ++k) o += x.s; return Val::str(o); }
    if (op == "%" && x.kind == Val::Str) throw Unsupported("string formatting with %");
    if (!x.is_number() || !y.is_number()) throw TemplateError("arithmetic on something that is no number");
    const bool fl = x.kind == Val::Float || y.kind == Val::Float;
    if (op == "-") return fl ? Val::real(x.num() - y.num()) : Val::integer((long long)x.num() - (long long)y.num());
    if (op == "*") return fl ? Val::real(x.num() * y.num()) : Val::integer((long long)x.num() * (long long)y.num());
    if (y.num() == 0) throw TemplateError("division by zero");
    if (op == "/") return Val::real(x.num() / y.num());
    if (op == "//") return fl ? Val::real(std::floor(x.num() / y.num())) : Val::integer((long long)std::floor((double)(long long)x.num() / (double)(long long)y.num()));
    if (op == "%") {
      if (fl) { const double r = std::fmod(x.num(), y.num()); return Val::real(r != 0 && ((r < 0) != (y.num() < 0)) ? r + y.num() : r); }
      const long long p = (long long)x.num(), q = (long long)y.num();
      long long r = p % q;
      if (r != 0 && ((r < 0) != (q < 0))) r += q;
      return Val::integer(r);
    }
    throw Unsupported("operator " + op);
  }
};
struct Cond : Expr {
  ExprP then, test, otherwise;
  Val eval(Context& c) const override { return test->eval(c).truthy() ? then->eval(c) : (otherwise ? otherwise->eval(c) : Val()); }
};

// ------------------------------------------------------------------------------------------------ statements
struct Node {
  virtual ~Node() = default;
  virtual void render(Context& c, std::string& out) const = 0;
};
using NodeP = std::unique_ptr<Node>;
using Body = std::vector<NodeP>;
inline void render_body(const Body& b, Context& c, std::string& out) { for (auto& n : b) n->render(c, out); }

struct TextNode : Node { std::string text; void render(Context&, std::string& out) const override { out += text; } };
struct OutputNode : Node { ExprP e; void render(Context& c, std::string& out) const override { out += to_text(e->eval(c)); } };
struct IfNode : Node {
  std::vector<std::pair<ExprP, Body>> branches;      // a null condition is the else branch
  void render(Context& c, std::string& out) const override {
    for (auto& br : branches) if (!br.first || br.first->eval(c).truthy()) { render_body(br.second, c, out); return; }
  }
};
struct SetNode : Node {
  std::string name, attr;       // attr: `set ns.attr = ...`
  ExprP value;                  // null: `{% set x %}...{% endset %}`, the rendered body is the value
  Body block;
  void render(Context& c, std::string&) const override {
    Val v;
    if (value) v = value->eval(c);
    else { std::string text; render_body(block, c, text); v = Val::str(text); }
    if (attr.empty()) { c.assign(name, std::move(v)); return; }
    Val ns = c.lookup(name);
    if (ns.kind != Val::DictK || !ns.is_namespace) throw TemplateError("cannot assign attribute on non-namespace object");
    ns.set(attr, std::move(v));
  }
};
struct LoopControl { bool is_break; };          // thrown by `break` / `continue`, caught by the enclosing for
struct LoopControlNode : Node {
  bool is_break = false;
  void render(Context&, std::string&) const override { throw LoopControl{is_break}; }
};
struct ForNode : Node {
  std::vector<std::string> vars;
  ExprP iterable, filter;
  Body body, otherwise;
  void render(Context& c, std::string& out) const override {
    const Val it = iterable->eval(c);
    List items;
    if (it.kind == Val::ListK) items = *it.list;
    else if (it.kind == Val::DictK) for (auto& kv : *it.dict) items.push_back(Val::str(kv.first));
    else if (it.kind == Val::Str) for (uint32_t ch : uni::from_utf8(it.s)) items.push_back(Val::str(uni::to_utf8(&ch, 1)));
    else if (it.kind == Val::Undefined) { /* an undefined iterable is an empty one */ }
    else throw TemplateError("the value is not iterable");
    auto bind = [&](const Val& v) {
      if (vars.size() == 1) { c.assign(vars[0], v); return; }
      if (v.kind != Val::ListK || v.list->size() != vars.size()) throw TemplateError("cannot unpack the loop item");
      for (size_t k = 0; k < vars.size(); ++k) c.assign(vars[k], (*v.list)[k]);
    };
    if (filter) {
      List kept;
      c.scopes.emplace_back();
      for (auto& v : items) { bind(v); if (filter->eval(c).truthy()) kept.push_back(v); }
      c.scopes.pop_back();
      items.swap(kept);
    }
    if (items.empty()) { render_body(otherwise, c, out); return; }
    const long long n = (long long)items.size();
    for (long long k = 0; k < n; ++k) {
      c.scopes.emplace_back();
      bind(items[(size_t)k]);
      Val loop = Val::make_dict();
      loop.set("index", Val::integer(k + 1));
      loop.set("index0", Val::integer(k));
      loop.set("revindex", Val::integer(n - k));
      loop.set("revindex0", Val::integer(n - k - 1));
      loop.set("first", Val::boolean(k == 0));
      loop.set("last", Val::boolean(k == n - 1));
      loop.set("length", Val::integer(n));
      if (k > 0) loop.set("previtem", items[(size_t)k - 1]);
      if (k + 1 < n) loop.set("nextitem", items[(size_t)k + 1]);
      c.assign("loop", loop);
      bool stop = false;
      try {
        render_body(body, c, out);
      } catch (const LoopControl& lc) {
        stop = lc.is_break;
      }
      c.scopes.pop_back();
      if (stop) break;
    }
  }
};

struct MacroDef {
  std::string name;
  std::vector<std::pair<std::string, ExprP>> params;      // name, default (may be null)
  Body body;
};
struct MacroNode : Node {
  std::shared_ptr<MacroDef> def;
  void render(Context& c, std::string&) const override { c.macros[def->name] = def.get(); }
};
inline Val call_macro(const MacroDef& m, const std::vector<std::pair<std::string, Val>>& args, Context& c) {
  if (c.depth > 64) throw TemplateError("macro recursion too deep");
  std::map<std::string, Val> frame;
  size_t k = 0;
  for (auto& a : args) {
    if (a.first.empty()) { if (k >= m.params.size()) throw TemplateError("macro '" + m.name + "' takes fewer arguments"); frame[m.params[k++].first] = a.second; }
  }
  for (auto& a : args) {
    if (a.first.empty()) continue;
    bool known = false;
    for (auto& p : m.params) if (p.first == a.first) known = true;
    if (!known) throw TemplateError("macro '" + m.name + "' has no argument '" + a.first + "'");
    frame[a.first] = a.second;
  }
  // a macro sees the template's globals and its own arguments, not the caller's loop variables
  Context inner;
  inner.scopes.push_back(c.scopes.front());
  if (c.scopes.size() > 1) inner.scopes.push_back(c.scopes[1]);
  inner.macros = c.macros;
  inner.depth = c.depth + 1;
  inner.scopes.emplace_back();
  for (auto& p : m.params) {
    auto it = frame.find(p.first);
    if (it != frame.end()) inner.assign(p.first, it->second);
    else if (p.second) inner.assign(p.first, p.second->eval(inner));
    else inner.assign(p.first, Val());
  }
  std::string out;
  render_body(m.body, inner, out);
  return Val::str(out);
}

// ------------------------------------------------------------------------------------------------ lexer and parser
struct Tok { enum Kind { End, Name, Int, Float, Str, Op } kind = End; std::string text; };

class ExprParser {
 public:
  ExprParser(const std::string& src, std::set<std::string>* names) : names_(names) { lex(src); }
  bool at_end() const { return toks_[pos_].kind == Tok::End; }
  const Tok& peek() const { return toks_[pos_]; }
  Tok next() { return toks_[pos_ < toks_.size() - 1 ? pos_++ : pos_]; }
  bool is_op(const char* s) const { return peek().kind == Tok::Op && peek().text == s; }
  bool is_name(const char* s) const { return peek().kind == Tok::Name && peek().text == s; }
  bool eat_op(const char* s) { if (is_op(s)) { ++pos_; return true; } return false; }
  bool eat_name(const char* s) { if (is_name(s)) { ++pos_; return true; } return false; }
  void expect_op(const char* s) { if (!eat_op(s)) throw Unsupported(std::string("expected `") + s + "` near `" + peek().text + "`"); }
  std::string expect_name() { if (peek().kind != Tok::Name) throw Unsupported("expected a name near `" + peek().text + "`"); return next().text; }

  ExprP expression() {            // a if c else b
    ExprP e = or_();
    if (is_name("if")) {
      ++pos_;
      auto cnd = std::make_unique<Cond>();
      cnd->then = std::move(e);
      cnd->test = or_();
      if (eat_name("else")) cnd->otherwise = expression();
      return cnd;
    }
    return e;
  }
  ExprP or_() { ExprP a = and_(); while (eat_name("or")) a = bin("or", std::move(a), and_()); return a; }
  ExprP and_() { ExprP a = not_(); while (eat_name("and")) a = bin("and", std::move(a), not_()); return a; }
  ExprP not_() {
    if (eat_name("not")) { auto u = std::make_unique<Unary>(); u->op = '!'; u->x = not_(); return u; }
    return compare();
  }

 private:
  static ExprP bin(const std::string& op, ExprP a, ExprP b) { auto n = std::make_unique<Binary>(); n->op = op; n->a = std::move(a); n->b = std::move(b); return n; }
  ExprP compare() {
    ExprP a = additive();
    while (true) {
      if (peek().kind == Tok::Op && (peek().text == "==" || peek().text == "!=" || peek().text == "<" || peek().text == ">" || peek().text == "<=" || peek().text == ">=")) {
        const std::string op = next().text;
        a = bin(op, std::move(a), additive());
      } else if (is_name("in")) {
        ++pos_;
        a = bin("in", std::move(a), additive());
      } else if (is_name("not") && toks_[pos_ + 1].kind == Tok::Name && toks_[pos_ + 1].text == "in") {
        pos_ += 2;
        a = bin("not in", std::move(a), additive());
      } else if (is_name("is")) {
        ++pos_;
        auto t = std::make_unique<Test>();
        t->negated = eat_name("not");
        t->name = expect_name();
        t->obj = std::move(a);
        if (eat_op("(")) { while (!is_op(")")) { t->args.push_back(expression()); if (!eat_op(",")) break; } expect_op(")"); }
        else if (peek().kind == Tok::Str || peek().kind == Tok::Int || peek().kind == Tok::Float ||
                 (peek().kind == Tok::Name && !is_name("and") && !is_name("or") && !is_name("else") && !is_name("if") && !is_name("not") && !is_name("is") && !is_name("in")))
          t->args.push_back(postfix(primary()));
        a = std::move(t);
      } else {
        return a;
      }
    }
  }
  ExprP additive() {
    ExprP a = multiplicative();
    while (is_op("+") || is_op("-") || is_op("~")) { const std::string op = next().text; a = bin(op, std::move(a), multiplicative()); }
    return a;
  }
  ExprP multiplicative() {
    ExprP a = unary();
    while (is_op("*") || is_op("/") || is_op("//") || is_op("%")) { const std::string op = next().text; a = bin(op, std::move(a), unary()); }
    return a;
  }
  ExprP unary() {
    if (is_op("-") || is_op("+")) { auto u = std::make_unique<Unary>(); u->op = next().text[0]; u->x = unary(); return u; }
    return postfix(primary());
  }
  std::vector<Arg> call_args() {          // after '('
    std::vector<Arg> args;
    while (!is_op(")")) {
      Arg a;
      if (peek().kind == Tok::Name && toks_[pos_ + 1].kind == Tok::Op && toks_[pos_ + 1].text == "=") { a.name = next().text; ++pos_; }
      if (is_op("*") || is_op("**")) throw Unsupported("argument unpacking");
      a.value = expression();
      args.push_back(std::move(a));
      if (!eat_op(",")) break;
    }
    expect_op(")");
    return args;
  }
  ExprP postfix(ExprP e) {
    while (true) {
      if (eat_op(".")) {
        auto a = std::make_unique<Attr>();
        a->obj = std::move(e);
        if (peek().kind == Tok::Int) a->key = next().text; else a->key = expect_name();
        e = std::move(a);
      } else if (eat_op("[")) {
        ExprP lo, hi;
        bool slice = false;
        if (!is_op(":")) lo = expression();
        if (eat_op(":")) {
          slice = true;
          if (!is_op("]")) hi = expression();
          if (is_op(":")) throw Unsupported("slice with a step");
        }
        expect_op("]");
        if (slice) { auto s = std::make_unique<Slice>(); s->obj = std::move(e); s->lo = std::move(lo); s->hi = std::move(hi); e = std::move(s); }
        else { auto it = std::make_unique<Item>(); it->obj = std::move(e); it->idx = std::move(lo); e = std::move(it); }
      } else if (eat_op("(")) {
        auto cl = std::make_unique<Call>();
        cl->callee = std::move(e);
        cl->args = call_args();
        e = std::move(cl);
      } else if (eat_op("|")) {
        auto f = std::make_unique<Filter>();
        f->obj = std::move(e);
        f->name = expect_name();
        if (eat_op("(")) f->args = call_args();
        e = std::move(f);
      } else {
        return e;
      }
    }
  }
  ExprP primary() {
    const Tok t = next();
    switch (t.kind) {
      case Tok::Int: return std::make_unique<Lit>(Val::integer(std::strtoll(t.text.c_str(), nullptr, 10)));
      case Tok::Float: return std::make_unique<Lit>(Val::real(std::strtod(t.text.c_str(), nullptr)));
      case Tok::Str: {
        std::string s = t.text;
        while (peek().kind == Tok::Str) s += next().text;       // adjacent literals are one string
        return std::make_unique<Lit>(Val::str(s));
      }
      case Tok::Name:
        if (t.text == "true" || t.text == "True") return std::make_unique<Lit>(Val::boolean(true));
        if (t.text == "false" || t.text == "False") return std::make_unique<Lit>(Val::boolean(false));
        if (t.text == "none" || t.text == "None") return std::make_unique<Lit>(Val::none());
        if (names_) names_->insert(t.text);
        return std::make_unique<Name>(t.text);
      case Tok::Op:
        if (t.text == "(") {
          ExprP e = expression();
          if (is_op(",")) throw Unsupported("tuple literal");
          expect_op(")");
          return e;
        }
        if (t.text == "[") {
          auto l = std::make_unique<ListLit>();
          while (!is_op("]")) { l->items.push_back(expression()); if (!eat_op(",")) break; }
          expect_op("]");
          return l;
        }
        if (t.text == "{") {
          auto d = std::make_unique<DictLit>();
          while (!is_op("}")) {
            ExprP k = expression();
            expect_op(":");
            d->items.emplace_back(std::move(k), expression());
            if (!eat_op(",")) break;
          }
          expect_op("}");
          return d;
        }
        break;
      default: break;
    }
    throw Unsupported("unexpected `" + t.text + "` in an expression");
  }
  void lex(const std::string& s) {
    size_t i = 0;
    const size_t n = s.size();
    while (i < n) {
      const unsigned char c = (unsigned char)s[i];
      if (c == ' ' || c == '\t' || c == '\n' || c == '\r') { ++i; continue; }
      Tok t;
      if (((c | 32) >= 'a' && (c | 32) <= 'z') || c == '_' || c >= 0x80) {
        size_t j = i;
        while (j < n && ((((unsigned char)s[j] | 32) >= 'a' && ((unsigned char)s[j] | 32) <= 'z') || s[j] == '_' || (s[j] >= '0' && s[j] <= '9') || (unsigned char)s[j] >= 0x80)) ++j;
        t.kind = Tok::Name; t.text = s.substr(i, j - i); i = j;
      } else if (c >= '0' && c <= '9') {
        size_t j = i;
        bool fl = false;
        while (j < n && ((s[j] >= '0' && s[j] <= '9') || s[j] == '_')) ++j;
        if (j + 1 < n && s[j] == '.' && s[j + 1] >= '0' && s[j + 1] <= '9') { fl = true; ++j; while (j < n && s[j] >= '0' && s[j] <= '9') ++j; }
        if (j < n && (s[j] == 'e' || s[j] == 'E')) { fl = true; ++j; if (j < n && (s[j] == '+' || s[j] == '-')) ++j; while (j < n && s[j] >= '0' && s[j] <= '9') ++j; }
        t.kind = fl ? Tok::Float : Tok::Int;
        for (size_t k = i; k < j; ++k) if (s[k] != '_') t.text.push_back(s[k]);
        i = j;
      } else if (c == '\'' || c == '"') {
        size_t j = i + 1;
        std::string v;
        while (j < n && s[j] != (char)c) {
          if (s[j] == '\\' && j + 1 < n) {
            const char e = s[j + 1];
            j += 2;
            switch (e) {
              case 'n': v.push_back('\n'); break;
              case 't': v.push_back('\t'); break;
              case 'r': v.push_back('\r'); break;
              case '\\': v.push_back('\\'); break;
              case '\'': v.push_back('\''); break;
              case '"': v.push_back('"'); break;
              case '\n': break;
              case 'u': case 'x': {
                const int digits = e == 'u' ? 4 : 2;
                uint32_t cp = 0;
                int k = 0;
                for (; k < digits && j < n && std::isxdigit((unsigned char)s[j]); ++k, ++j) cp = cp * 16 + (uint32_t)(std::isdigit((unsigned char)s[j]) ? s[j] - '0' : (s[j] | 32) - 'a' + 10);
                if (k != digits) throw Unsupported("malformed escape in a string literal");
                uni::append_utf8(v, cp);
                break;
              }
              default: v.push_back('\\'); v.push_back(e);
            }
          } else {
            v.push_back(s[j++]);
          }
        }
        if (j >= n) throw Unsupported("unterminated string literal");
        t.kind = Tok::Str; t.text = v; i = j + 1;
      } else {
        static const char* two[] = {"==", "!=", "<=", ">=", "//", "**"};
        t.kind = Tok::Op;
        for (const char* o : two) if (i + 1 < n && s[i] == o[0] && s[i + 1] == o[1]) t.text = o;
        if (t.text.empty()) {
          if (std::string("+-*/%~|.,:()[]{}=<>").find((char)c) == std::string::npos) throw Unsupported(std::string("unexpected character `") + (char)c + "`");
          t.text = std::string(1, (char)c);
        }
        i += t.text.size();
      }
      toks_.push_back(std::move(t));
    }
    toks_.push_back(Tok{});
    toks_.push_back(Tok{});
  }
  std::vector<Tok> toks_;
  size_t pos_ = 0;
  std::set<std::string>* names_;
};

class Template {
 public:
  // Parses `source` the way chat templates are rendered: trim_blocks and lstrip_blocks on.  Throws Unsupported.
  static std::unique_ptr<Template> compile(const std::string& source) {
    std::unique_ptr<Template> t(new Template());
    std::string src = source;                 // one newline at the very end does not count (keep_trailing_newline is off)
    if (!src.empty() && src.back() == '\n') { src.pop_back(); if (!src.empty() && src.back() == '\r') src.pop_back(); }
    std::vector<Segment> segs = t->segments(src);
    size_t pos = 0;
    std::string end;
    t->body_ = t->parse_body(segs, pos, {}, &end);
    if (pos != segs.size()) throw Unsupported("unexpected `" + end + "` block");
    return t;
  }
  // Names the template reads (loop variables and assigned names included: a superset of its undeclared variables).
  bool mentions(const std::string& name) const { return names_.count(name) != 0; }

  std::string render(const Val& globals) const {
    Context c;
    c.scopes.emplace_back();
    if (globals.kind == Val::DictK) for (auto& kv : *globals.dict) c.scopes.back()[kv.first] = kv.second;
    c.scopes.emplace_back();
    std::string out;
    render_body(body_, c, out);
    return out;
  }

 private:
  struct Segment { enum Kind { Text, Output, Block } kind; std::string text; };

  // Splits the source into text, `{{ }}` and `{% %}` pieces and applies white-space control the way Jinja2's lexer does with
  // trim_blocks and lstrip_blocks on: a `-` at a tag's edge strips all white space on that side; the spaces and tabs between a
  // line's start and a block or comment tag go (unless the tag opens with `+`); one newline right after such a tag goes.
  std::vector<Segment> segments(const std::string& s) const {
    std::vector<Segment> out;
    size_t i = 0;
    const size_t n = s.size();
    std::string text;
    bool line_starting = true;       // the text collected since the last tag begins at a line's start
    while (i < n) {
      if (!(s[i] == '{' && i + 1 < n && (s[i + 1] == '{' || s[i + 1] == '%' || s[i + 1] == '#'))) { text.push_back(s[i++]); continue; }
      const char kind = s[i + 1];
      const char* close = kind == '{' ? "}}" : kind == '%' ? "%}" : "#}";
      size_t j = i + 2;
      bool plus = false, strip_left = false;
      if (j < n && s[j] == '-') { strip_left = true; ++j; }
      else if (j < n && s[j] == '+' && kind != '{') { plus = true; ++j; }
      size_t k = j;                    // the closing delimiter, outside string literals and outside dict literals ("}}" may close two)
      char quote = 0;
      int braces = 0;
      while (k + 1 < n) {
        if (kind != '#' && quote) { if (s[k] == '\\') { k += 2; continue; } if (s[k] == quote) quote = 0; ++k; continue; }
        if (kind != '#' && (s[k] == '\'' || s[k] == '"')) { quote = s[k]; ++k; continue; }
        if (kind != '#' && s[k] == '{') { ++braces; ++k; continue; }
        if (kind != '#' && s[k] == '}' && braces > 0) { --braces; ++k; continue; }
        if (s[k] == close[0] && s[k + 1] == close[1]) break;
        ++k;
      }
      if (k + 1 >= n) throw Unsupported("unterminated tag");
      size_t inner_end = k;
      bool strip_right = false, keep_newline = false;
      if (inner_end > j && s[inner_end - 1] == '-') { strip_right = true; --inner_end; }
      else if (kind != '{' && inner_end > j && s[inner_end - 1] == '+') { keep_newline = true; --inner_end; }
      // the text in front of the tag
      if (strip_left) {
        while (!text.empty() && std::isspace((unsigned char)text.back())) text.pop_back();
      } else if (kind != '{' && !plus) {
        const size_t l_pos = text.rfind('\n') == std::string::npos ? 0 : text.rfind('\n') + 1;
        if (l_pos > 0 || line_starting) {
          bool blank = true;
          for (size_t q = l_pos; q < text.size(); ++q) if (text[q] != ' ' && text[q] != '\t') { blank = false; break; }
          if (blank) text.erase(l_pos);
        }
      }
      if (!text.empty()) out.push_back(Segment{Segment::Text, text});
      text.clear();
      const std::string inner = s.substr(j, inner_end - j);
      if (kind == '{') out.push_back(Segment{Segment::Output, inner});
      else if (kind == '%') out.push_back(Segment{Segment::Block, inner});
      // what the tag takes along behind it
      i = k + 2;
      line_starting = false;
      if (strip_right) {
        size_t q = i;
        while (q < n && std::isspace((unsigned char)s[q])) ++q;
        line_starting = q > i && s[q - 1] == '\n';
        i = q;
      } else if (kind != '{' && !keep_newline && i < n && s[i] == '\n') {
        ++i;
        line_starting = true;
      }
    }
    if (!text.empty()) out.push_back(Segment{Segment::Text, text});
    return out;
  }

  static std::string first_word(const std::string& s, std::string* rest) {
    size_t b = 0;
    while (b < s.size() && std::isspace((unsigned char)s[b])) ++b;
    size_t e = b;
    while (e < s.size() && (std::isalnum((unsigned char)s[e]) || s[e] == '_')) ++e;
    if (rest) *rest = s.substr(e);
    return s.substr(b, e - b);
  }

  Body parse_body(const std::vector<Segment>& segs, size_t& pos, const std::set<std::string>& until, std::string* ended_by) {
    Body body;
    while (pos < segs.size()) {
      const Segment& sg = segs[pos];
      if (sg.kind == Segment::Text) { auto t = std::make_unique<TextNode>(); t->text = sg.text; body.push_back(std::move(t)); ++pos; continue; }
      if (sg.kind == Segment::Output) {
        ExprParser ep(sg.text, &names_);
        auto o = std::make_unique<OutputNode>();
        o->e = ep.expression();
        if (!ep.at_end()) throw Unsupported("unexpected `" + ep.peek().text + "` in `{{" + sg.text + "}}`");
        body.push_back(std::move(o));
        ++pos;
        continue;
      }
      std::string rest;
      const std::string kw = first_word(sg.text, &rest);
      if (until.count(kw)) { if (ended_by) *ended_by = kw; return body; }
      ++pos;
      if (kw == "if") {
        auto node = std::make_unique<IfNode>();
        std::string cond_src = rest, end;
        while (true) {
          ExprP cond;
          if (!cond_src.empty()) { ExprParser ep(cond_src, &names_); cond = ep.expression(); if (!ep.at_end()) throw Unsupported("unexpected `" + ep.peek().text + "` in an if"); }
          Body b = parse_body(segs, pos, {"elif", "else", "endif"}, &end);
          if (pos >= segs.size()) throw Unsupported("if without endif");
          node->branches.emplace_back(std::move(cond), std::move(b));
          std::string r2;
          first_word(segs[pos].text, &r2);
          ++pos;
          if (end == "endif") break;
          if (end == "elif") cond_src = r2; else cond_src.clear();
          if (end == "else" && !cond_src.empty()) throw Unsupported("else with a condition");
        }
        body.push_back(std::move(node));
      } else if (kw == "for") {
        auto node = std::make_unique<ForNode>();
        ExprParser ep(rest, &names_);
        node->vars.push_back(ep.expect_name());
        while (ep.eat_op(",")) node->vars.push_back(ep.expect_name());
        if (!ep.eat_name("in")) throw Unsupported("for without in");
        node->iterable = ep.or_();
        if (ep.eat_name("if")) node->filter = ep.or_();
        if (!ep.at_end()) throw Unsupported("unexpected `" + ep.peek().text + "` in a for");
        std::string end;
        ++in_loop_;
        node->body = parse_body(segs, pos, {"else", "endfor"}, &end);
        --in_loop_;
        if (pos >= segs.size()) throw Unsupported("for without endfor");
        ++pos;
        if (end == "else") {
          node->otherwise = parse_body(segs, pos, {"endfor"}, &end);
          if (pos >= segs.size()) throw Unsupported("for without endfor");
          ++pos;
        }
        body.push_back(std::move(node));
      } else if (kw == "set") {
        ExprParser ep(rest, &names_);
        auto node = std::make_unique<SetNode>();
        node->name = ep.expect_name();
        if (ep.eat_op(".")) node->attr = ep.expect_name();
        if (ep.is_op(",")) throw Unsupported("set of several names");
        if (ep.eat_op("=")) {
          node->value = ep.expression();
          if (!ep.at_end()) throw Unsupported("unexpected `" + ep.peek().text + "` in a set");
        } else {
          if (!ep.at_end()) throw Unsupported("block set with a filter");
          std::string end;
          node->block = parse_body(segs, pos, {"endset"}, &end);
          if (pos >= segs.size()) throw Unsupported("set without endset");
          ++pos;
        }
        body.push_back(std::move(node));
      } else if (kw == "macro") {
        ExprParser ep(rest, &names_);
        auto def = std::make_shared<MacroDef>();
        def->name = ep.expect_name();
        ep.expect_op("(");
        while (!ep.is_op(")")) {
          std::string pn = ep.expect_name();
          ExprP dflt;
          if (ep.eat_op("=")) dflt = ep.expression();
          def->params.emplace_back(pn, std::move(dflt));
          if (!ep.eat_op(",")) break;
        }
        ep.expect_op(")");
        if (!ep.at_end()) throw Unsupported("unexpected `" + ep.peek().text + "` in a macro");
        std::string end;
        def->body = parse_body(segs, pos, {"endmacro"}, &end);
        if (pos >= segs.size()) throw Unsupported("macro without endmacro");
        ++pos;
        auto node = std::make_unique<MacroNode>();
        node->def = std::move(def);
        body.push_back(std::move(node));
      } else if (kw == "break" || kw == "continue") {
        if (!in_loop_) throw Unsupported("`" + kw + "` outside a loop");
        auto node = std::make_unique<LoopControlNode>();
        node->is_break = kw == "break";
        body.push_back(std::move(node));
      } else if (kw == "generation" || kw == "endgeneration") {
        // markers around the assistant's text (used for training masks): nothing to render
      } else {
        throw Unsupported("`" + kw + "` block");
      }
    }
    if (ended_by) ended_by->clear();
    return body;
  }

  Body body_;
  std::set<std::string> names_;
  int in_loop_ = 0;
};

// ------------------------------------------------------------------------------------------------ chat requests
// The prompt of a chat request, as the shard's renderer builds it (reference: router/src/infer.rs:97-147): content parts become
// text, a template that names `guideline` needs one, and with tools the tool prompt is appended to the last message, preceded by the
// tools as JSON when the template has no place for them.
inline const char* default_tool_prompt() {
  return "\nGiven the functions available, please respond with a JSON for a function call with its proper arguments that best answers the "
         "given prompt. Respond in the format {name: function name, parameters: dictionary of argument name and its value}.Do not use "
         "variables.\n";
}
struct ChatRenderer {
  std::unique_ptr<Template> tmpl;
  std::string bos_token, eos_token;

  std::string render(const json::Value& req) const {
    List msgs;
    for (auto& m : req["messages"].items()) {
      Val mv = from_json(m);
      if (mv.kind != Val::DictK) throw TemplateError("a message is no object");
      if (m["content"].is_array()) {
        std::string text;
        for (auto& part : m["content"].items()) if (part.is_object() && part["text"].is_string()) text += part["text"].as_string();
        mv.set("content", Val::str(text));
      }
      msgs.push_back(mv);
    }
    const bool has_tools = req["tools"].is_array() && req["tools"].size() > 0;
    if (tmpl->mentions("guideline") && !req["guideline"].is_string()) throw TemplateError("Missing template vatiable: guideline");
    if (has_tools) {
      const std::string prompt = req["tool_prompt"].is_string() ? req["tool_prompt"].as_string() : default_tool_prompt();
      std::string tools_json;           // json.dumps(tools, separators=(",", ":"))
      JsonStyle plain;
      plain.sort_keys = false; plain.html_safe = false; plain.compact = true;
      json_dump(from_json(req["tools"]), tools_json, -1, 0, plain);
      const std::string text = tmpl->mentions("tools") ? "\n---\n" + prompt : "\n---\n" + tools_json + "\n" + prompt;
      if (!msgs.empty()) {
        const Val* c = msgs.back().find("content");
        msgs.back().set("content", Val::str((c && c->kind == Val::Str ? c->s : std::string()) + text));
      }
    }
    Val g = Val::make_dict();
    g.set("messages", Val::make_list(std::move(msgs)));
    g.set("bos_token", Val::str(bos_token));
    g.set("eos_token", Val::str(eos_token));
    g.set("add_generation_prompt", Val::boolean(true));
    g.set("tools", has_tools ? from_json(req["tools"]) : Val::none());
    g.set("tools_in_user_message", Val::boolean(false));
    g.set("guideline", req["guideline"].is_string() ? Val::str(req["guideline"].as_string()) : Val::none());
    return tmpl->render(g);
  }
};

}  // namespace jinja
}  // namespace lx
