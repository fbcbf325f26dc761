// Small JSON value with a strict parser and a serialiser: enough for the REST / OpenAI request and response
// bodies of the router (the reference uses serde_json, router/src/lib.rs).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <cstring>
#include <utility>
#include <vector>

namespace json {

class Value;
using Array = std::vector<Value>;
using Object = std::vector<std::pair<std::string, Value>>;   // insertion ordered

class Value {
 public:
  enum Type { Null, Bool, Number, String, Arr, Obj };
  Value() : type_(Null) {}
  Value(std::nullptr_t) : type_(Null) {}
  Value(bool b) : type_(Bool), b_(b) {}
  Value(int v) : type_(Number), n_(v), is_int_(true) {}
  Value(unsigned v) : type_(Number), n_(v), is_int_(true) {}
  Value(long v) : type_(Number), n_((double)v), is_int_(true) {}
  Value(long long v) : type_(Number), n_((double)v), is_int_(true) {}
  Value(unsigned long v) : type_(Number), n_((double)v), is_int_(true) {}
  Value(unsigned long long v) : type_(Number), n_((double)v), is_int_(true) {}
  Value(double v) : type_(Number), n_(v) {}
  Value(float v) : type_(Number), n_(v) {}
  Value(const char* s) : type_(String), s_(s) {}
  Value(std::string s) : type_(String), s_(std::move(s)) {}
  Value(Array a) : type_(Arr), a_(std::make_shared<Array>(std::move(a))) {}
  Value(Object o) : type_(Obj), o_(std::make_shared<Object>(std::move(o))) {}
  static Value array() { return Value(Array{}); }
  static Value object() { return Value(Object{}); }

  Type type() const { return type_; }
  bool is_null() const { return type_ == Null; }
  bool is_bool() const { return type_ == Bool; }
  bool is_number() const { return type_ == Number; }
  bool is_string() const { return type_ == String; }
  bool is_array() const { return type_ == Arr; }
  bool is_object() const { return type_ == Obj; }
  bool as_bool(bool d = false) const { return type_ == Bool ? b_ : d; }
  double as_double(double d = 0) const { return type_ == Number ? n_ : d; }
  long long as_int(long long d = 0) const { return type_ == Number ? (long long)n_ : d; }
  const std::string& as_string() const { static const std::string e; return type_ == String ? s_ : e; }
  const Array& items() const { static const Array e; return type_ == Arr ? *a_ : e; }
  const Object& members() const { static const Object e; return type_ == Obj ? *o_ : e; }

  const Value& operator[](const std::string& key) const {
    static const Value none;
    if (type_ != Obj) return none;
    for (const auto& kv : *o_) if (kv.first == key) return kv.second;
    return none;
  }
  bool has(const std::string& key) const { return type_ == Obj && !(*this)[key].is_null_missing(key, *this); }
  Value& set(const std::string& key, Value v) {
    if (type_ != Obj) { type_ = Obj; o_ = std::make_shared<Object>(); }
    for (auto& kv : *o_) if (kv.first == key) { kv.second = std::move(v); return kv.second; }
    o_->emplace_back(key, std::move(v));
    return o_->back().second;
  }
  void push(Value v) {
    if (type_ != Arr) { type_ = Arr; a_ = std::make_shared<Array>(); }
    a_->push_back(std::move(v));
  }
  size_t size() const { return type_ == Arr ? a_->size() : type_ == Obj ? o_->size() : 0; }

  std::string dump() const { std::string out; dump_to(out); return out; }
  void dump_to(std::string& out) const {
    switch (type_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Number: {
        char buf[40];
        if (is_int_ || (std::floor(n_) == n_ && std::fabs(n_) < 1e15)) snprintf(buf, sizeof buf, "%lld", (long long)n_);
        else if (!std::isfinite(n_)) snprintf(buf, sizeof buf, "null");
        else snprintf(buf, sizeof buf, "%.9g", n_);
        out += buf;
        break;
      }
      case String: escape(s_, out); break;
      case Arr: {
        out += '[';
        bool first = true;
        for (const auto& v : *a_) { if (!first) out += ','; first = false; v.dump_to(out); }
        out += ']';
        break;
      }
      case Obj: {
        out += '{';
        bool first = true;
        for (const auto& kv : *o_) {
          if (!first) out += ',';
          first = false;
          escape(kv.first, out);
          out += ':';
          kv.second.dump_to(out);
        }
        out += '}';
        break;
      }
    }
  }
  static void escape(const std::string& s, std::string& out) {
    out += '"';
    for (unsigned char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        case '\b': out += "\\b"; break;
        case '\f': out += "\\f"; break;
        default:
          if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
          else out += (char)c;
      }
    }
    out += '"';
  }

 private:
  bool is_null_missing(const std::string& key, const Value& parent) const {
    for (const auto& kv : *parent.o_) if (kv.first == key) return false;
    return true;
  }
  Type type_;
  bool b_ = false;
  double n_ = 0;
  bool is_int_ = false;
  std::string s_;
  std::shared_ptr<Array> a_;
  std::shared_ptr<Object> o_;
};

class Parser {
 public:
  explicit Parser(const std::string& s) : p_(s.data()), end_(s.data() + s.size()) {}
  bool parse(Value& out, std::string* err = nullptr) {
    bool ok = value(out, 0);
    ws();
    if (ok && p_ != end_) { ok = false; err_ = "trailing characters"; }
    if (!ok && err) *err = err_.empty() ? "invalid JSON" : err_;
    return ok;
  }

 private:
  void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
  bool lit(const char* s) {
    size_t n = strlen(s);
    if ((size_t)(end_ - p_) < n || strncmp(p_, s, n) != 0) return false;
    p_ += n;
    return true;
  }
  bool value(Value& out, int depth) {
    if (depth > 128) { err_ = "nesting too deep"; return false; }
    ws();
    if (p_ >= end_) { err_ = "unexpected end"; return false; }
    switch (*p_) {
      case 'n': if (lit("null")) { out = Value(); return true; } break;
      case 't': if (lit("true")) { out = Value(true); return true; } break;
      case 'f': if (lit("false")) { out = Value(false); return true; } break;
      case '"': { std::string s; if (!str(s)) return false; out = Value(std::move(s)); return true; }
      case '[': {
        ++p_;
        Array a;
        ws();
        if (p_ < end_ && *p_ == ']') { ++p_; out = Value(std::move(a)); return true; }
        while (true) {
          Value v;
          if (!value(v, depth + 1)) return false;
          a.push_back(std::move(v));
          ws();
          if (p_ < end_ && *p_ == ',') { ++p_; continue; }
          if (p_ < end_ && *p_ == ']') { ++p_; break; }
          err_ = "expected , or ]";
          return false;
        }
        out = Value(std::move(a));
        return true;
      }
      case '{': {
        ++p_;
        Object o;
        ws();
        if (p_ < end_ && *p_ == '}') { ++p_; out = Value(std::move(o)); return true; }
        while (true) {
          ws();
          std::string k;
          if (p_ >= end_ || *p_ != '"' || !str(k)) { err_ = "expected string key"; return false; }
          ws();
          if (p_ >= end_ || *p_ != ':') { err_ = "expected :"; return false; }
          ++p_;
          Value v;
          if (!value(v, depth + 1)) return false;
          o.emplace_back(std::move(k), std::move(v));
          ws();
          if (p_ < end_ && *p_ == ',') { ++p_; continue; }
          if (p_ < end_ && *p_ == '}') { ++p_; break; }
          err_ = "expected , or }";
          return false;
        }
        out = Value(std::move(o));
        return true;
      }
      default: {
        char* e = nullptr;
        double d = strtod(p_, &e);
        if (e == p_ || e > end_) break;
        bool is_int = true;
        for (const char* q = p_; q < e; ++q) if (*q == '.' || *q == 'e' || *q == 'E') is_int = false;
        p_ = e;
        out = is_int ? Value((long long)d) : Value(d);
        return true;
      }
    }
    err_ = "unexpected token";
    return false;
  }
  static void utf8(unsigned cp, std::string& s) {
    if (cp < 0x80) s += (char)cp;
    else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
    else { s += (char)(0xF0 | (cp >> 18)); s += (char)(0x80 | ((cp >> 12) & 0x3F)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
  }
  bool hex4(unsigned& v) {
    if (end_ - p_ < 4) return false;
    v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else return false;
    }
    return true;
  }
  bool str(std::string& s) {
    ++p_;
    while (p_ < end_) {
      char c = *p_++;
      if (c == '"') return true;
      if (c == '\\') {
        if (p_ >= end_) break;
        char e = *p_++;
        switch (e) {
          case '"': s += '"'; break; case '\\': s += '\\'; break; case '/': s += '/'; break;
          case 'b': s += '\b'; break; case 'f': s += '\f'; break; case 'n': s += '\n'; break;
          case 'r': s += '\r'; break; case 't': s += '\t'; break;
          case 'u': {
            unsigned cp;
            if (!hex4(cp)) { err_ = "bad \\u escape"; return false; }
            if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
              p_ += 2;
              unsigned lo;
              if (!hex4(lo)) { err_ = "bad surrogate"; return false; }
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(cp, s);
            break;
          }
          default: err_ = "bad escape"; return false;
        }
      } else {
        s += c;
      }
    }
    err_ = "unterminated string";
    return false;
  }
  const char* p_;
  const char* end_;
  std::string err_;
};

inline bool parse(const std::string& s, Value& out, std::string* err = nullptr) { return Parser(s).parse(out, err); }

}  // namespace json
