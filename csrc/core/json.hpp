// Minimal JSON value with insertion-ordered objects, a strict parser and a compact serialiser.
// Objects keep the order in which keys were inserted, so a struct serialised field by field gives
// the same bytes every time; the plan's content hash is taken over those bytes (the reference hashes
// serde_json's struct-order output: crates/skein_ir/src/plan.rs:140).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace skein {

struct JsonError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Json {
 public:
  enum Type { Null, Bool, Int, Float, String, Array, Object };
  using Arr = std::vector<Json>;
  using Obj = std::vector<std::pair<std::string, Json>>;

  Json() : t_(Null) {}
  Json(std::nullptr_t) : t_(Null) {}
  Json(bool b) : t_(Bool), b_(b) {}
  Json(int v) : t_(Int), i_(v) {}
  Json(unsigned v) : t_(Int), i_(v) {}
  Json(long v) : t_(Int), i_(v) {}
  Json(long long v) : t_(Int), i_(v) {}
  Json(unsigned long v) : t_(Int), i_((long long)v) {}
  Json(unsigned long long v) : t_(Int), i_((long long)v) {}
  Json(double v) : t_(Float), f_(v) {}
  Json(const char* s) : t_(String), s_(s) {}
  Json(std::string s) : t_(String), s_(std::move(s)) {}
  static Json array() { Json j; j.t_ = Array; return j; }
  static Json object() { Json j; j.t_ = Object; return j; }

  Type type() const { return t_; }
  bool is_null() const { return t_ == Null; }
  bool is_number() const { return t_ == Int || t_ == Float; }
  bool is_string() const { return t_ == String; }
  bool is_object() const { return t_ == Object; }
  bool is_array() const { return t_ == Array; }
  bool is_bool() const { return t_ == Bool; }

  bool as_bool() const { need(Bool, "bool"); return b_; }
  long long as_int() const {
    if (t_ == Int) return i_;
    if (t_ == Float && std::floor(f_) == f_) return (long long)f_;
    throw JsonError("expected an integer");
  }
  double as_double() const {
    if (t_ == Int) return (double)i_;
    if (t_ == Float) return f_;
    throw JsonError("expected a number");
  }
  const std::string& as_string() const { need(String, "string"); return s_; }
  const Arr& items() const { need(Array, "array"); return a_; }
  Arr& items() { need(Array, "array"); return a_; }
  const Obj& members() const { need(Object, "object"); return o_; }

  void push(Json v) { need(Array, "array"); a_.push_back(std::move(v)); }
  // insert or replace, keeping first-insertion order
  Json& set(const std::string& k, Json v) {
    need(Object, "object");
    for (auto& kv : o_) if (kv.first == k) { kv.second = std::move(v); return *this; }
    o_.emplace_back(k, std::move(v));
    return *this;
  }
  bool has(const std::string& k) const {
    if (t_ != Object) return false;
    for (auto& kv : o_) if (kv.first == k) return true;
    return false;
  }
  const Json& at(const std::string& k) const {
    need(Object, "object");
    for (auto& kv : o_) if (kv.first == k) return kv.second;
    throw JsonError("missing key `" + k + "`");
  }
  Json* find(const std::string& k) {
    if (t_ != Object) return nullptr;
    for (auto& kv : o_) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  const Json* find(const std::string& k) const { return const_cast<Json*>(this)->find(k); }
  size_t size() const { return t_ == Array ? a_.size() : t_ == Object ? o_.size() : 0; }

  // ---- serialise -----------------------------------------------------------------------------
  std::string dump(int indent = -1) const { std::string out; write(out, indent, 0); return out; }

  static std::string fmt_double(double v) {
    if (std::isnan(v) || std::isinf(v)) return "null";
    if (std::floor(v) == v && std::fabs(v) < 1e15) {
      char b[40]; snprintf(b, sizeof b, "%.1f", v); return b;
    }
    for (int prec = 1; prec <= 17; ++prec) {
      char b[40]; snprintf(b, sizeof b, "%.*g", prec, v);
      if (strtod(b, nullptr) == v) return b;
    }
    char b[40]; snprintf(b, sizeof b, "%.17g", v); return b;
  }

  // ---- parse -----------------------------------------------------------------------------------
  static Json parse(const std::string& text) {
    size_t i = 0;
    Json v = parse_value(text, i);
    skip_ws(text, i);
    if (i != text.size()) throw JsonError("trailing characters after JSON value at offset " + std::to_string(i));
    return v;
  }

 private:
  Type t_;
  bool b_ = false;
  long long i_ = 0;
  double f_ = 0;
  std::string s_;
  Arr a_;
  Obj o_;

  void need(Type t, const char* what) const {
    if (t_ != t) throw JsonError(std::string("expected ") + what);
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
        default:
          if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
          else out += (char)c;
      }
    }
    out += '"';
  }
  void write(std::string& out, int indent, int depth) const {
    auto nl = [&](int d) { if (indent >= 0) { out += '\n'; out.append((size_t)(indent * d), ' '); } };
    switch (t_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Int: out += std::to_string(i_); break;
      case Float: out += fmt_double(f_); break;
      case String: escape(s_, out); break;
      case Array:
        out += '[';
        for (size_t k = 0; k < a_.size(); ++k) { if (k) out += ','; nl(depth + 1); a_[k].write(out, indent, depth + 1); }
        if (!a_.empty()) nl(depth);
        out += ']';
        break;
      case Object:
        out += '{';
        for (size_t k = 0; k < o_.size(); ++k) {
          if (k) out += ',';
          nl(depth + 1);
          escape(o_[k].first, out);
          out += indent >= 0 ? ": " : ":";
          o_[k].second.write(out, indent, depth + 1);
        }
        if (!o_.empty()) nl(depth);
        out += '}';
        break;
    }
  }
  static void skip_ws(const std::string& s, size_t& i) {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  static std::string parse_string(const std::string& s, size_t& i) {
    std::string out;
    ++i;  // opening quote
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c != '\\') { out += c; continue; }
      if (i >= s.size()) break;
      char e = s[i++];
      switch (e) {
        case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
        case 'b': out += '\b'; break; case 'f': out += '\f'; break;
        case 'u': {
          if (i + 4 > s.size()) throw JsonError("bad \\u escape");
          unsigned cp = (unsigned)strtoul(s.substr(i, 4).c_str(), nullptr, 16);
          i += 4;
          if (cp < 0x80) out += (char)cp;
          else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
          else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
          break;
        }
        default: out += e;
      }
    }
    if (i >= s.size()) throw JsonError("unterminated string");
    ++i;
    return out;
  }
  static Json parse_value(const std::string& s, size_t& i) {
    skip_ws(s, i);
    if (i >= s.size()) throw JsonError("unexpected end of JSON");
    char c = s[i];
    if (c == '{') {
      Json o = object();
      ++i; skip_ws(s, i);
      if (i < s.size() && s[i] == '}') { ++i; return o; }
      for (;;) {
        skip_ws(s, i);
        if (i >= s.size() || s[i] != '"') throw JsonError("expected a key at offset " + std::to_string(i));
        std::string k = parse_string(s, i);
        skip_ws(s, i);
        if (i >= s.size() || s[i] != ':') throw JsonError("expected `:` at offset " + std::to_string(i));
        ++i;
        o.o_.emplace_back(std::move(k), parse_value(s, i));
        skip_ws(s, i);
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; return o; }
        throw JsonError("expected `,` or `}` at offset " + std::to_string(i));
      }
    }
    if (c == '[') {
      Json a = array();
      ++i; skip_ws(s, i);
      if (i < s.size() && s[i] == ']') { ++i; return a; }
      for (;;) {
        a.a_.push_back(parse_value(s, i));
        skip_ws(s, i);
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; return a; }
        throw JsonError("expected `,` or `]` at offset " + std::to_string(i));
      }
    }
    if (c == '"') return Json(parse_string(s, i));
    if (s.compare(i, 4, "true") == 0) { i += 4; return Json(true); }
    if (s.compare(i, 5, "false") == 0) { i += 5; return Json(false); }
    if (s.compare(i, 4, "null") == 0) { i += 4; return Json(); }
    size_t j = i;
    bool is_float = false;
    if (j < s.size() && (s[j] == '-' || s[j] == '+')) ++j;
    while (j < s.size() && (isdigit((unsigned char)s[j]) || s[j] == '.' || s[j] == 'e' || s[j] == 'E' || s[j] == '-' || s[j] == '+')) {
      if (s[j] == '.' || s[j] == 'e' || s[j] == 'E') is_float = true;
      ++j;
    }
    if (j == i) throw JsonError("unexpected character at offset " + std::to_string(i));
    std::string num = s.substr(i, j - i);
    i = j;
    if (is_float) return Json(strtod(num.c_str(), nullptr));
    return Json((long long)strtoll(num.c_str(), nullptr, 10));
  }
};

}  // namespace skein
