// The subset of TOML that the cluster, cost-constant, drift-table and calibration-corpus files
// use: comments, `key = value`, `[a.b]` tables, `[[a]]` arrays of tables, strings, integers, floats,
// booleans and (possibly multi-line) arrays. Parses into a Json object.
#pragma once
#include "json.hpp"

namespace skein {

struct TomlError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

namespace toml_detail {

inline std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && isspace((unsigned char)s[a])) ++a;
  while (b > a && isspace((unsigned char)s[b - 1])) --b;
  return s.substr(a, b - a);
}

inline std::string strip_comment(const std::string& line) {
  bool in_str = false;
  for (size_t i = 0; i < line.size(); ++i) {
    if (line[i] == '"' && (i == 0 || line[i - 1] != '\\')) in_str = !in_str;
    if (line[i] == '#' && !in_str) return line.substr(0, i);
  }
  return line;
}

inline std::vector<std::string> split_key(const std::string& k) {
  std::vector<std::string> parts;
  std::string cur;
  bool in_str = false;
  for (char c : k) {
    if (c == '"') { in_str = !in_str; continue; }
    if (c == '.' && !in_str) { parts.push_back(trim(cur)); cur.clear(); continue; }
    cur += c;
  }
  parts.push_back(trim(cur));
  for (auto& p : parts) if (p.empty()) throw TomlError("empty key component in `" + k + "`");
  return parts;
}

inline Json parse_scalar(const std::string& v, int line_no);

inline Json parse_value(const std::string& raw, int line_no) {
  std::string v = trim(raw);
  if (v.empty()) throw TomlError("line " + std::to_string(line_no) + ": missing value");
  if (v[0] == '[') {
    if (v.back() != ']') throw TomlError("line " + std::to_string(line_no) + ": unterminated array");
    Json arr = Json::array();
    std::string inner = v.substr(1, v.size() - 2), cur;
    int depth = 0;
    bool in_str = false;
    for (size_t i = 0; i <= inner.size(); ++i) {
      char c = i < inner.size() ? inner[i] : ',';
      if (c == '"' && (i == 0 || inner[i - 1] != '\\')) in_str = !in_str;
      if (!in_str && c == '[') ++depth;
      if (!in_str && c == ']') --depth;
      if (c == ',' && depth == 0 && !in_str) {
        if (!trim(cur).empty()) arr.push(parse_value(cur, line_no));
        cur.clear();
      } else {
        cur += c;
      }
    }
    return arr;
  }
  return parse_scalar(v, line_no);
}

inline Json parse_scalar(const std::string& v, int line_no) {
  if (v[0] == '"') {
    if (v.size() < 2 || v.back() != '"') throw TomlError("line " + std::to_string(line_no) + ": unterminated string");
    std::string out;
    for (size_t i = 1; i + 1 < v.size(); ++i) {
      if (v[i] == '\\' && i + 2 < v.size()) {
        char e = v[++i];
        out += e == 'n' ? '\n' : e == 't' ? '\t' : e;
      } else out += v[i];
    }
    return Json(out);
  }
  if (v == "true") return Json(true);
  if (v == "false") return Json(false);
  std::string num;
  for (char c : v) if (c != '_') num += c;
  char* end = nullptr;
  bool is_float = num.find_first_of(".eE") != std::string::npos || num == "inf" || num == "nan";
  if (is_float) {
    double d = strtod(num.c_str(), &end);
    if (end && *end == 0) return Json(d);
  } else {
    long long i = strtoll(num.c_str(), &end, 10);
    if (end && *end == 0 && !num.empty()) return Json(i);
  }
  throw TomlError("line " + std::to_string(line_no) + ": cannot parse value `" + v + "`");
}

inline Json* descend(Json* cur, const std::string& key) {
  Json* next = cur->find(key);
  if (!next) { cur->set(key, Json::object()); next = cur->find(key); }
  if (next->is_array()) {
    if (next->size() == 0) throw TomlError("empty array of tables `" + key + "`");
    return &next->items().back();
  }
  if (!next->is_object()) throw TomlError("key `" + key + "` is not a table");
  return next;
}

}  // namespace toml_detail

inline Json parse_toml(const std::string& text) {
  using namespace toml_detail;
  Json root = Json::object();
  Json* cur = &root;
  std::vector<std::string> lines;
  {
    std::string l;
    for (char c : text) { if (c == '\n') { lines.push_back(l); l.clear(); } else l += c; }
    lines.push_back(l);
  }
  for (size_t li = 0; li < lines.size(); ++li) {
    int line_no = (int)li + 1;
    std::string line = trim(strip_comment(lines[li]));
    if (line.empty()) continue;
    if (line.size() >= 4 && line.compare(0, 2, "[[") == 0) {
      if (line.compare(line.size() - 2, 2, "]]") != 0) throw TomlError("line " + std::to_string(line_no) + ": bad table array header");
      auto parts = split_key(line.substr(2, line.size() - 4));
      Json* t = &root;
      for (size_t i = 0; i + 1 < parts.size(); ++i) t = descend(t, parts[i]);
      Json* arr = t->find(parts.back());
      if (!arr) { t->set(parts.back(), Json::array()); arr = t->find(parts.back()); }
      if (!arr->is_array()) throw TomlError("line " + std::to_string(line_no) + ": `" + parts.back() + "` is not an array of tables");
      arr->push(Json::object());
      cur = &arr->items().back();
      continue;
    }
    if (line[0] == '[') {
      if (line.back() != ']') throw TomlError("line " + std::to_string(line_no) + ": bad table header");
      auto parts = split_key(line.substr(1, line.size() - 2));
      Json* t = &root;
      for (auto& p : parts) t = descend(t, p);
      cur = t;
      continue;
    }
    size_t eq = std::string::npos;
    {
      bool in_str = false;
      for (size_t i = 0; i < line.size(); ++i) {
        if (line[i] == '"') in_str = !in_str;
        if (line[i] == '=' && !in_str) { eq = i; break; }
      }
    }
    if (eq == std::string::npos) throw TomlError("line " + std::to_string(line_no) + ": expected `key = value`");
    std::string val = line.substr(eq + 1);
    // multi-line arrays: keep reading until brackets balance
    auto balance = [](const std::string& s) {
      int d = 0; bool in_str = false;
      for (char c : s) { if (c == '"') in_str = !in_str; if (!in_str && c == '[') ++d; if (!in_str && c == ']') --d; }
      return d;
    };
    while (balance(val) > 0 && li + 1 < lines.size()) val += " " + trim(strip_comment(lines[++li]));
    auto parts = split_key(line.substr(0, eq));
    Json* t = cur;
    for (size_t i = 0; i + 1 < parts.size(); ++i) t = descend(t, parts[i]);
    if (t->has(parts.back())) throw TomlError("line " + std::to_string(line_no) + ": duplicate key `" + parts.back() + "`");
    t->set(parts.back(), parse_value(val, line_no));
  }
  return root;
}

}  // namespace skein
