// A small JSON value with a strict parser and a serialiser: just enough for the IntentIR
// wire format (objects, arrays, strings, numbers, booleans, null).  Object member order is
// preserved, which keeps `tensors` and `ops` in the order the graph declared them.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace ib200 {

struct Json {
  enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
  bool b = false;
  double num = 0.0;
  bool integral = false;  // the literal had no fraction / exponent
  std::string s;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  Json() = default;
  static Json boolean(bool v) { Json j; j.type = Bool; j.b = v; return j; }
  static Json number(double v) { Json j; j.type = Num; j.num = v; j.integral = std::floor(v) == v && std::fabs(v) < 9e15; return j; }
  static Json string(std::string v) { Json j; j.type = Str; j.s = std::move(v); return j; }
  static Json array() { Json j; j.type = Arr; return j; }
  static Json object() { Json j; j.type = Obj; return j; }

  bool is_null() const { return type == Null; }
  bool is_num() const { return type == Num; }
  bool is_str() const { return type == Str; }
  bool is_arr() const { return type == Arr; }
  bool is_obj() const { return type == Obj; }
  bool is_int() const { return type == Num && integral; }
  int64_t as_int() const { return (int64_t)num; }

  const Json* find(const std::string& key) const {
    if (type != Obj) return nullptr;
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  Json& set(const std::string& key, Json v) {
    for (auto& kv : obj)
      if (kv.first == key) { kv.second = std::move(v); return kv.second; }
    obj.emplace_back(key, std::move(v));
    return obj.back().second;
  }
  Json& push(Json v) { arr.push_back(std::move(v)); return arr.back(); }

  // ---- serialise -----------------------------------------------------------------------
  static void escape(const std::string& in, std::string& out) {
    out.push_back('"');
    for (unsigned char c : in) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        default:
          if (c < 0x20) { char buf[8]; std::snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
          else out.push_back((char)c);
      }
    }
    out.push_back('"');
  }
  void dump(std::string& out) const {
    switch (type) {
      case Null: out += "null"; break;
      case Bool: out += b ? "true" : "false"; break;
      case Num: {
        char buf[40];
        if (integral) std::snprintf(buf, sizeof buf, "%lld", (long long)num);
        else if (std::isfinite(num)) std::snprintf(buf, sizeof buf, "%.17g", num);
        else std::snprintf(buf, sizeof buf, "%s", std::isnan(num) ? "NaN" : num > 0 ? "Infinity" : "-Infinity");  // as read above
        out += buf;
        break;
      }
      case Str: escape(s, out); break;
      case Arr:
        out.push_back('[');
        for (size_t i = 0; i < arr.size(); ++i) { if (i) out.push_back(','); arr[i].dump(out); }
        out.push_back(']');
        break;
      case Obj:
        out.push_back('{');
        for (size_t i = 0; i < obj.size(); ++i) {
          if (i) out.push_back(',');
          escape(obj[i].first, out);
          out.push_back(':');
          obj[i].second.dump(out);
        }
        out.push_back('}');
        break;
    }
  }
  std::string dump() const { std::string o; dump(o); return o; }

  // ---- parse ------------------------------------------------------------------------------
  static Json parse(const char* text) {
    if (!text) throw std::runtime_error("json: null text");
    const char* p = text;
    Json v = parse_value(p, 0);
    skip_ws(p);
    if (*p) throw std::runtime_error("json: trailing characters");
    return v;
  }

 private:
  static void skip_ws(const char*& p) { while (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r') ++p; }
  static void append_utf8(unsigned cp, std::string& out) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  }
  static unsigned hex4(const char*& p) {
    unsigned v = 0;
    for (int i = 0; i < 4; ++i, ++p) {
      char c = *p;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else throw std::runtime_error("json: bad \\u escape");
    }
    return v;
  }
  static std::string parse_string(const char*& p) {
    std::string out;
    ++p;  // opening quote
    while (*p && *p != '"') {
      if (*p == '\\') {
        ++p;
        switch (*p) {
          case '"': out.push_back('"'); ++p; break;
          case '\\': out.push_back('\\'); ++p; break;
          case '/': out.push_back('/'); ++p; break;
          case 'b': out.push_back('\b'); ++p; break;
          case 'f': out.push_back('\f'); ++p; break;
          case 'n': out.push_back('\n'); ++p; break;
          case 'r': out.push_back('\r'); ++p; break;
          case 't': out.push_back('\t'); ++p; break;
          case 'u': {
            ++p;
            unsigned cp = hex4(p);
            if (cp >= 0xD800 && cp < 0xDC00 && p[0] == '\\' && p[1] == 'u') {
              p += 2;
              unsigned lo = hex4(p);
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            append_utf8(cp, out);
            break;
          }
          default: throw std::runtime_error("json: bad escape");
        }
      } else {
        out.push_back(*p++);
      }
    }
    if (*p != '"') throw std::runtime_error("json: unterminated string");
    ++p;
    return out;
  }
  static Json parse_value(const char*& p, int depth) {
    if (depth > 200) throw std::runtime_error("json: nesting too deep");
    skip_ws(p);
    Json v;
    if (*p == '{') {
      v.type = Obj;
      ++p;
      skip_ws(p);
      if (*p == '}') { ++p; return v; }
      for (;;) {
        skip_ws(p);
        if (*p != '"') throw std::runtime_error("json: expected a member name");
        std::string key = parse_string(p);
        skip_ws(p);
        if (*p != ':') throw std::runtime_error("json: expected ':'");
        ++p;
        v.obj.emplace_back(std::move(key), parse_value(p, depth + 1));
        skip_ws(p);
        if (*p == ',') { ++p; continue; }
        if (*p == '}') { ++p; return v; }
        throw std::runtime_error("json: expected ',' or '}'");
      }
    }
    if (*p == '[') {
      v.type = Arr;
      ++p;
      skip_ws(p);
      if (*p == ']') { ++p; return v; }
      for (;;) {
        v.arr.push_back(parse_value(p, depth + 1));
        skip_ws(p);
        if (*p == ',') { ++p; continue; }
        if (*p == ']') { ++p; return v; }
        throw std::runtime_error("json: expected ',' or ']'");
      }
    }
    if (*p == '"') { v.type = Str; v.s = parse_string(p); return v; }
    if (!std::strncmp(p, "true", 4)) { p += 4; return boolean(true); }
    if (!std::strncmp(p, "false", 5)) { p += 5; return boolean(false); }
    if (!std::strncmp(p, "null", 4)) { p += 4; return v; }
    if (!std::strncmp(p, "NaN", 3)) { p += 3; v.type = Num; v.num = NAN; return v; }  // Python's json.dumps emits these
    if (!std::strncmp(p, "Infinity", 8)) { p += 8; v.type = Num; v.num = INFINITY; return v; }
    if (!std::strncmp(p, "-Infinity", 9)) { p += 9; v.type = Num; v.num = -INFINITY; return v; }
    if (*p == '-' || (*p >= '0' && *p <= '9')) {
      char* end = nullptr;
      v.type = Num;
      v.num = std::strtod(p, &end);
      if (end == p) throw std::runtime_error("json: bad number");
      v.integral = true;
      for (const char* q = p; q < end; ++q)
        if (*q == '.' || *q == 'e' || *q == 'E') v.integral = false;
      p = end;
      return v;
    }
    throw std::runtime_error("json: unexpected character");
  }
};

}  // namespace ib200
