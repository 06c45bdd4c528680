// Minimal JSON value, parser and serialiser used by the host library (tokenizer.json, chat-template
// variables, protocol payloads). Object key order is preserved (templates iterate dictionaries in
// insertion order). The reference depends on nlohmann/json for the same jobs (deps/json submodule).
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace vh {

struct Json;
using JsonPtr = std::shared_ptr<Json>;

struct Json {
  enum Type { Null, Bool, Int, Float, String, Array, Object } type = Null;
  bool b = false;
  int64_t i = 0;
  double f = 0.0;
  std::string s;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  Json() {}
  static Json null() { return Json(); }
  static Json boolean(bool v) { Json j; j.type = Bool; j.b = v; return j; }
  static Json integer(int64_t v) { Json j; j.type = Int; j.i = v; return j; }
  static Json number(double v) { Json j; j.type = Float; j.f = v; return j; }
  static Json string(std::string v) { Json j; j.type = String; j.s = std::move(v); return j; }
  static Json array() { Json j; j.type = Array; return j; }
  static Json object() { Json j; j.type = Object; return j; }

  bool is_null() const { return type == Null; }
  bool is_string() const { return type == String; }
  bool is_number() const { return type == Int || type == Float; }
  bool is_array() const { return type == Array; }
  bool is_object() const { return type == Object; }
  double as_double() const { return type == Int ? (double)i : type == Float ? f : type == Bool ? (b ? 1 : 0) : 0.0; }
  int64_t as_int() const { return type == Int ? i : type == Float ? (int64_t)f : type == Bool ? (b ? 1 : 0) : 0; }

  const Json* find(const std::string& k) const {
    if (type != Object) return nullptr;
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  Json* find(const std::string& k) {
    if (type != Object) return nullptr;
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  Json& set(const std::string& k, Json v) {
    if (type != Object) { *this = object(); }
    for (auto& kv : obj) if (kv.first == k) { kv.second = std::move(v); return kv.second; }
    obj.emplace_back(k, std::move(v));
    return obj.back().second;
  }
  std::string get_string(const std::string& k, const std::string& d = "") const {
    const Json* p = find(k);
    return p && p->type == String ? p->s : d;
  }
};

inline void json_escape(const std::string& s, std::string& out, bool ascii_only = false) {
  out.push_back('"');
  for (size_t n = 0; n < s.size(); ++n) {
    unsigned char c = (unsigned char)s[n];
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      case '\b': out += "\\b"; break;
      case '\f': out += "\\f"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out.push_back((char)c);
        }
    }
  }
  (void)ascii_only;
  out.push_back('"');
}

inline void json_dump(const Json& j, std::string& out, int indent = -1, int depth = 0) {
  auto nl = [&](int d) {
    if (indent < 0) return;
    out.push_back('\n');
    out.append((size_t)(d * indent), ' ');
  };
  switch (j.type) {
    case Json::Null: out += "null"; break;
    case Json::Bool: out += j.b ? "true" : "false"; break;
    case Json::Int: out += std::to_string(j.i); break;
    case Json::Float: {
      char buf[40];
      if (j.f == (double)(int64_t)j.f && j.f > -1e15 && j.f < 1e15) snprintf(buf, sizeof buf, "%.1f", j.f);
      else snprintf(buf, sizeof buf, "%.17g", j.f);
      out += buf;
      break;
    }
    case Json::String: json_escape(j.s, out); break;
    case Json::Array:
      out.push_back('[');
      for (size_t n = 0; n < j.arr.size(); ++n) {
        if (n) out += indent < 0 ? ", " : ",";
        nl(depth + 1);
        json_dump(j.arr[n], out, indent, depth + 1);
      }
      if (!j.arr.empty()) nl(depth);
      out.push_back(']');
      break;
    case Json::Object:
      out.push_back('{');
      for (size_t n = 0; n < j.obj.size(); ++n) {
        if (n) out += indent < 0 ? ", " : ",";
        nl(depth + 1);
        json_escape(j.obj[n].first, out);
        out += ": ";
        json_dump(j.obj[n].second, out, indent, depth + 1);
      }
      if (!j.obj.empty()) nl(depth);
      out.push_back('}');
      break;
  }
}

class JsonParser {
 public:
  explicit JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}
  Json parse() {
    Json v = value();
    ws();
    if (p_ != end_) fail("trailing characters");
    return v;
  }

 private:
  const char* p_;
  const char* end_;
  [[noreturn]] void fail(const char* m) { throw std::runtime_error(std::string("json: ") + m); }
  void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
  static void utf8(uint32_t cp, std::string& out) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }
  uint32_t hex4() {
    if (end_ - p_ < 4) fail("bad \\u escape");
    uint32_t v = 0;
    for (int n = 0; n < 4; ++n) {
      char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad hex digit");
    }
    return v;
  }
  std::string str() {
    ++p_;  // opening quote
    std::string out;
    while (p_ < end_ && *p_ != '"') {
      char c = *p_++;
      if (c != '\\') { out.push_back(c); continue; }
      if (p_ >= end_) fail("bad escape");
      char e = *p_++;
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            uint32_t lo = hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(cp, out);
          break;
        }
        default: out.push_back(e);
      }
    }
    if (p_ >= end_) fail("unterminated string");
    ++p_;
    return out;
  }
  Json value() {
    ws();
    if (p_ >= end_) fail("unexpected end");
    char c = *p_;
    if (c == '{') {
      ++p_;
      Json o = Json::object();
      ws();
      if (p_ < end_ && *p_ == '}') { ++p_; return o; }
      for (;;) {
        ws();
        if (p_ >= end_ || *p_ != '"') fail("expected key");
        std::string k = str();
        ws();
        if (p_ >= end_ || *p_ != ':') fail("expected ':'");
        ++p_;
        o.obj.emplace_back(std::move(k), value());
        ws();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == '}') { ++p_; return o; }
        fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++p_;
      Json a = Json::array();
      ws();
      if (p_ < end_ && *p_ == ']') { ++p_; return a; }
      for (;;) {
        a.arr.push_back(value());
        ws();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == ']') { ++p_; return a; }
        fail("expected ',' or ']'");
      }
    }
    if (c == '"') return Json::string(str());
    if (c == 't' && end_ - p_ >= 4 && !memcmp(p_, "true", 4)) { p_ += 4; return Json::boolean(true); }
    if (c == 'f' && end_ - p_ >= 5 && !memcmp(p_, "false", 5)) { p_ += 5; return Json::boolean(false); }
    if (c == 'n' && end_ - p_ >= 4 && !memcmp(p_, "null", 4)) { p_ += 4; return Json::null(); }
    const char* s = p_;
    bool isf = false;
    if (p_ < end_ && (*p_ == '-' || *p_ == '+')) ++p_;
    while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '-' || *p_ == '+')) {
      if (*p_ == '.' || *p_ == 'e' || *p_ == 'E') isf = true;
      ++p_;
    }
    if (s == p_) fail("unexpected character");
    std::string num(s, p_);
    return isf ? Json::number(strtod(num.c_str(), nullptr)) : Json::integer(strtoll(num.c_str(), nullptr, 10));
  }
};

inline Json json_parse(const std::string& s) { return JsonParser(s.data(), s.size()).parse(); }

}  // namespace vh
