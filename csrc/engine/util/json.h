// Minimal JSON value, parser and serialiser (RFC 8259) for config.json, tokenizer.json,
// the OpenAI protocol and the chat entry points of the C ABI. Header-only, no dependencies.
// Object key order is preserved (chat templates and schemas care about it).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace b200 {

class Json {
 public:
  enum Type { kNull, kBool, kNumber, kString, kArray, kObject };
  using Array = std::vector<Json>;
  using Object = std::vector<std::pair<std::string, Json>>;

  Json() = default;
  Json(std::nullptr_t) {}
  Json(bool b) : type_(kBool), b_(b) {}
  Json(int v) : type_(kNumber), n_(v), is_int_(true) {}
  Json(int64_t v) : type_(kNumber), n_((double)v), is_int_(true) {}
  Json(double v) : type_(kNumber), n_(v) {}
  Json(const char* s) : type_(kString), s_(s) {}
  Json(std::string s) : type_(kString), s_(std::move(s)) {}
  static Json array() { Json j; j.type_ = kArray; return j; }
  static Json object() { Json j; j.type_ = kObject; return j; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == kNull; }
  bool is_bool() const { return type_ == kBool; }
  bool is_number() const { return type_ == kNumber; }
  bool is_string() const { return type_ == kString; }
  bool is_array() const { return type_ == kArray; }
  bool is_object() const { return type_ == kObject; }

  bool as_bool(bool d = false) const { return type_ == kBool ? b_ : d; }
  double as_double(double d = 0) const { return type_ == kNumber ? n_ : d; }
  int64_t as_int(int64_t d = 0) const { return type_ == kNumber ? (int64_t)n_ : d; }
  const std::string& as_string() const {
    static const std::string kEmpty;
    return type_ == kString ? s_ : kEmpty;
  }
  const Array& items() const { static const Array e; return type_ == kArray ? a_ : e; }
  Array& items() { if (type_ != kArray) { *this = array(); } return a_; }
  const Object& members() const { static const Object e; return type_ == kObject ? o_ : e; }
  size_t size() const { return type_ == kArray ? a_.size() : type_ == kObject ? o_.size() : 0; }

  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json* find(const std::string& k) const {
    if (type_ != kObject) return nullptr;
    for (auto& kv : o_) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  const Json& operator[](const std::string& k) const {
    static const Json kNullJson;
    const Json* p = find(k);
    return p ? *p : kNullJson;
  }
  Json& operator[](const std::string& k) {
    if (type_ != kObject) *this = object();
    for (auto& kv : o_) if (kv.first == k) return kv.second;
    o_.emplace_back(k, Json());
    return o_.back().second;
  }
  const Json& operator[](size_t i) const {
    static const Json kNullJson;
    return (type_ == kArray && i < a_.size()) ? a_[i] : kNullJson;
  }
  void push_back(Json v) { if (type_ != kArray) *this = array(); a_.push_back(std::move(v)); }
  void erase(const std::string& k) {
    if (type_ != kObject) return;
    for (size_t i = 0; i < o_.size(); ++i) if (o_[i].first == k) { o_.erase(o_.begin() + i); return; }
  }

  // ------------------------------------------------------------------ parse
  static Json parse(const std::string& text) {
    Parser p{text.data(), text.data() + text.size()};
    p.ws();
    Json v = p.value(0);
    p.ws();
    if (p.cur != p.end) p.fail("trailing characters");
    return v;
  }
  static bool try_parse(const std::string& text, Json* out, std::string* err = nullptr) {
    try { *out = parse(text); return true; }
    catch (const std::exception& e) { if (err) *err = e.what(); return false; }
  }

  // ------------------------------------------------------------------ dump
  std::string dump(int indent = -1) const { std::string s; write(s, indent, 0); return s; }

  static void escape(const std::string& in, std::string& out) {
    out.push_back('"');
    for (unsigned char c : in) {
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
          else out.push_back((char)c);
      }
    }
    out.push_back('"');
  }

 private:
  struct Parser {
    const char* cur; const char* end;
    [[noreturn]] void fail(const char* m) { throw std::runtime_error(std::string("JSON parse error: ") + m); }
    void ws() { while (cur < end && (*cur == ' ' || *cur == '\n' || *cur == '\t' || *cur == '\r')) ++cur; }
    Json value(int depth) {
      if (depth > 256) fail("nesting too deep");
      if (cur >= end) fail("unexpected end");
      switch (*cur) {
        case '{': return obj(depth);
        case '[': return arr(depth);
        case '"': return Json(str());
        case 't': lit("true"); return Json(true);
        case 'f': lit("false"); return Json(false);
        case 'n': lit("null"); return Json();
        default: return num();
      }
    }
    void lit(const char* w) { for (; *w; ++w, ++cur) if (cur >= end || *cur != *w) fail("bad literal"); }
    Json num() {
      const char* s = cur;
      bool is_int = true;
      if (cur < end && *cur == '-') ++cur;
      if (cur >= end || !(*cur >= '0' && *cur <= '9')) fail("bad number");
      while (cur < end && *cur >= '0' && *cur <= '9') ++cur;
      if (cur < end && *cur == '.') { is_int = false; ++cur; while (cur < end && *cur >= '0' && *cur <= '9') ++cur; }
      if (cur < end && (*cur == 'e' || *cur == 'E')) {
        is_int = false; ++cur;
        if (cur < end && (*cur == '+' || *cur == '-')) ++cur;
        while (cur < end && *cur >= '0' && *cur <= '9') ++cur;
      }
      Json j(std::strtod(std::string(s, cur).c_str(), nullptr));
      j.is_int_ = is_int;
      return j;
    }
    static void utf8(uint32_t cp, std::string& o) {
      if (cp < 0x80) o.push_back((char)cp);
      else if (cp < 0x800) { o.push_back((char)(0xC0 | (cp >> 6))); o.push_back((char)(0x80 | (cp & 63))); }
      else if (cp < 0x10000) { o.push_back((char)(0xE0 | (cp >> 12))); o.push_back((char)(0x80 | ((cp >> 6) & 63))); o.push_back((char)(0x80 | (cp & 63))); }
      else { o.push_back((char)(0xF0 | (cp >> 18))); o.push_back((char)(0x80 | ((cp >> 12) & 63))); o.push_back((char)(0x80 | ((cp >> 6) & 63))); o.push_back((char)(0x80 | (cp & 63))); }
    }
    uint32_t hex4() {
      if (end - cur < 4) fail("bad \\u escape");
      uint32_t v = 0;
      for (int i = 0; i < 4; ++i, ++cur) {
        char c = *cur; v <<= 4;
        if (c >= '0' && c <= '9') v |= c - '0';
        else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
        else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
        else fail("bad \\u escape");
      }
      return v;
    }
    std::string str() {
      ++cur;
      std::string o;
      while (true) {
        if (cur >= end) fail("unterminated string");
        char c = *cur++;
        if (c == '"') break;
        if (c == '\\') {
          if (cur >= end) fail("bad escape");
          char e = *cur++;
          switch (e) {
            case '"': o.push_back('"'); break; case '\\': o.push_back('\\'); break;
            case '/': o.push_back('/'); break; case 'b': o.push_back('\b'); break;
            case 'f': o.push_back('\f'); break; case 'n': o.push_back('\n'); break;
            case 'r': o.push_back('\r'); break; case 't': o.push_back('\t'); break;
            case 'u': {
              uint32_t cp = hex4();
              if (cp >= 0xD800 && cp <= 0xDBFF && end - cur >= 6 && cur[0] == '\\' && cur[1] == 'u') {
                cur += 2;
                uint32_t lo = hex4();
                if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
              }
              utf8(cp, o);
              break;
            }
            default: fail("bad escape");
          }
        } else {
          o.push_back(c);
        }
      }
      return o;
    }
    Json arr(int depth) {
      ++cur;
      Json j = Json::array();
      ws();
      if (cur < end && *cur == ']') { ++cur; return j; }
      while (true) {
        ws();
        j.a_.push_back(value(depth + 1));
        ws();
        if (cur >= end) fail("unterminated array");
        if (*cur == ',') { ++cur; continue; }
        if (*cur == ']') { ++cur; break; }
        fail("expected , or ]");
      }
      return j;
    }
    Json obj(int depth) {
      ++cur;
      Json j = Json::object();
      ws();
      if (cur < end && *cur == '}') { ++cur; return j; }
      while (true) {
        ws();
        if (cur >= end || *cur != '"') fail("expected string key");
        std::string k = str();
        ws();
        if (cur >= end || *cur != ':') fail("expected :");
        ++cur;
        ws();
        j.o_.emplace_back(std::move(k), value(depth + 1));
        ws();
        if (cur >= end) fail("unterminated object");
        if (*cur == ',') { ++cur; continue; }
        if (*cur == '}') { ++cur; break; }
        fail("expected , or }");
      }
      return j;
    }
  };

  void write(std::string& s, int indent, int level) const {
    auto nl = [&](int lv) { if (indent >= 0) { s.push_back('\n'); s.append((size_t)indent * lv, ' '); } };
    switch (type_) {
      case kNull: s += "null"; break;
      case kBool: s += b_ ? "true" : "false"; break;
      case kNumber: {
        char b[40];
        if (is_int_ && std::fabs(n_) < 9e15) snprintf(b, sizeof b, "%lld", (long long)n_);
        else if (std::isfinite(n_)) snprintf(b, sizeof b, "%.17g", n_);
        else snprintf(b, sizeof b, "null");
        s += b;
        break;
      }
      case kString: escape(s_, s); break;
      case kArray:
        s.push_back('[');
        for (size_t i = 0; i < a_.size(); ++i) { if (i) s.push_back(','); nl(level + 1); a_[i].write(s, indent, level + 1); }
        if (!a_.empty()) nl(level);
        s.push_back(']');
        break;
      case kObject:
        s.push_back('{');
        for (size_t i = 0; i < o_.size(); ++i) {
          if (i) s.push_back(',');
          nl(level + 1);
          escape(o_[i].first, s);
          s.push_back(':');
          if (indent >= 0) s.push_back(' ');
          o_[i].second.write(s, indent, level + 1);
        }
        if (!o_.empty()) nl(level);
        s.push_back('}');
        break;
    }
  }

  Type type_ = kNull;
  bool b_ = false;
  double n_ = 0;
  bool is_int_ = false;
  std::string s_;
  Array a_;
  Object o_;
};

}  // namespace b200
