// json.hpp — a small JSON reader for model configuration files (objects, arrays, strings, numbers, true / false / null).
// Values are kept in a tree; look-ups return a null value for missing keys so that optional fields read naturally:
//   cfg["loop"]["times"].as_int(1)
#pragma once

#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace nvllm {
namespace json {

struct Value {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Value> arr;
  std::vector<std::pair<std::string, Value>> obj;

  bool is_null() const { return kind == Null; }
  bool is_object() const { return kind == Object; }
  bool is_array() const { return kind == Array; }
  bool has(const std::string& k) const {
    for (const auto& kv : obj) if (kv.first == k) return true;
    return false;
  }
  const Value& operator[](const std::string& k) const {
    static const Value none;
    for (const auto& kv : obj) if (kv.first == k) return kv.second;
    return none;
  }
  const Value& operator[](size_t i) const {
    static const Value none;
    return i < arr.size() ? arr[i] : none;
  }
  size_t size() const { return kind == Array ? arr.size() : obj.size(); }
  double as_double(double dflt = 0.0) const { return kind == Number ? num : (kind == Bool ? (b ? 1.0 : 0.0) : dflt); }
  int as_int(int dflt = 0) const { return kind == Number ? static_cast<int>(num) : (kind == Bool ? (b ? 1 : 0) : dflt); }
  std::string as_string(const std::string& dflt = "") const { return kind == String ? str : dflt; }
  // required fields: a message that names the key instead of a silent default
  double need_double(const char* what) const {
    if (kind != Number) throw std::invalid_argument(std::string("model config: missing number '") + what + "'");
    return num;
  }
  int need_int(const char* what) const { return static_cast<int>(need_double(what)); }
};

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}
  Value parse() {
    Value v = value();
    ws();
    if (p_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  [[noreturn]] void fail(const char* what) const {
    throw std::invalid_argument(std::string("JSON: ") + what + " at offset " + std::to_string(p_));
  }
  void ws() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) ++p_; }
  bool lit(const char* w) {
    size_t n = 0;
    while (w[n]) ++n;
    if (s_.compare(p_, n, w) == 0) { p_ += n; return true; }
    return false;
  }
  Value value() {
    ws();
    if (p_ >= s_.size()) fail("unexpected end");
    Value v;
    const char c = s_[p_];
    if (c == '{') {
      v.kind = Value::Object;
      ++p_; ws();
      if (p_ < s_.size() && s_[p_] == '}') { ++p_; return v; }
      for (;;) {
        ws();
        if (p_ >= s_.size() || s_[p_] != '"') fail("expected a key");
        std::string k = string();
        ws();
        if (p_ >= s_.size() || s_[p_] != ':') fail("expected ':'");
        ++p_;
        v.obj.emplace_back(std::move(k), value());
        ws();
        if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
        if (p_ < s_.size() && s_[p_] == '}') { ++p_; return v; }
        fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      v.kind = Value::Array;
      ++p_; ws();
      if (p_ < s_.size() && s_[p_] == ']') { ++p_; return v; }
      for (;;) {
        v.arr.push_back(value());
        ws();
        if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
        if (p_ < s_.size() && s_[p_] == ']') { ++p_; return v; }
        fail("expected ',' or ']'");
      }
    }
    if (c == '"') { v.kind = Value::String; v.str = string(); return v; }
    if (lit("true")) { v.kind = Value::Bool; v.b = true; return v; }
    if (lit("false")) { v.kind = Value::Bool; v.b = false; return v; }
    if (lit("null")) return v;
    if (lit("NaN")) { v.kind = Value::Number; v.num = std::strtod("nan", nullptr); return v; }
    if (lit("Infinity")) { v.kind = Value::Number; v.num = std::strtod("inf", nullptr); return v; }
    if (lit("-Infinity")) { v.kind = Value::Number; v.num = -std::strtod("inf", nullptr); return v; }
    char* end = nullptr;
    v.num = std::strtod(s_.c_str() + p_, &end);
    if (end == s_.c_str() + p_) fail("unexpected character");
    v.kind = Value::Number;
    p_ = static_cast<size_t>(end - s_.c_str());
    return v;
  }
  std::string string() {
    std::string out;
    ++p_;  // opening quote
    while (p_ < s_.size() && s_[p_] != '"') {
      char c = s_[p_++];
      if (c == '\\') {
        if (p_ >= s_.size()) fail("bad escape");
        const char e = s_[p_++];
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            if (p_ + 4 > s_.size()) fail("bad \\u escape");
            const unsigned cp = static_cast<unsigned>(std::strtoul(s_.substr(p_, 4).c_str(), nullptr, 16));
            p_ += 4;
            if (cp < 0x80) out += static_cast<char>(cp);
            else if (cp < 0x800) { out += static_cast<char>(0xC0 | (cp >> 6)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
            else { out += static_cast<char>(0xE0 | (cp >> 12)); out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
            break;
          }
          default: out += e;
        }
      } else {
        out += c;
      }
    }
    if (p_ >= s_.size()) fail("unterminated string");
    ++p_;
    return out;
  }
  const std::string& s_;
  size_t p_ = 0;
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

}  // namespace json
}  // namespace nvllm
