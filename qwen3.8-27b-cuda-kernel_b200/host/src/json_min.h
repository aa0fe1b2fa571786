// A small JSON reader: enough for .q38 headers and tuning tables (objects, arrays, strings with the
// common escapes, numbers, booleans, null). Object members keep their insertion order.
#pragma once

#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace qwen38::jsonmin {

struct Value {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Value> arr;
  std::vector<std::pair<std::string, Value>> obj;

  const Value* find(const std::string& key) const {
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const Value& at(const std::string& key) const {
    const Value* v = find(key);
    if (!v) throw std::runtime_error("json: missing key '" + key + "'");
    return *v;
  }
  bool has(const std::string& key) const { return find(key) != nullptr; }
  int64_t as_int() const {
    if (kind != Number) throw std::runtime_error("json: number expected");
    return int64_t(num);
  }
  double as_double() const {
    if (kind != Number) throw std::runtime_error("json: number expected");
    return num;
  }
  const std::string& as_string() const {
    if (kind != String) throw std::runtime_error("json: string expected");
    return str;
  }
  bool as_bool() const {
    if (kind != Bool) throw std::runtime_error("json: boolean expected");
    return b;
  }
};

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}
  Value parse() {
    Value v = value();
    ws();
    if (i_ != s_.size()) err("trailing characters");
    return v;
  }

 private:
  const std::string& s_;
  size_t i_ = 0;

  [[noreturn]] void err(const char* what) const {
    throw std::runtime_error(std::string("json: ") + what + " at offset " + std::to_string(i_));
  }
  void ws() {
    while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
  }
  bool eat(char c) {
    ws();
    if (i_ < s_.size() && s_[i_] == c) {
      ++i_;
      return true;
    }
    return false;
  }
  Value value() {
    ws();
    if (i_ >= s_.size()) err("unexpected end");
    const char c = s_[i_];
    Value v;
    if (c == '{') {
      ++i_;
      v.kind = Value::Object;
      if (eat('}')) return v;
      do {
        ws();
        std::string key = string();
        if (!eat(':')) err("':' expected");
        v.obj.emplace_back(std::move(key), value());
      } while (eat(','));
      if (!eat('}')) err("'}' expected");
    } else if (c == '[') {
      ++i_;
      v.kind = Value::Array;
      if (eat(']')) return v;
      do v.arr.push_back(value());
      while (eat(','));
      if (!eat(']')) err("']' expected");
    } else if (c == '"') {
      v.kind = Value::String;
      v.str = string();
    } else if (s_.compare(i_, 4, "true") == 0) {
      v.kind = Value::Bool;
      v.b = true;
      i_ += 4;
    } else if (s_.compare(i_, 5, "false") == 0) {
      v.kind = Value::Bool;
      i_ += 5;
    } else if (s_.compare(i_, 4, "null") == 0) {
      i_ += 4;
    } else {
      char* end = nullptr;
      v.num = std::strtod(s_.c_str() + i_, &end);
      if (end == s_.c_str() + i_) err("value expected");
      v.kind = Value::Number;
      i_ = size_t(end - s_.c_str());
    }
    return v;
  }
  std::string string() {
    if (i_ >= s_.size() || s_[i_] != '"') err("string expected");
    ++i_;
    std::string out;
    while (i_ < s_.size() && s_[i_] != '"') {
      char c = s_[i_++];
      if (c == '\\') {
        if (i_ >= s_.size()) err("bad escape");
        const char e = s_[i_++];
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            if (i_ + 4 > s_.size()) err("bad \\u escape");
            const unsigned cp = unsigned(std::strtoul(s_.substr(i_, 4).c_str(), nullptr, 16));
            i_ += 4;
            if (cp < 0x80) out += char(cp);
            else if (cp < 0x800) {
              out += char(0xC0 | (cp >> 6));
              out += char(0x80 | (cp & 0x3F));
            } else {
              out += char(0xE0 | (cp >> 12));
              out += char(0x80 | ((cp >> 6) & 0x3F));
              out += char(0x80 | (cp & 0x3F));
            }
            break;
          }
          default: out += e;
        }
      } else {
        out += c;
      }
    }
    if (i_ >= s_.size()) err("unterminated string");
    ++i_;
    return out;
  }
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

}  // namespace qwen38::jsonmin
