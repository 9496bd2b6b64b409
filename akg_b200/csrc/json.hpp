// Minimal JSON document model + recursive-descent parser for the fused-op
// description.  Accepts what nlohmann::json accepts for these files, plus the
// bare tokens NaN / Infinity / -Infinity that Python's json module emits.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace akgb {

struct JsonError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Json {
 public:
  enum Kind { Null, Bool, Number, String, Array, Object };
  Kind kind = Null;
  bool b = false;
  double num = 0.0;
  bool is_integer = false;
  int64_t inum = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;  // keeps file order

  bool is_null() const { return kind == Null; }
  bool is_bool() const { return kind == Bool; }
  bool is_number() const { return kind == Number; }
  bool is_string() const { return kind == String; }
  bool is_array() const { return kind == Array; }
  bool is_object() const { return kind == Object; }
  size_t size() const { return kind == Array ? arr.size() : kind == Object ? obj.size() : 0; }

  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json* find(const std::string& k) const {
    if (kind != Object) return nullptr;
    for (auto& kv : obj)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
  const Json& at(const std::string& k) const {
    const Json* p = find(k);
    if (!p) throw JsonError("missing key '" + k + "'");
    return *p;
  }
  const Json& operator[](size_t i) const {
    if (kind != Array || i >= arr.size()) throw JsonError("array index out of range");
    return arr[i];
  }
  const std::string& as_string() const {
    if (kind != String) throw JsonError("expected a string");
    return str;
  }
  double as_double() const {
    if (kind == Number) return num;
    if (kind == Bool) return b ? 1.0 : 0.0;
    throw JsonError("expected a number");
  }
  int64_t as_int() const {
    if (kind == Number) return is_integer ? inum : (int64_t)num;
    if (kind == Bool) return b ? 1 : 0;
    throw JsonError("expected an integer");
  }
  bool as_bool() const {
    if (kind == Bool) return b;
    if (kind == Number) return num != 0.0;
    throw JsonError("expected a bool");
  }
  std::vector<int64_t> as_int_list() const {
    std::vector<int64_t> v;
    if (kind == Number) {
      v.push_back(as_int());
      return v;
    }
    if (kind != Array) throw JsonError("expected a list of integers");
    for (auto& e : arr) v.push_back(e.as_int());
    return v;
  }

  static Json parse(const char* text, size_t len) {
    Parser p{text, text + len};
    p.skip_ws();
    Json j = p.value(0);
    p.skip_ws();
    if (p.cur != p.end) throw JsonError("trailing characters after JSON value");
    return j;
  }

 private:
  struct Parser {
    const char* cur;
    const char* end;
    void skip_ws() {
      while (cur < end && (*cur == ' ' || *cur == '\t' || *cur == '\n' || *cur == '\r')) ++cur;
    }
    bool lit(const char* s) {
      size_t n = std::char_traits<char>::length(s);
      if ((size_t)(end - cur) >= n && std::char_traits<char>::compare(cur, s, n) == 0) {
        cur += n;
        return true;
      }
      return false;
    }
    Json value(int depth) {
      if (depth > 200) throw JsonError("nesting too deep");
      if (cur >= end) throw JsonError("unexpected end of text");
      char c = *cur;
      Json j;
      if (c == '{') {
        ++cur;
        j.kind = Object;
        skip_ws();
        if (cur < end && *cur == '}') {
          ++cur;
          return j;
        }
        for (;;) {
          skip_ws();
          if (cur >= end || *cur != '"') throw JsonError("expected object key");
          std::string k = string_body();
          skip_ws();
          if (cur >= end || *cur != ':') throw JsonError("expected ':'");
          ++cur;
          skip_ws();
          j.obj.emplace_back(std::move(k), value(depth + 1));
          skip_ws();
          if (cur < end && *cur == ',') {
            ++cur;
            continue;
          }
          if (cur < end && *cur == '}') {
            ++cur;
            return j;
          }
          throw JsonError("expected ',' or '}'");
        }
      }
      if (c == '[') {
        ++cur;
        j.kind = Array;
        skip_ws();
        if (cur < end && *cur == ']') {
          ++cur;
          return j;
        }
        for (;;) {
          skip_ws();
          j.arr.push_back(value(depth + 1));
          skip_ws();
          if (cur < end && *cur == ',') {
            ++cur;
            continue;
          }
          if (cur < end && *cur == ']') {
            ++cur;
            return j;
          }
          throw JsonError("expected ',' or ']'");
        }
      }
      if (c == '"') {
        j.kind = String;
        j.str = string_body();
        return j;
      }
      if (lit("true")) {
        j.kind = Bool;
        j.b = true;
        return j;
      }
      if (lit("false")) {
        j.kind = Bool;
        j.b = false;
        return j;
      }
      if (lit("null")) return j;
      if (lit("NaN")) {
        j.kind = Number;
        j.num = std::nan("");
        return j;
      }
      if (lit("Infinity")) {
        j.kind = Number;
        j.num = INFINITY;
        return j;
      }
      if (lit("-Infinity")) {
        j.kind = Number;
        j.num = -INFINITY;
        return j;
      }
      if (c == '-' || (c >= '0' && c <= '9')) {
        const char* s = cur;
        bool integral = true;
        if (*cur == '-') ++cur;
        while (cur < end && ((*cur >= '0' && *cur <= '9') || *cur == '.' || *cur == 'e' || *cur == 'E' ||
                             *cur == '+' || *cur == '-')) {
          if (*cur == '.' || *cur == 'e' || *cur == 'E') integral = false;
          ++cur;
        }
        std::string tok(s, cur);
        j.kind = Number;
        char* endp = nullptr;
        j.num = std::strtod(tok.c_str(), &endp);
        if (endp == tok.c_str() || *endp != '\0') throw JsonError("bad number '" + tok + "'");
        if (integral) {
          j.is_integer = true;
          j.inum = std::strtoll(tok.c_str(), nullptr, 10);
        }
        return j;
      }
      throw JsonError(std::string("unexpected character '") + c + "'");
    }
    std::string string_body() {
      ++cur;  // opening quote
      std::string out;
      while (cur < end && *cur != '"') {
        char c = *cur++;
        if (c != '\\') {
          out.push_back(c);
          continue;
        }
        if (cur >= end) break;
        char e = *cur++;
        switch (e) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            if (end - cur < 4) throw JsonError("bad \\u escape");
            unsigned cp = (unsigned)std::strtoul(std::string(cur, cur + 4).c_str(), nullptr, 16);
            cur += 4;
            if (cp < 0x80) out.push_back((char)cp);
            else if (cp < 0x800) {
              out.push_back((char)(0xC0 | (cp >> 6)));
              out.push_back((char)(0x80 | (cp & 0x3F)));
            } else {
              out.push_back((char)(0xE0 | (cp >> 12)));
              out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
              out.push_back((char)(0x80 | (cp & 0x3F)));
            }
            break;
          }
          default: out.push_back(e);
        }
      }
      if (cur >= end) throw JsonError("unterminated string");
      ++cur;  // closing quote
      return out;
    }
  };
};

}  // namespace akgb
