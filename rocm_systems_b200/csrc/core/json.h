// A small JSON reader (objects, arrays, strings, numbers, true/false/null) for the tuning
// table and schedule files. Header-only; no external dependency.
#pragma once

#include <stdlib.h>
#include <string.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b200 {

struct JsonValue {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<JsonValue> arr;
  std::map<std::string, JsonValue> obj;
  const JsonValue* get(const std::string& k) const {
    auto it = obj.find(k);
    return it == obj.end() ? nullptr : &it->second;
  }
  double numberOr(const std::string& k, double d) const {
    const JsonValue* v = get(k);
    return v && v->kind == Number ? v->num : d;
  }
  std::string stringOr(const std::string& k, const std::string& d) const {
    const JsonValue* v = get(k);
    return v && v->kind == String ? v->str : d;
  }
};

class JsonParser {
 public:
  explicit JsonParser(const std::string& s) : s_(s) {}
  bool parse(JsonValue* out) {
    skip();
    if (!value(out)) return false;
    skip();
    return p_ == s_.size();
  }

 private:
  void skip() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) p_++; }
  bool lit(const char* w) {
    size_t n = strlen(w);
    if (s_.compare(p_, n, w) == 0) { p_ += n; return true; }
    return false;
  }
  // Containers nest at most kMaxDepth deep: the parser recurses once per level and the text is a user's file.
  static constexpr int kMaxDepth = 64;
  struct Level {
    int& d;
    explicit Level(int& depth) : d(depth) { d++; }
    ~Level() { d--; }
  };
  bool value(JsonValue* v) {
    if (p_ >= s_.size()) return false;
    Level level(depth_);
    if (depth_ > kMaxDepth) return false;
    char c = s_[p_];
    if (c == '{') {
      v->kind = JsonValue::Object;
      p_++;
      skip();
      if (p_ < s_.size() && s_[p_] == '}') { p_++; return true; }
      while (true) {
        skip();
        JsonValue k;
        if (!string(&k.str)) return false;
        skip();
        if (p_ >= s_.size() || s_[p_] != ':') return false;
        p_++;
        skip();
        JsonValue x;
        if (!value(&x)) return false;
        v->obj[k.str] = std::move(x);
        skip();
        if (p_ < s_.size() && s_[p_] == ',') { p_++; continue; }
        if (p_ < s_.size() && s_[p_] == '}') { p_++; return true; }
        return false;
      }
    }
    if (c == '[') {
      v->kind = JsonValue::Array;
      p_++;
      skip();
      if (p_ < s_.size() && s_[p_] == ']') { p_++; return true; }
      while (true) {
        skip();
        JsonValue x;
        if (!value(&x)) return false;
        v->arr.push_back(std::move(x));
        skip();
        if (p_ < s_.size() && s_[p_] == ',') { p_++; continue; }
        if (p_ < s_.size() && s_[p_] == ']') { p_++; return true; }
        return false;
      }
    }
    if (c == '"') { v->kind = JsonValue::String; return string(&v->str); }
    if (lit("true")) { v->kind = JsonValue::Bool; v->b = true; return true; }
    if (lit("false")) { v->kind = JsonValue::Bool; v->b = false; return true; }
    if (lit("null")) { v->kind = JsonValue::Null; return true; }
    char* end = nullptr;
    double d = strtod(s_.c_str() + p_, &end);
    if (end == s_.c_str() + p_) return false;
    p_ = end - s_.c_str();
    v->kind = JsonValue::Number;
    v->num = d;
    return true;
  }
  bool string(std::string* out) {
    if (p_ >= s_.size() || s_[p_] != '"') return false;
    p_++;
    out->clear();
    while (p_ < s_.size() && s_[p_] != '"') {
      if (s_[p_] == '\\' && p_ + 1 < s_.size()) {
        p_++;
        char e = s_[p_];
        out->push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e);
      } else {
        out->push_back(s_[p_]);
      }
      p_++;
    }
    if (p_ >= s_.size()) return false;
    p_++;
    return true;
  }
  const std::string& s_;
  size_t p_ = 0;
  int depth_ = 0;
};

}  // namespace b200
