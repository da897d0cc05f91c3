// Minimal JSON reader for the model descriptor (objects, arrays, strings,
// numbers, true/false/null). Header-only, no dependencies.
#pragma once

#include <stdlib.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace dyn {

struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::map<std::string, Json> obj;

  const Json* get(const std::string& k) const {
    if (kind != Obj) return nullptr;
    auto it = obj.find(k);
    return it == obj.end() ? nullptr : &it->second;
  }
  double number(const std::string& k, double dflt) const {
    const Json* j = get(k);
    if (!j) return dflt;
    if (j->kind == Num) return j->num;
    if (j->kind == Bool) return j->b ? 1 : 0;
    return dflt;
  }
  std::string string(const std::string& k, const std::string& dflt) const {
    const Json* j = get(k);
    return (j && j->kind == Str) ? j->str : dflt;
  }
};

class JsonParser {
 public:
  explicit JsonParser(const char* s) : p_(s) {}
  bool parse(Json* out, std::string* err) {
    if (!value(out, 0)) {
      *err = err_.empty() ? "malformed JSON" : err_;
      return false;
    }
    ws();
    if (*p_) {
      *err = "trailing characters after JSON document";
      return false;
    }
    return true;
  }

 private:
  const char* p_;
  std::string err_;
  void ws() {
    while (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r') p_++;
  }
  bool lit(const char* s) {
    const char* q = p_;
    while (*s) {
      if (*q++ != *s++) return false;
    }
    p_ = q;
    return true;
  }
  bool str(std::string* out) {
    if (*p_ != '"') return false;
    p_++;
    out->clear();
    while (*p_ && *p_ != '"') {
      if (*p_ == '\\') {
        p_++;
        switch (*p_) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {
            unsigned v = 0;
            for (int i = 1; i <= 4; i++) {
              char c = p_[i];
              if (!c) return false;
              v = v * 16 + (c <= '9' ? c - '0' : (c | 32) - 'a' + 10);
            }
            p_ += 4;
            out->push_back(v < 128 ? (char)v : '?');
          } break;
          case 0: return false;
          default: out->push_back(*p_);
        }
        p_++;
      } else {
        out->push_back(*p_++);
      }
    }
    if (*p_ != '"') return false;
    p_++;
    return true;
  }
  bool value(Json* out, int depth) {
    if (depth > 32) {
      err_ = "JSON nesting too deep";
      return false;
    }
    ws();
    if (*p_ == '{') {
      p_++;
      out->kind = Json::Obj;
      ws();
      if (*p_ == '}') {
        p_++;
        return true;
      }
      for (;;) {
        ws();
        std::string k;
        if (!str(&k)) return false;
        ws();
        if (*p_++ != ':') return false;
        Json v;
        if (!value(&v, depth + 1)) return false;
        out->obj.emplace(std::move(k), std::move(v));
        ws();
        if (*p_ == ',') {
          p_++;
          continue;
        }
        if (*p_ == '}') {
          p_++;
          return true;
        }
        return false;
      }
    }
    if (*p_ == '[') {
      p_++;
      out->kind = Json::Arr;
      ws();
      if (*p_ == ']') {
        p_++;
        return true;
      }
      for (;;) {
        Json v;
        if (!value(&v, depth + 1)) return false;
        out->arr.push_back(std::move(v));
        ws();
        if (*p_ == ',') {
          p_++;
          continue;
        }
        if (*p_ == ']') {
          p_++;
          return true;
        }
        return false;
      }
    }
    if (*p_ == '"') {
      out->kind = Json::Str;
      return str(&out->str);
    }
    if (lit("true")) {
      out->kind = Json::Bool;
      out->b = true;
      return true;
    }
    if (lit("false")) {
      out->kind = Json::Bool;
      out->b = false;
      return true;
    }
    if (lit("null")) {
      out->kind = Json::Null;
      return true;
    }
    char* end = nullptr;
    double d = strtod(p_, &end);
    if (end == p_) return false;
    p_ = end;
    out->kind = Json::Num;
    out->num = d;
    return true;
  }
};

}  // namespace dyn
