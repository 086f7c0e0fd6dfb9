// Minimal JSON reader for the flat configuration objects the runtime accepts
// ({"key": number | "string" | true | false, ...}; nested values are skipped).  The reference
// passes the same kind of flat JSON strings to its KV engines and to its cache controller
// (src/storage/kv_engine/base_kv.h:14-17, src/framework/pytorch/kg_controller.h:58-83).
#pragma once
#include <cstdlib>
#include <map>
#include <string>

namespace rs {

class JsonLite {
 public:
  explicit JsonLite(const std::string& text) { parse(text); }
  bool ok() const { return ok_; }
  bool has(const std::string& k) const { return kv_.count(k) != 0; }
  std::string str(const std::string& k, const std::string& dflt = "") const {
    auto it = kv_.find(k);
    return it == kv_.end() ? dflt : it->second;
  }
  double num(const std::string& k, double dflt = 0) const {
    auto it = kv_.find(k);
    if (it == kv_.end()) return dflt;
    if (it->second == "true") return 1;
    if (it->second == "false") return 0;
    char* e = nullptr;
    const double v = std::strtod(it->second.c_str(), &e);
    return e == it->second.c_str() ? dflt : v;
  }
  long long i64(const std::string& k, long long dflt = 0) const { return static_cast<long long>(num(k, static_cast<double>(dflt))); }
  const std::map<std::string, std::string>& items() const { return kv_; }

 private:
  void skip_ws(const std::string& s, size_t& i) {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  bool parse_string(const std::string& s, size_t& i, std::string* out) {
    if (i >= s.size() || s[i] != '"') return false;
    ++i;
    out->clear();
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) {
        ++i;
        switch (s[i]) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          default: out->push_back(s[i]);
        }
      } else {
        out->push_back(s[i]);
      }
      ++i;
    }
    if (i >= s.size()) return false;
    ++i;
    return true;
  }
  // Skips a nested object/array, returns its raw text.
  bool skip_nested(const std::string& s, size_t& i, std::string* raw) {
    const size_t b = i;
    int depth = 0;
    bool in_str = false;
    for (; i < s.size(); ++i) {
      const char c = s[i];
      if (in_str) {
        if (c == '\\') ++i;
        else if (c == '"') in_str = false;
        continue;
      }
      if (c == '"') in_str = true;
      else if (c == '{' || c == '[') ++depth;
      else if (c == '}' || c == ']') {
        if (--depth == 0) { ++i; *raw = s.substr(b, i - b); return true; }
      }
    }
    return false;
  }
  void parse(const std::string& s) {
    size_t i = 0;
    skip_ws(s, i);
    if (i >= s.size() || s[i] != '{') { ok_ = s.find_first_not_of(" \n\t\r") == std::string::npos; return; }
    ++i;
    while (true) {
      skip_ws(s, i);
      if (i < s.size() && s[i] == '}') { ok_ = true; return; }
      std::string key, val;
      if (!parse_string(s, i, &key)) return;
      skip_ws(s, i);
      if (i >= s.size() || s[i] != ':') return;
      ++i;
      skip_ws(s, i);
      if (i >= s.size()) return;
      if (s[i] == '"') {
        if (!parse_string(s, i, &val)) return;
      } else if (s[i] == '{' || s[i] == '[') {
        if (!skip_nested(s, i, &val)) return;
      } else {
        const size_t b = i;
        while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ' ' && s[i] != '\n') ++i;
        val = s.substr(b, i - b);
      }
      kv_[key] = val;
      skip_ws(s, i);
      if (i < s.size() && s[i] == ',') { ++i; continue; }
      if (i < s.size() && s[i] == '}') { ok_ = true; return; }
      return;
    }
  }
  std::map<std::string, std::string> kv_;
  bool ok_ = false;
};

}  // namespace rs
