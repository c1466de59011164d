// Minimal JSON value, parser and writer used by the host-side runtime (config.json, safetensors headers, the
// OpenAI protocol).  The writer can reproduce Python's json.dumps default formatting (", " / ": " separators,
// ensure_ascii), which the reference keeps byte-compatible with its Python server (crates/agens-server/src/pyjson.rs).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace b2 {

class Json {
 public:
  enum Type { Null, Bool, Int, Double, String, Array, Object };
  using Arr = std::vector<Json>;
  using Obj = std::vector<std::pair<std::string, Json>>;   // insertion order is kept (Python dict semantics)

  Json() : t_(Null) {}
  Json(std::nullptr_t) : t_(Null) {}
  Json(bool b) : t_(Bool), b_(b) {}
  Json(int v) : t_(Int), i_(v) {}
  Json(long v) : t_(Int), i_(v) {}
  Json(long long v) : t_(Int), i_(v) {}
  Json(unsigned v) : t_(Int), i_(v) {}
  Json(unsigned long v) : t_(Int), i_((long long)v) {}
  Json(double v) : t_(Double), d_(v) {}
  // An integer beyond 64 bits that only survives as a double: written with all its digits, as an integer
  static Json big_integer(double v) { Json j(v); j.int_like_ = true; return j; }
  Json(const char* s) : t_(String), s_(s) {}
  Json(std::string s) : t_(String), s_(std::move(s)) {}
  static Json array() { Json j; j.t_ = Array; return j; }
  static Json object() { Json j; j.t_ = Object; return j; }

  Type type() const { return t_; }
  bool is_null() const { return t_ == Null; }
  bool is_bool() const { return t_ == Bool; }
  bool is_int() const { return t_ == Int; }
  bool is_number() const { return t_ == Int || t_ == Double; }
  bool is_string() const { return t_ == String; }
  bool is_array() const { return t_ == Array; }
  bool is_object() const { return t_ == Object; }

  bool as_bool() const { return b_; }
  long long as_int() const {                                  // a double saturates (the plain cast is undefined out of range)
    if (t_ != Double) return i_;
    if (!(d_ == d_)) return 0;
    if (d_ >= 9.2e18) return 9223372036854775807ll;
    if (d_ <= -9.2e18) return -9223372036854775807ll - 1;
    return (long long)d_;
  }
  double as_double() const { return t_ == Int ? (double)i_ : d_; }
  const std::string& as_string() const { return s_; }
  const Arr& items() const { return a_; }
  Arr& items() { return a_; }
  const Obj& members() const { return o_; }
  Obj& members() { return o_; }

  size_t size() const { return t_ == Array ? a_.size() : (t_ == Object ? o_.size() : 0); }
  void push_back(Json v) { a_.push_back(std::move(v)); }
  const Json& operator[](size_t i) const {
    if (i >= a_.size()) throw std::runtime_error("JSON array index out of range");
    return a_[i];
  }

  const Json* find(const std::string& k) const {
    if (t_ != Object) return nullptr;
    for (auto& kv : o_) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json& at(const std::string& k) const {
    const Json* p = find(k);
    if (!p) throw std::runtime_error("missing key: " + k);
    return *p;
  }
  Json& set(const std::string& k, Json v) {
    for (auto& kv : o_) if (kv.first == k) { kv.second = std::move(v); return kv.second; }
    o_.emplace_back(k, std::move(v));
    return o_.back().second;
  }
  // typed getters with defaults
  long long get_int(const std::string& k, long long d) const { auto p = find(k); return p && p->is_number() ? p->as_int() : d; }
  double get_double(const std::string& k, double d) const { auto p = find(k); return p && p->is_number() ? p->as_double() : d; }
  bool get_bool(const std::string& k, bool d) const { auto p = find(k); return p && p->is_bool() ? p->as_bool() : d; }
  std::string get_string(const std::string& k, const std::string& d) const { auto p = find(k); return p && p->is_string() ? p->as_string() : d; }

  // ---- parsing ----
  static Json parse(const std::string& text) {
    size_t pos = 0;
    Json v = parse_value(text, pos, 0);
    skip_ws(text, pos);
    if (pos != text.size()) throw std::runtime_error("trailing characters after JSON value");
    return v;
  }

  // ---- writing ----
  struct Style {
    bool python;       // ", " and ": " separators
    bool ensure_ascii; // \uXXXX for non-ASCII
  };
  std::string dump() const { std::string out; write(out, Style{false, false}); return out; }
  std::string dump(Style st) const { std::string out; write(out, st); return out; }
  std::string dump_python() const { return dump(Style{true, true}); }

 private:
  Type t_;
  bool b_ = false;
  long long i_ = 0;
  double d_ = 0;
  bool int_like_ = false;
  std::string s_;
  Arr a_;
  Obj o_;

  static void skip_ws(const std::string& s, size_t& p) {
    while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\t' || s[p] == '\r')) ++p;
  }
  static void append_utf8(std::string& out, unsigned cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  }
  static unsigned hex4(const std::string& s, size_t p) {
    if (p + 4 > s.size()) throw std::runtime_error("bad \\u escape");
    unsigned v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = s[p + i];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else throw std::runtime_error("bad \\u escape");
    }
    return v;
  }
  static std::string parse_string(const std::string& s, size_t& p) {
    std::string out;
    ++p;  // opening quote
    while (true) {
      if (p >= s.size()) throw std::runtime_error("unterminated string");
      char c = s[p++];
      if (c == '"') break;
      if (c != '\\') { out.push_back(c); continue; }
      if (p >= s.size()) throw std::runtime_error("bad escape");
      char e = s[p++];
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          unsigned cp = hex4(s, p); p += 4;
          if (cp >= 0xD800 && cp < 0xDC00 && p + 6 <= s.size() && s[p] == '\\' && s[p + 1] == 'u') {
            unsigned lo = hex4(s, p + 2);
            if (lo >= 0xDC00 && lo < 0xE000) { cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00); p += 6; }
          }
          append_utf8(out, cp);
          break;
        }
        default: throw std::runtime_error("bad escape");
      }
    }
    return out;
  }
  static Json parse_value(const std::string& s, size_t& p, int depth) {
    if (depth > 200) throw std::runtime_error("JSON nested too deeply");
    skip_ws(s, p);
    if (p >= s.size()) throw std::runtime_error("unexpected end of JSON");
    char c = s[p];
    if (c == '{') {
      Json o = object();
      ++p; skip_ws(s, p);
      if (p < s.size() && s[p] == '}') { ++p; return o; }
      while (true) {
        skip_ws(s, p);
        if (p >= s.size() || s[p] != '"') throw std::runtime_error("expected object key");
        std::string k = parse_string(s, p);
        skip_ws(s, p);
        if (p >= s.size() || s[p] != ':') throw std::runtime_error("expected ':'");
        ++p;
        o.set(k, parse_value(s, p, depth + 1));
        skip_ws(s, p);
        if (p < s.size() && s[p] == ',') { ++p; continue; }
        if (p < s.size() && s[p] == '}') { ++p; break; }
        throw std::runtime_error("expected ',' or '}'");
      }
      return o;
    }
    if (c == '[') {
      Json a = array();
      ++p; skip_ws(s, p);
      if (p < s.size() && s[p] == ']') { ++p; return a; }
      while (true) {
        a.push_back(parse_value(s, p, depth + 1));
        skip_ws(s, p);
        if (p < s.size() && s[p] == ',') { ++p; continue; }
        if (p < s.size() && s[p] == ']') { ++p; break; }
        throw std::runtime_error("expected ',' or ']'");
      }
      return a;
    }
    if (c == '"') return Json(parse_string(s, p));
    if (s.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
    if (s.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
    if (s.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    // number
    size_t q = p;
    bool is_float = false;
    if (q < s.size() && (s[q] == '-' || s[q] == '+')) ++q;
    while (q < s.size() && ((s[q] >= '0' && s[q] <= '9') || s[q] == '.' || s[q] == 'e' || s[q] == 'E' || s[q] == '-' || s[q] == '+')) {
      if (s[q] == '.' || s[q] == 'e' || s[q] == 'E') is_float = true;
      ++q;
    }
    if (q == p) throw std::runtime_error(std::string("unexpected character in JSON: ") + c);
    std::string num = s.substr(p, q - p);
    p = q;
    if (is_float) return Json(std::strtod(num.c_str(), nullptr));
    errno = 0;
    long long v = std::strtoll(num.c_str(), nullptr, 10);
    if (errno == ERANGE) {
      // an integer beyond 64 bits: the value survives as a double, the digits as written (Python keeps such integers exact)
      Json j = Json::big_integer(std::strtod(num.c_str(), nullptr));
      j.s_ = num;
      return j;
    }
    return Json(v);
  }

  static void write_string(std::string& out, const std::string& s, bool ensure_ascii) {
    out.push_back('"');
    for (size_t i = 0; i < s.size(); ++i) {
      unsigned char c = (unsigned char)s[i];
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
          else if (c < 0x80 || !ensure_ascii) out.push_back((char)c);
          else {
            // decode one UTF-8 sequence, emit \uXXXX (with surrogates)
            unsigned cp = 0; int n = 0;
            if ((c & 0xE0) == 0xC0) { cp = c & 0x1F; n = 1; }
            else if ((c & 0xF0) == 0xE0) { cp = c & 0x0F; n = 2; }
            else if ((c & 0xF8) == 0xF0) { cp = c & 0x07; n = 3; }
            else { cp = 0xFFFD; n = 0; }
            for (int k = 0; k < n && i + 1 < s.size(); ++k) cp = (cp << 6) | ((unsigned char)s[++i] & 0x3F);
            char b[16];
            if (cp >= 0x10000) {
              unsigned v = cp - 0x10000;
              snprintf(b, sizeof b, "\\u%04x\\u%04x", 0xD800 + (v >> 10), 0xDC00 + (v & 0x3FF));
            } else snprintf(b, sizeof b, "\\u%04x", cp);
            out += b;
          }
      }
    }
    out.push_back('"');
  }
  void write(std::string& out, const Style& st) const {
    switch (t_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Int: out += std::to_string(i_); break;
      case Double: {
        if (std::isnan(d_)) { out += "NaN"; break; }
        if (std::isinf(d_)) { out += d_ > 0 ? "Infinity" : "-Infinity"; break; }
        if (int_like_) {
          if (!s_.empty()) { out += s_; break; }            // parsed from text: the digits as written
          char ib[64];
          snprintf(ib, sizeof ib, "%.0f", d_);
          out += ib;
          break;
        }
        // Python's repr(float): the shortest digits that round-trip, fixed notation for decimal exponents in
        // [-4, 16), else d.ddde+XX with at least two exponent digits
        char b[40];
        int prec = 1;
        for (; prec <= 17; ++prec) {
          snprintf(b, sizeof b, "%.*e", prec - 1, d_);
          if (std::strtod(b, nullptr) == d_) break;
        }
        std::string m = b;                       // [-]d[.ddd]e[+-]XX
        const size_t epos = m.find('e');
        const int e10 = std::atoi(m.c_str() + epos + 1);
        std::string digits;
        bool neg = false;
        for (size_t i = 0; i < epos; ++i) { if (m[i] == '-') neg = true; else if (m[i] != '.') digits.push_back(m[i]); }
        std::string s = neg ? "-" : "";
        if (e10 >= -4 && e10 < 16) {
          if (e10 < 0) {
            s += "0." + std::string((size_t)(-e10 - 1), '0') + digits;
          } else if ((int)digits.size() <= e10 + 1) {
            s += digits + std::string((size_t)(e10 + 1 - (int)digits.size()), '0') + ".0";
          } else {
            s += digits.substr(0, (size_t)e10 + 1) + "." + digits.substr((size_t)e10 + 1);
          }
        } else {
          s += digits.substr(0, 1);
          if (digits.size() > 1) s += "." + digits.substr(1);
          char eb[16];
          snprintf(eb, sizeof eb, "e%c%02d", e10 < 0 ? '-' : '+', e10 < 0 ? -e10 : e10);
          s += eb;
        }
        out += s;
        break;
      }
      case String: write_string(out, s_, st.ensure_ascii); break;
      case Array:
        out.push_back('[');
        for (size_t i = 0; i < a_.size(); ++i) { if (i) out += st.python ? ", " : ","; a_[i].write(out, st); }
        out.push_back(']');
        break;
      case Object:
        out.push_back('{');
        for (size_t i = 0; i < o_.size(); ++i) {
          if (i) out += st.python ? ", " : ",";
          write_string(out, o_[i].first, st.ensure_ascii);
          out += st.python ? ": " : ":";
          o_[i].second.write(out, st);
        }
        out.push_back('}');
        break;
    }
  }
};

}  // namespace b2
