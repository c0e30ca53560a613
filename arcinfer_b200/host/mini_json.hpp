// A small JSON value with a parser and a compact serialiser, for the schemas and tool lists the
// constraint automata are built from. It reads what the reference's src/json.h reads and writes
// the same compact text (src/json.h:72-76, :89-150: "," and ":" separators, integers below 1e15
// without a fraction, other numbers with 17 significant digits, control characters as \u00xx,
// every other byte raw; objects keep insertion order, a repeated key keeps its first place and
// its last value), because enum / const values are matched against that text
// (tools/json_constraint.h:112-124).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <utility>
#include <vector>

namespace arcinfer_b200 {

class JVal {
 public:
  enum Type { Null, Bool, Number, String, Array, Object };
  Type t = Null;
  bool b = false;
  double n = 0;
  std::string s;
  std::vector<JVal> a;
  std::vector<std::pair<std::string, JVal>> o;

  bool is_null() const { return t == Null; }
  bool is_bool() const { return t == Bool; }
  bool is_string() const { return t == String; }
  bool is_array() const { return t == Array; }
  bool is_object() const { return t == Object; }
  bool as_bool(bool def = false) const { return t == Bool ? b : def; }
  int64_t as_int(int64_t def = 0) const { return t == Number && std::isfinite(n) && std::fabs(n) < 9.2e18 ? (int64_t)n : def; }
  std::string str() const { return t == String ? s : std::string(); }
  bool has(const std::string& k) const {
    for (const auto& kv : o)
      if (kv.first == k) return true;
    return false;
  }
  const JVal& operator[](const std::string& k) const {
    for (const auto& kv : o)
      if (kv.first == k) return kv.second;
    return null_ref();
  }
  const JVal& operator[](const char* k) const { return (*this)[std::string(k)]; }
  static const JVal& null_ref() {
    static const JVal z;
    return z;
  }

  std::string dump() const {
    std::string out;
    write(out);
    return out;
  }
  // false when the text is not JSON
  static bool parse(const std::string& text, JVal& out) {
    size_t i = 0;
    if (!value(text, i, out, 0)) return false;
    ws(text, i);
    return i == text.size();
  }

 private:
  static void escape(std::string& out, const std::string& str) {
    out.push_back('"');
    for (unsigned char c : str) {
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
    out.push_back('"');
  }
  void write(std::string& out) const {
    switch (t) {
      case Null: out += "null"; break;
      case Bool: out += b ? "true" : "false"; break;
      case Number: {
        char buf[32];
        if (!std::isfinite(n)) snprintf(buf, sizeof buf, "null");
        else if (n == std::floor(n) && std::fabs(n) < 1e15) snprintf(buf, sizeof buf, "%lld", (long long)n);
        else snprintf(buf, sizeof buf, "%.17g", n);
        out += buf;
        break;
      }
      case String: escape(out, s); break;
      case Array:
        out.push_back('[');
        for (size_t i = 0; i < a.size(); ++i) {
          if (i) out.push_back(',');
          a[i].write(out);
        }
        out.push_back(']');
        break;
      case Object:
        out.push_back('{');
        for (size_t i = 0; i < o.size(); ++i) {
          if (i) out.push_back(',');
          escape(out, o[i].first);
          out.push_back(':');
          o[i].second.write(out);
        }
        out.push_back('}');
        break;
    }
  }
  static void ws(const std::string& s, size_t& i) {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\r' || s[i] == '\t')) ++i;
  }
  static void utf8(std::string& o, uint32_t cp) {
    if (cp < 0x80) {
      o.push_back((char)cp);
    } else if (cp < 0x800) {
      o.push_back((char)(0xC0 | (cp >> 6)));
      o.push_back((char)(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      o.push_back((char)(0xE0 | (cp >> 12)));
      o.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      o.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      o.push_back((char)(0xF0 | (cp >> 18)));
      o.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      o.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      o.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }
  static bool hex4(const std::string& s, size_t p, uint32_t& v) {
    if (p + 4 > s.size()) return false;
    v = 0;
    for (size_t q = p; q < p + 4; ++q) {
      const char h = s[q];
      const int d = h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : -1;
      if (d < 0) return false;
      v = v * 16 + (uint32_t)d;
    }
    return true;
  }
  static bool string(const std::string& s, size_t& i, std::string& o) {
    if (i >= s.size() || s[i] != '"') return false;
    ++i;
    while (i < s.size() && s[i] != '"') {
      const char c = s[i++];
      if (c != '\\') {
        o.push_back(c);
        continue;
      }
      if (i >= s.size()) break;
      const char e = s[i++];
      switch (e) {
        case 'n': o.push_back('\n'); break;
        case 't': o.push_back('\t'); break;
        case 'r': o.push_back('\r'); break;
        case 'b': o.push_back('\b'); break;
        case 'f': o.push_back('\f'); break;
        case 'u': {
          uint32_t cp, lo;
          if (!hex4(s, i, cp)) return false;
          i += 4;
          if (cp >= 0xD800 && cp < 0xDC00 && i + 6 <= s.size() && s[i] == '\\' && s[i + 1] == 'u') {
            if (!hex4(s, i + 2, lo)) return false;
            if (lo >= 0xDC00 && lo < 0xE000) {
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
              i += 6;
            }
          }
          utf8(o, cp);
          break;
        }
        default: o.push_back(e);
      }
    }
    if (i >= s.size()) return false;
    ++i;
    return true;
  }
  static bool value(const std::string& s, size_t& i, JVal& out, int depth) {
    if (depth > 256) return false;
    ws(s, i);
    if (i >= s.size()) return false;
    const char c = s[i];
    if (c == '{') {
      out = JVal();
      out.t = Object;
      ++i;
      ws(s, i);
      if (i < s.size() && s[i] == '}') {
        ++i;
        return true;
      }
      while (true) {
        ws(s, i);
        std::string k;
        if (!string(s, i, k)) return false;
        ws(s, i);
        if (i >= s.size() || s[i] != ':') return false;
        ++i;
        JVal v;
        if (!value(s, i, v, depth + 1)) return false;
        bool fresh = true;
        for (auto& kv : out.o)
          if (kv.first == k) {
            kv.second = std::move(v);
            fresh = false;
            break;
          }
        if (fresh) out.o.push_back({std::move(k), std::move(v)});
        ws(s, i);
        if (i < s.size() && s[i] == ',') {
          ++i;
          continue;
        }
        if (i < s.size() && s[i] == '}') {
          ++i;
          return true;
        }
        return false;
      }
    }
    if (c == '[') {
      out = JVal();
      out.t = Array;
      ++i;
      ws(s, i);
      if (i < s.size() && s[i] == ']') {
        ++i;
        return true;
      }
      while (true) {
        JVal v;
        if (!value(s, i, v, depth + 1)) return false;
        out.a.push_back(std::move(v));
        ws(s, i);
        if (i < s.size() && s[i] == ',') {
          ++i;
          continue;
        }
        if (i < s.size() && s[i] == ']') {
          ++i;
          return true;
        }
        return false;
      }
    }
    out = JVal();
    if (c == '"') {
      out.t = String;
      return string(s, i, out.s);
    }
    if (s.compare(i, 4, "true") == 0) {
      i += 4;
      out.t = Bool;
      out.b = true;
      return true;
    }
    if (s.compare(i, 5, "false") == 0) {
      i += 5;
      out.t = Bool;
      return true;
    }
    if (s.compare(i, 4, "null") == 0) {
      i += 4;
      return true;
    }
    size_t j = i;
    while (j < s.size() && ((s[j] >= '0' && s[j] <= '9') || s[j] == '-' || s[j] == '+' || s[j] == '.' || s[j] == 'e' || s[j] == 'E')) ++j;
    if (j == i) return false;
    const std::string tok = s.substr(i, j - i);
    char* end = nullptr;
    const double v = std::strtod(tok.c_str(), &end);
    if (end != tok.c_str() + tok.size() || !std::isfinite(v)) return false;
    i = j;
    out.t = Number;
    out.n = v;
    return true;
  }
};

}  // namespace arcinfer_b200
