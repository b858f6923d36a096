// Minimal JSON reader / writer used for kernel plans and trace events.
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace spike {

class Json {
 public:
  enum Type { Null, Bool, Number, String, Array, Object };
  Type type = Null;
  bool b = false;
  bool is_int = false;   // number written without fraction / exponent
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  bool is_null() const { return type == Null; }
  bool has(const std::string& k) const {
    for (auto& kv : obj)
      if (kv.first == k) return true;
    return false;
  }
  const Json& at(const std::string& k) const {
    for (auto& kv : obj)
      if (kv.first == k) return kv.second;
    throw std::runtime_error("json: missing key '" + k + "'");
  }
  const Json& at(size_t i) const { return arr.at(i); }
  long long as_int() const { return static_cast<long long>(num); }
  double as_double() const { return num; }
  const std::string& as_string() const { return str; }
  size_t size() const { return type == Array ? arr.size() : obj.size(); }

  static Json parse(const std::string& text) {
    size_t pos = 0;
    Json j = parse_value(text, pos);
    skip_ws(text, pos);
    if (pos != text.size()) throw std::runtime_error("json: trailing characters");
    return j;
  }

  static Json make_int(long long v) { Json j; j.type = Number; j.num = double(v); j.is_int = true; return j; }
  static Json make_num(double v) { Json j; j.type = Number; j.num = v; return j; }
  static Json make_str(const std::string& v) { Json j; j.type = String; j.str = v; return j; }
  static Json make_bool(bool v) { Json j; j.type = Bool; j.b = v; return j; }
  static Json make_array() { Json j; j.type = Array; return j; }
  static Json make_object() { Json j; j.type = Object; return j; }
  void set(const std::string& k, const Json& v) {
    type = Object;
    for (auto& kv : obj)
      if (kv.first == k) { kv.second = v; return; }
    obj.emplace_back(k, v);
  }
  void erase(const std::string& k) {
    for (size_t i = 0; i < obj.size(); ++i)
      if (obj[i].first == k) { obj.erase(obj.begin() + long(i)); return; }
  }
  // Same separators as Python's json.dumps(separators=(", ", ": ")); object keys sorted.
  std::string dump() const {
    std::ostringstream os;
    switch (type) {
      case Null: os << "null"; break;
      case Bool: os << (b ? "true" : "false"); break;
      case Number:
        if (is_int) os << static_cast<long long>(num);
        else { os.precision(17); os << num; if (os.str().find_first_of(".eE") == std::string::npos) os << ".0"; }
        break;
      case String: os << quote(str); break;
      case Array:
        os << "[";
        for (size_t i = 0; i < arr.size(); ++i) os << (i ? ", " : "") << arr[i].dump();
        os << "]";
        break;
      case Object: {
        std::vector<const std::pair<std::string, Json>*> items;
        for (auto& kv : obj) items.push_back(&kv);
        std::sort(items.begin(), items.end(), [](auto* a, auto* b2) { return a->first < b2->first; });
        os << "{";
        for (size_t i = 0; i < items.size(); ++i)
          os << (i ? ", " : "") << quote(items[i]->first) << ": " << items[i]->second.dump();
        os << "}";
        break;
      }
    }
    return os.str();
  }

  static std::string quote(const std::string& s) {
    std::string out = "\"";
    for (char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\t': out += "\\t"; break;
        case '\r': out += "\\r"; break;
        default: out += c;
      }
    }
    return out + "\"";
  }

 private:
  static void skip_ws(const std::string& t, size_t& p) {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
  }
  static Json parse_value(const std::string& t, size_t& p) {
    skip_ws(t, p);
    if (p >= t.size()) throw std::runtime_error("json: unexpected end");
    char c = t[p];
    Json j;
    if (c == '{') {
      j.type = Object;
      ++p;
      skip_ws(t, p);
      if (t[p] == '}') { ++p; return j; }
      while (true) {
        skip_ws(t, p);
        Json key = parse_string(t, p);
        skip_ws(t, p);
        if (t[p] != ':') throw std::runtime_error("json: expected ':'");
        ++p;
        j.obj.emplace_back(key.str, parse_value(t, p));
        skip_ws(t, p);
        if (t[p] == ',') { ++p; continue; }
        if (t[p] == '}') { ++p; break; }
        throw std::runtime_error("json: expected ',' or '}'");
      }
      return j;
    }
    if (c == '[') {
      j.type = Array;
      ++p;
      skip_ws(t, p);
      if (t[p] == ']') { ++p; return j; }
      while (true) {
        j.arr.push_back(parse_value(t, p));
        skip_ws(t, p);
        if (t[p] == ',') { ++p; continue; }
        if (t[p] == ']') { ++p; break; }
        throw std::runtime_error("json: expected ',' or ']'");
      }
      return j;
    }
    if (c == '"') return parse_string(t, p);
    if (t.compare(p, 4, "true") == 0) { p += 4; j.type = Bool; j.b = true; return j; }
    if (t.compare(p, 5, "false") == 0) { p += 5; j.type = Bool; j.b = false; return j; }
    if (t.compare(p, 4, "null") == 0) { p += 4; return j; }
    size_t end = p;
    while (end < t.size() && (isdigit(t[end]) || t[end] == '-' || t[end] == '+' || t[end] == '.' || t[end] == 'e' ||
                              t[end] == 'E'))
      ++end;
    if (end == p) throw std::runtime_error("json: unexpected character");
    j.type = Number;
    {
      const std::string tok = t.substr(p, end - p);
      j.num = std::stod(tok);
      j.is_int = tok.find_first_of(".eE") == std::string::npos;
    }
    p = end;
    return j;
  }
  static Json parse_string(const std::string& t, size_t& p) {
    if (t[p] != '"') throw std::runtime_error("json: expected string");
    ++p;
    Json j;
    j.type = String;
    while (p < t.size() && t[p] != '"') {
      if (t[p] == '\\' && p + 1 < t.size()) {
        ++p;
        switch (t[p]) {
          case 'n': j.str += '\n'; break;
          case 't': j.str += '\t'; break;
          case 'r': j.str += '\r'; break;
          case 'u': {
            unsigned code = std::stoul(t.substr(p + 1, 4), nullptr, 16);
            j.str += static_cast<char>(code < 128 ? code : '?');
            p += 4;
            break;
          }
          default: j.str += t[p];
        }
      } else {
        j.str += t[p];
      }
      ++p;
    }
    ++p;
    return j;
  }
};

inline std::vector<uint8_t> base64_decode(const std::string& in) {
  static int8_t table[256];
  static bool init = false;
  if (!init) {
    for (int i = 0; i < 256; ++i) table[i] = -1;
    const char* a = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    for (int i = 0; i < 64; ++i) table[static_cast<unsigned char>(a[i])] = static_cast<int8_t>(i);
    init = true;
  }
  std::vector<uint8_t> out;
  uint32_t acc = 0;
  int bits = 0;
  for (unsigned char c : in) {
    if (table[c] < 0) continue;
    acc = (acc << 6) | static_cast<uint32_t>(table[c]);
    bits += 6;
    if (bits >= 8) {
      bits -= 8;
      out.push_back(static_cast<uint8_t>((acc >> bits) & 0xFF));
    }
  }
  return out;
}

}  // namespace spike
