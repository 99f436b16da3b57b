// Minimal JSON reader for the two formats the runtime parses: tokenizer lines (one JSON string per line) and
// safetensors headers (an object of objects with strings and integer arrays).  Values are kept as a small tree.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace fbam {

struct JsonValue {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  double number = 0;
  bool boolean = false;
  std::string str;
  std::vector<JsonValue> items;
  std::vector<std::pair<std::string, JsonValue>> members;

  const JsonValue* find(const std::string& key) const {
    for (const auto& m : members)
      if (m.first == key) return &m.second;
    return nullptr;
  }
};

class JsonParser {
 public:
  explicit JsonParser(const std::string& text) : s_(text) {}

  JsonValue parse() {
    JsonValue v = value();
    skip();
    if (i_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  const std::string& s_;
  size_t i_ = 0;

  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("JSON: ") + what + " at offset " + std::to_string(i_));
  }
  void skip() {
    while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\t' || s_[i_] == '\n' || s_[i_] == '\r')) ++i_;
  }
  static void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += static_cast<char>(cp);
    else if (cp < 0x800) { out += static_cast<char>(0xC0 | (cp >> 6)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) {
      out += static_cast<char>(0xE0 | (cp >> 12));
      out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
      out += static_cast<char>(0x80 | (cp & 0x3F));
    } else {
      out += static_cast<char>(0xF0 | (cp >> 18));
      out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
      out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
      out += static_cast<char>(0x80 | (cp & 0x3F));
    }
  }
  uint32_t hex4() {
    if (i_ + 4 > s_.size()) fail("short \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      const char c = s_[i_++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad hex digit");
    }
    return v;
  }
  std::string string() {
    if (s_[i_] != '"') fail("expected string");
    ++i_;
    std::string out;
    while (true) {
      if (i_ >= s_.size()) fail("unterminated string");
      const char c = s_[i_++];
      if (c == '"') break;
      if (c != '\\') { out += c; continue; }
      if (i_ >= s_.size()) fail("dangling escape");
      const char e = s_[i_++];
      switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'n': out += '\n'; break;
        case 'r': out += '\r'; break;
        case 't': out += '\t'; break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp <= 0xDBFF && i_ + 1 < s_.size() && s_[i_] == '\\' && s_[i_ + 1] == 'u') {
            i_ += 2;
            const uint32_t lo = hex4();
            if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            else fail("unpaired surrogate");
          }
          append_utf8(out, cp);
          break;
        }
        default: fail("unknown escape");
      }
    }
    return out;
  }
  JsonValue value() {
    skip();
    if (i_ >= s_.size()) fail("unexpected end");
    JsonValue v;
    const char c = s_[i_];
    if (c == '"') { v.kind = JsonValue::String; v.str = string(); return v; }
    if (c == '{') {
      v.kind = JsonValue::Object;
      ++i_;
      skip();
      if (i_ < s_.size() && s_[i_] == '}') { ++i_; return v; }
      while (true) {
        skip();
        std::string key = string();
        skip();
        if (i_ >= s_.size() || s_[i_] != ':') fail("expected ':'");
        ++i_;
        v.members.emplace_back(std::move(key), value());
        skip();
        if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
        if (i_ < s_.size() && s_[i_] == '}') { ++i_; break; }
        fail("expected ',' or '}'");
      }
      return v;
    }
    if (c == '[') {
      v.kind = JsonValue::Array;
      ++i_;
      skip();
      if (i_ < s_.size() && s_[i_] == ']') { ++i_; return v; }
      while (true) {
        v.items.push_back(value());
        skip();
        if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
        if (i_ < s_.size() && s_[i_] == ']') { ++i_; break; }
        fail("expected ',' or ']'");
      }
      return v;
    }
    if (s_.compare(i_, 4, "true") == 0) { i_ += 4; v.kind = JsonValue::Bool; v.boolean = true; return v; }
    if (s_.compare(i_, 5, "false") == 0) { i_ += 5; v.kind = JsonValue::Bool; return v; }
    if (s_.compare(i_, 4, "null") == 0) { i_ += 4; return v; }
    size_t used = 0;
    try { v.number = std::stod(s_.substr(i_), &used); } catch (...) { fail("bad number"); }
    v.kind = JsonValue::Number;
    i_ += used;
    return v;
  }
};

inline std::u32string utf8_to_u32(const std::string& s) {
  std::u32string out;
  for (size_t i = 0; i < s.size();) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    uint32_t cp;
    int n;
    if (c < 0x80) { cp = c; n = 1; }
    else if ((c >> 5) == 6) { cp = c & 0x1F; n = 2; }
    else if ((c >> 4) == 14) { cp = c & 0x0F; n = 3; }
    else { cp = c & 0x07; n = 4; }
    if (i + n > s.size()) throw std::runtime_error("truncated UTF-8 sequence");
    for (int k = 1; k < n; ++k) cp = (cp << 6) | (static_cast<unsigned char>(s[i + k]) & 0x3F);
    out.push_back(cp);
    i += n;
  }
  return out;
}

}  // namespace fbam
