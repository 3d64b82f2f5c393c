#include "json.h"

#include <cmath>
#include <cstdlib>
#include <stdexcept>

namespace tei {

class JsonParser {
 public:
  JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}

  Json parse_document() {
    Json v = parse_value(0);
    skip_ws();
    if (p_ != end_) fail("trailing characters");
    return v;
  }

 private:
  const char* p_;
  const char* end_;

  [[noreturn]] void fail(const char* what) { throw std::runtime_error(std::string("JSON: ") + what); }

  void skip_ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }

  bool consume(const char* lit) {
    const char* q = p_;
    while (*lit) {
      if (q >= end_ || *q != *lit) return false;
      ++q;
      ++lit;
    }
    p_ = q;
    return true;
  }

  static void append_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) {
      s.push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
      s.push_back(static_cast<char>(0xC0 | (cp >> 6)));
      s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      s.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      s.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      s.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      s.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      s.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }

  uint32_t parse_hex4() {
    if (end_ - p_ < 4) fail("short \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad \\u escape");
    }
    return v;
  }

  std::string parse_string() {
    if (p_ >= end_ || *p_ != '"') fail("expected string");
    ++p_;
    std::string s;
    while (true) {
      if (p_ >= end_) fail("unterminated string");
      const char c = *p_++;
      if (c == '"') break;
      if (c != '\\') {
        s.push_back(c);
        continue;
      }
      if (p_ >= end_) fail("unterminated escape");
      const char e = *p_++;
      switch (e) {
        case '"': s.push_back('"'); break;
        case '\\': s.push_back('\\'); break;
        case '/': s.push_back('/'); break;
        case 'b': s.push_back('\b'); break;
        case 'f': s.push_back('\f'); break;
        case 'n': s.push_back('\n'); break;
        case 'r': s.push_back('\r'); break;
        case 't': s.push_back('\t'); break;
        case 'u': {
          uint32_t cp = parse_hex4();
          if (cp >= 0xD800 && cp <= 0xDBFF && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            const uint32_t lo = parse_hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          append_utf8(s, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
    return s;
  }

  Json parse_value(int depth) {
    if (depth > 64) fail("nesting too deep");
    skip_ws();
    if (p_ >= end_) fail("unexpected end");
    Json v;
    const char c = *p_;
    if (c == '{') {
      ++p_;
      v.kind_ = Json::Object;
      skip_ws();
      if (p_ < end_ && *p_ == '}') {
        ++p_;
        return v;
      }
      while (true) {
        skip_ws();
        std::string key = parse_string();
        skip_ws();
        if (p_ >= end_ || *p_ != ':') fail("expected ':'");
        ++p_;
        Json member = parse_value(depth + 1);
        v.object_.emplace_back(std::move(key), std::move(member));
        skip_ws();
        if (p_ < end_ && *p_ == ',') {
          ++p_;
          continue;
        }
        if (p_ < end_ && *p_ == '}') {
          ++p_;
          break;
        }
        fail("expected ',' or '}'");
      }
    } else if (c == '[') {
      ++p_;
      v.kind_ = Json::Array;
      skip_ws();
      if (p_ < end_ && *p_ == ']') {
        ++p_;
        return v;
      }
      while (true) {
        v.array_.push_back(parse_value(depth + 1));
        skip_ws();
        if (p_ < end_ && *p_ == ',') {
          ++p_;
          continue;
        }
        if (p_ < end_ && *p_ == ']') {
          ++p_;
          break;
        }
        fail("expected ',' or ']'");
      }
    } else if (c == '"') {
      v.kind_ = Json::String;
      v.string_ = parse_string();
    } else if (consume("true")) {
      v.kind_ = Json::Bool;
      v.bool_ = true;
    } else if (consume("false")) {
      v.kind_ = Json::Bool;
      v.bool_ = false;
    } else if (consume("null")) {
      v.kind_ = Json::Null;
    } else if (consume("NaN")) {
      v.kind_ = Json::Number;
      v.number_ = std::nan("");
    } else if (consume("Infinity")) {
      v.kind_ = Json::Number;
      v.number_ = INFINITY;
    } else if (consume("-Infinity")) {
      v.kind_ = Json::Number;
      v.number_ = -INFINITY;
    } else {
      const char* start = p_;
      while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '-' || *p_ == '+' || *p_ == '.' ||
                           *p_ == 'e' || *p_ == 'E')) {
        ++p_;
      }
      if (p_ == start) fail("unexpected character");
      std::string num(start, p_);
      char* endp = nullptr;
      v.kind_ = Json::Number;
      v.number_ = std::strtod(num.c_str(), &endp);
      if (endp == num.c_str() || *endp != '\0') fail("bad number");
    }
    return v;
  }
};

Json Json::parse(const std::string& text) { return parse(text.data(), text.size()); }

Json Json::parse(const char* data, size_t len) {
  JsonParser p(data, len);
  return p.parse_document();
}

bool Json::has(const std::string& key) const {
  if (kind_ != Object) return false;
  for (const auto& m : object_) {
    if (m.first == key) return true;
  }
  return false;
}

const Json& Json::operator[](const std::string& key) const {
  static const Json null_value;
  if (kind_ != Object) return null_value;
  for (const auto& m : object_) {
    if (m.first == key) return m.second;
  }
  return null_value;
}

const Json& Json::at(size_t i) const {
  if (kind_ != Array || i >= array_.size()) throw std::runtime_error("JSON: array index out of range");
  return array_[i];
}

size_t Json::size() const {
  if (kind_ == Array) return array_.size();
  if (kind_ == Object) return object_.size();
  return 0;
}

double Json::as_double() const {
  if (kind_ != Number) throw std::runtime_error("JSON: expected a number");
  return number_;
}

int64_t Json::as_int() const {
  if (kind_ != Number) throw std::runtime_error("JSON: expected a number");
  return static_cast<int64_t>(std::llround(number_));
}

bool Json::as_bool() const {
  if (kind_ != Bool) throw std::runtime_error("JSON: expected a boolean");
  return bool_;
}

const std::string& Json::as_string() const {
  if (kind_ != String) throw std::runtime_error("JSON: expected a string");
  return string_;
}

int64_t Json::get_int(const std::string& key, int64_t dflt) const {
  const Json& v = (*this)[key];
  return v.is_number() ? v.as_int() : dflt;
}

double Json::get_double(const std::string& key, double dflt) const {
  const Json& v = (*this)[key];
  return v.is_number() ? v.as_double() : dflt;
}

bool Json::get_bool(const std::string& key, bool dflt) const {
  const Json& v = (*this)[key];
  return v.is_bool() ? v.as_bool() : dflt;
}

std::string Json::get_string(const std::string& key, const std::string& dflt) const {
  const Json& v = (*this)[key];
  return v.is_string() ? v.as_string() : dflt;
}

}  // namespace tei
