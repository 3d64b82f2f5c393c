// Minimal JSON reader for config.json and safetensors headers (objects, arrays, strings, numbers,
// booleans, null).  No third-party dependency; throws std::runtime_error on malformed input.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace tei {

class Json {
 public:
  enum Kind { Null, Bool, Number, String, Array, Object };

  static Json parse(const std::string& text);
  static Json parse(const char* data, size_t len);

  Kind kind() const { return kind_; }
  bool is_null() const { return kind_ == Null; }
  bool is_object() const { return kind_ == Object; }
  bool is_array() const { return kind_ == Array; }
  bool is_number() const { return kind_ == Number; }
  bool is_string() const { return kind_ == String; }
  bool is_bool() const { return kind_ == Bool; }

  bool has(const std::string& key) const;
  // Object member; a shared Null value when absent.
  const Json& operator[](const std::string& key) const;
  const Json& at(size_t i) const;
  size_t size() const;

  double as_double() const;
  int64_t as_int() const;
  bool as_bool() const;
  const std::string& as_string() const;
  const std::vector<std::pair<std::string, Json>>& members() const { return object_; }
  const std::vector<Json>& items() const { return array_; }

  // Typed getters with defaults for optional config fields.
  int64_t get_int(const std::string& key, int64_t dflt) const;
  double get_double(const std::string& key, double dflt) const;
  bool get_bool(const std::string& key, bool dflt) const;
  std::string get_string(const std::string& key, const std::string& dflt) const;

 private:
  friend class JsonParser;
  Kind kind_ = Null;
  bool bool_ = false;
  double number_ = 0.0;
  std::string string_;
  std::vector<Json> array_;
  std::vector<std::pair<std::string, Json>> object_;
};

}  // namespace tei
