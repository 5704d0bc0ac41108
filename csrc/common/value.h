// A small dynamically typed value tree with a TOML reader and a JSON reader/writer.
// The daemon configuration keeps the TOML schema of the reference service
// (src/mccs/src/config.rs:14-89, mccs.toml); admin messages and trace/statistics
// dumps use JSON.
#pragma once
#include <stdint.h>

#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace mccs {

class Value {
 public:
  enum Type { kNull, kBool, kInt, kDouble, kString, kArray, kObject };
  using Array = std::vector<Value>;
  using Object = std::map<std::string, Value>;

  Value() : type_(kNull) {}
  Value(bool b) : type_(kBool), b_(b) {}
  Value(int v) : type_(kInt), i_(v) {}
  Value(int64_t v) : type_(kInt), i_(v) {}
  Value(uint64_t v) : type_(kInt), i_((int64_t)v) {}
  Value(double v) : type_(kDouble), d_(v) {}
  Value(const char* s) : type_(kString), s_(s) {}
  Value(const std::string& s) : type_(kString), s_(s) {}
  static Value array() { Value v; v.type_ = kArray; return v; }
  static Value object() { Value v; v.type_ = kObject; return v; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == kNull; }
  bool is_object() const { return type_ == kObject; }
  bool is_array() const { return type_ == kArray; }
  bool is_string() const { return type_ == kString; }
  bool is_number() const { return type_ == kInt || type_ == kDouble; }

  bool as_bool(bool dflt = false) const { return type_ == kBool ? b_ : (type_ == kInt ? i_ != 0 : dflt); }
  int64_t as_int(int64_t dflt = 0) const {
    return type_ == kInt ? i_ : (type_ == kDouble ? (int64_t)d_ : (type_ == kBool ? (int64_t)b_ : dflt));
  }
  double as_double(double dflt = 0) const { return type_ == kDouble ? d_ : (type_ == kInt ? (double)i_ : dflt); }
  const std::string& as_string() const { static const std::string empty; return type_ == kString ? s_ : empty; }
  std::string as_string(const std::string& dflt) const { return type_ == kString ? s_ : dflt; }

  const Array& items() const { static const Array empty; return type_ == kArray ? a_ : empty; }
  Array& items_mut() { if (type_ != kArray) { *this = array(); } return a_; }
  const Object& fields() const { static const Object empty; return type_ == kObject ? o_ : empty; }
  Object& fields_mut() { if (type_ != kObject) { *this = object(); } return o_; }

  bool has(const std::string& k) const { return type_ == kObject && o_.count(k) != 0; }
  // Missing keys read as a shared null value, so lookups can be chained.
  const Value& operator[](const std::string& k) const {
    static const Value null_value;
    if (type_ != kObject) return null_value;
    auto it = o_.find(k);
    return it == o_.end() ? null_value : it->second;
  }
  Value& set(const std::string& k, Value v) { fields_mut()[k] = std::move(v); return *this; }
  Value& push(Value v) { items_mut().push_back(std::move(v)); return *this; }
  size_t size() const { return type_ == kArray ? a_.size() : (type_ == kObject ? o_.size() : 0); }
  const Value& at(size_t i) const { static const Value null_value; return (type_ == kArray && i < a_.size()) ? a_[i] : null_value; }

  std::string to_json(bool pretty = false) const;

 private:
  void json_into(std::string& out, bool pretty, int indent) const;
  Type type_;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  Array a_;
  Object o_;
};

struct ParseError : std::runtime_error {
  explicit ParseError(const std::string& m) : std::runtime_error(m) {}
};

// Throws ParseError with a line number on malformed input.
Value parse_toml(const std::string& text);
Value parse_json(const std::string& text);
// Replaces ${NAME} by the environment variable NAME (empty when unset), the way the
// reference expands ${USER} in socket prefixes (src/mccs/src/control.rs:77-83).
std::string expand_env(const std::string& s);
std::string read_text_file(const std::string& path);  // throws std::runtime_error

}  // namespace mccs
