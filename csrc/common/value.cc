#include "value.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <fstream>
#include <sstream>

namespace mccs {

// ---------------------------------------------------------------------------
// JSON writer
// ---------------------------------------------------------------------------
static void json_escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
        else out.push_back((char)c);
    }
  }
  out.push_back('"');
}

void Value::json_into(std::string& out, bool pretty, int indent) const {
  auto nl = [&](int ind) { if (pretty) { out.push_back('\n'); out.append((size_t)ind * 2, ' '); } };
  switch (type_) {
    case kNull: out += "null"; break;
    case kBool: out += b_ ? "true" : "false"; break;
    case kInt: out += std::to_string(i_); break;
    case kDouble: {
      char buf[40];
      if (d_ != d_ || d_ - d_ != 0) snprintf(buf, sizeof buf, "null");
      else snprintf(buf, sizeof buf, "%.9g", d_);
      out += buf;
      break;
    }
    case kString: json_escape(s_, out); break;
    case kArray: {
      out.push_back('[');
      bool first = true;
      for (const auto& v : a_) {
        if (!first) out.push_back(',');
        first = false;
        nl(indent + 1);
        v.json_into(out, pretty, indent + 1);
      }
      if (!a_.empty()) nl(indent);
      out.push_back(']');
      break;
    }
    case kObject: {
      out.push_back('{');
      bool first = true;
      for (const auto& kv : o_) {
        if (!first) out.push_back(',');
        first = false;
        nl(indent + 1);
        json_escape(kv.first, out);
        out += pretty ? ": " : ":";
        kv.second.json_into(out, pretty, indent + 1);
      }
      if (!o_.empty()) nl(indent);
      out.push_back('}');
      break;
    }
  }
}

std::string Value::to_json(bool pretty) const {
  std::string out;
  json_into(out, pretty, 0);
  return out;
}

// ---------------------------------------------------------------------------
// Shared scanner
// ---------------------------------------------------------------------------
namespace {

struct Scanner {
  const std::string& s;
  size_t p = 0;
  int line = 1;
  explicit Scanner(const std::string& text) : s(text) {}
  bool eof() const { return p >= s.size(); }
  char peek() const { return p < s.size() ? s[p] : '\0'; }
  char get() { char c = peek(); if (c == '\n') line++; p++; return c; }
  [[noreturn]] void fail(const std::string& m) const {
    throw ParseError("line " + std::to_string(line) + ": " + m);
  }
  void expect(char c) { if (peek() != c) fail(std::string("expected '") + c + "'"); get(); }
  // Nesting of arrays and tables is bounded: the parsers recurse, and some of their
  // input (the admin endpoint's JSON) comes from the network.
  int depth = 0;
  static constexpr int kMaxDepth = 64;
};

struct Nested {
  Scanner& sc;
  explicit Nested(Scanner& s) : sc(s) { if (++sc.depth > Scanner::kMaxDepth) sc.fail("nested too deeply"); }
  ~Nested() { sc.depth--; }
};

void append_utf8(std::string& out, unsigned cp) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) {
    out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back((char)(0x80 | (cp & 0x3F)));
  } else {
    out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
  }
}

std::string scan_basic_string(Scanner& sc) {  // after opening quote
  std::string out;
  for (;;) {
    if (sc.eof()) sc.fail("unterminated string");
    char c = sc.get();
    if (c == '"') break;
    if (c == '\\') {
      char e = sc.get();
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case '/': out.push_back('/'); break;
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case 'u': case 'U': {
          int n = e == 'u' ? 4 : 8;
          unsigned cp = 0;
          for (int i = 0; i < n; i++) {
            char h = sc.get();
            cp <<= 4;
            if (h >= '0' && h <= '9') cp |= (unsigned)(h - '0');
            else if (h >= 'a' && h <= 'f') cp |= (unsigned)(h - 'a' + 10);
            else if (h >= 'A' && h <= 'F') cp |= (unsigned)(h - 'A' + 10);
            else sc.fail("bad unicode escape");
          }
          append_utf8(out, cp);
          break;
        }
        default: sc.fail("bad escape");
      }
    } else {
      out.push_back(c);
    }
  }
  return out;
}

Value scan_number(Scanner& sc, bool toml) {
  size_t start = sc.p;
  std::string tok;
  while (!sc.eof()) {
    char c = sc.peek();
    if ((c >= '0' && c <= '9') || c == '+' || c == '-' || c == '.' || c == 'e' || c == 'E' ||
        c == 'x' || c == 'X' || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F') || c == 'o' ||
        (toml && c == '_') || c == 'i' || c == 'n') {
      if (c != '_') tok.push_back(c);
      sc.get();
    } else {
      break;
    }
  }
  if (tok.empty()) { sc.p = start; sc.fail("expected a value"); }
  if (tok == "inf" || tok == "+inf") return Value(1.0 / 0.0);
  if (tok == "-inf") return Value(-1.0 / 0.0);
  if (tok == "nan" || tok == "+nan" || tok == "-nan") return Value(0.0 / 0.0);
  bool is_hex = tok.size() > 2 && tok[0] == '0' && (tok[1] == 'x' || tok[1] == 'X');
  bool is_float = !is_hex && (tok.find('.') != std::string::npos || tok.find('e') != std::string::npos ||
                              tok.find('E') != std::string::npos);
  char* end = nullptr;
  if (is_float) {
    double d = strtod(tok.c_str(), &end);
    if (*end) sc.fail("bad number '" + tok + "'");
    return Value(d);
  }
  long long v;
  if (tok.size() > 2 && tok[0] == '0' && tok[1] == 'o') v = strtoll(tok.c_str() + 2, &end, 8);
  else if (tok.size() > 2 && tok[0] == '0' && tok[1] == 'b') v = strtoll(tok.c_str() + 2, &end, 2);
  else v = strtoll(tok.c_str(), &end, 0);
  if (*end) sc.fail("bad number '" + tok + "'");
  return Value((int64_t)v);
}

// ---------------------------------------------------------------------------
// JSON
// ---------------------------------------------------------------------------
void json_ws(Scanner& sc) {
  while (!sc.eof() && (sc.peek() == ' ' || sc.peek() == '\t' || sc.peek() == '\n' || sc.peek() == '\r')) sc.get();
}

Value json_value(Scanner& sc) {
  Nested guard(sc);
  json_ws(sc);
  char c = sc.peek();
  if (c == '{') {
    sc.get();
    Value obj = Value::object();
    json_ws(sc);
    if (sc.peek() == '}') { sc.get(); return obj; }
    for (;;) {
      json_ws(sc);
      sc.expect('"');
      std::string key = scan_basic_string(sc);
      json_ws(sc);
      sc.expect(':');
      obj.set(key, json_value(sc));
      json_ws(sc);
      if (sc.peek() == ',') { sc.get(); continue; }
      sc.expect('}');
      break;
    }
    return obj;
  }
  if (c == '[') {
    sc.get();
    Value arr = Value::array();
    json_ws(sc);
    if (sc.peek() == ']') { sc.get(); return arr; }
    for (;;) {
      arr.push(json_value(sc));
      json_ws(sc);
      if (sc.peek() == ',') { sc.get(); continue; }
      sc.expect(']');
      break;
    }
    return arr;
  }
  if (c == '"') { sc.get(); return Value(scan_basic_string(sc)); }
  if (sc.s.compare(sc.p, 4, "true") == 0) { sc.p += 4; return Value(true); }
  if (sc.s.compare(sc.p, 5, "false") == 0) { sc.p += 5; return Value(false); }
  if (sc.s.compare(sc.p, 4, "null") == 0) { sc.p += 4; return Value(); }
  return scan_number(sc, false);
}

// ---------------------------------------------------------------------------
// TOML
// ---------------------------------------------------------------------------
void toml_ws(Scanner& sc) {  // spaces and tabs only
  while (!sc.eof() && (sc.peek() == ' ' || sc.peek() == '\t')) sc.get();
}
void toml_ws_nl(Scanner& sc) {  // whitespace, newlines and comments
  for (;;) {
    char c = sc.peek();
    if (c == ' ' || c == '\t' || c == '\n' || c == '\r') sc.get();
    else if (c == '#') { while (!sc.eof() && sc.peek() != '\n') sc.get(); }
    else break;
  }
}

std::string toml_key_part(Scanner& sc) {
  toml_ws(sc);
  char c = sc.peek();
  if (c == '"') { sc.get(); return scan_basic_string(sc); }
  if (c == '\'') {
    sc.get();
    std::string out;
    while (!sc.eof() && sc.peek() != '\'') out.push_back(sc.get());
    sc.expect('\'');
    return out;
  }
  std::string out;
  while (!sc.eof()) {
    c = sc.peek();
    if ((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_' || c == '-')
      out.push_back(sc.get());
    else break;
  }
  if (out.empty()) sc.fail("expected a key");
  return out;
}

std::vector<std::string> toml_key(Scanner& sc) {
  std::vector<std::string> parts;
  for (;;) {
    parts.push_back(toml_key_part(sc));
    toml_ws(sc);
    if (sc.peek() == '.') { sc.get(); continue; }
    break;
  }
  return parts;
}

Value toml_value(Scanner& sc);

Value toml_inline_table(Scanner& sc) {  // after '{'
  Value obj = Value::object();
  toml_ws_nl(sc);
  if (sc.peek() == '}') { sc.get(); return obj; }
  for (;;) {
    toml_ws_nl(sc);
    std::vector<std::string> key = toml_key(sc);
    toml_ws(sc);
    sc.expect('=');
    Value v = toml_value(sc);
    Value* cur = &obj;
    for (size_t i = 0; i + 1 < key.size(); i++) cur = &cur->fields_mut()[key[i]], cur->fields_mut();
    cur->fields_mut()[key.back()] = std::move(v);
    toml_ws_nl(sc);
    if (sc.peek() == ',') { sc.get(); toml_ws_nl(sc); if (sc.peek() == '}') { sc.get(); break; } continue; }
    sc.expect('}');
    break;
  }
  return obj;
}

Value toml_value(Scanner& sc) {
  Nested guard(sc);
  toml_ws(sc);
  char c = sc.peek();
  if (c == '"') {
    if (sc.s.compare(sc.p, 3, "\"\"\"") == 0) {
      sc.p += 3;
      if (sc.peek() == '\n') sc.get();
      std::string out;
      while (!sc.eof() && sc.s.compare(sc.p, 3, "\"\"\"") != 0) out.push_back(sc.get());
      if (sc.eof()) sc.fail("unterminated multi-line string");
      sc.p += 3;
      return Value(out);
    }
    sc.get();
    return Value(scan_basic_string(sc));
  }
  if (c == '\'') {
    sc.get();
    std::string out;
    while (!sc.eof() && sc.peek() != '\'' && sc.peek() != '\n') out.push_back(sc.get());
    sc.expect('\'');
    return Value(out);
  }
  if (c == '[') {
    sc.get();
    Value arr = Value::array();
    for (;;) {
      toml_ws_nl(sc);
      if (sc.peek() == ']') { sc.get(); break; }
      arr.push(toml_value(sc));
      toml_ws_nl(sc);
      if (sc.peek() == ',') { sc.get(); continue; }
      toml_ws_nl(sc);
      sc.expect(']');
      break;
    }
    return arr;
  }
  if (c == '{') { sc.get(); return toml_inline_table(sc); }
  if (sc.s.compare(sc.p, 4, "true") == 0) { sc.p += 4; return Value(true); }
  if (sc.s.compare(sc.p, 5, "false") == 0) { sc.p += 5; return Value(false); }
  return scan_number(sc, true);
}

// Walks (creating as needed) to the table named by `path` below `root`. When an
// element on the way is an array of tables, its last entry is used.
Value* toml_descend(Value* root, const std::vector<std::string>& path, size_t upto, Scanner& sc) {
  Value* cur = root;
  for (size_t i = 0; i < upto; i++) {
    Value& next = cur->fields_mut()[path[i]];
    if (next.is_null()) next = Value::object();
    if (next.is_array()) {
      if (next.items().empty()) sc.fail("empty array of tables '" + path[i] + "'");
      cur = &next.items_mut().back();
    } else if (next.is_object()) {
      cur = &next;
    } else {
      sc.fail("key '" + path[i] + "' is not a table");
    }
  }
  return cur;
}

}  // namespace

Value parse_json(const std::string& text) {
  Scanner sc(text);
  Value v = json_value(sc);
  json_ws(sc);
  if (!sc.eof()) sc.fail("trailing characters after JSON value");
  return v;
}

Value parse_toml(const std::string& text) {
  Scanner sc(text);
  Value root = Value::object();
  Value* table = &root;
  for (;;) {
    toml_ws_nl(sc);
    if (sc.eof()) break;
    if (sc.peek() == '[') {
      sc.get();
      bool is_array = false;
      if (sc.peek() == '[') { sc.get(); is_array = true; }
      std::vector<std::string> path = toml_key(sc);
      toml_ws(sc);
      sc.expect(']');
      if (is_array) sc.expect(']');
      Value* parent = toml_descend(&root, path, path.size() - 1, sc);
      Value& slot = parent->fields_mut()[path.back()];
      if (is_array) {
        if (slot.is_null()) slot = Value::array();
        if (!slot.is_array()) sc.fail("'" + path.back() + "' is not an array of tables");
        slot.items_mut().push_back(Value::object());
        table = &slot.items_mut().back();
      } else {
        if (slot.is_null()) slot = Value::object();
        if (slot.is_array()) table = &slot.items_mut().back();
        else if (slot.is_object()) table = &slot;
        else sc.fail("'" + path.back() + "' is not a table");
      }
    } else {
      std::vector<std::string> key = toml_key(sc);
      toml_ws(sc);
      sc.expect('=');
      Value v = toml_value(sc);
      Value* parent = toml_descend(table, key, key.size() - 1, sc);
      if (parent->has(key.back())) sc.fail("duplicate key '" + key.back() + "'");
      parent->fields_mut()[key.back()] = std::move(v);
      toml_ws(sc);
      if (sc.peek() == '#') while (!sc.eof() && sc.peek() != '\n') sc.get();
      if (!sc.eof() && sc.peek() != '\n' && sc.peek() != '\r') sc.fail("expected end of line");
    }
  }
  return root;
}

std::string expand_env(const std::string& s) {
  std::string out;
  for (size_t i = 0; i < s.size();) {
    if (s[i] == '$' && i + 1 < s.size() && s[i + 1] == '{') {
      size_t end = s.find('}', i + 2);
      if (end != std::string::npos) {
        std::string name = s.substr(i + 2, end - i - 2);
        const char* v = getenv(name.c_str());
        if (!v && name == "USER") v = getenv("LOGNAME");
        if (!v && name == "USER") v = "user";
        if (v) out += v;
        i = end + 1;
        continue;
      }
    }
    out.push_back(s[i++]);
  }
  return out;
}

std::string read_text_file(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

}  // namespace mccs
