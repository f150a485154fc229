// JSON-schema and regex front ends: both produce GBNF text that the grammar parser compiles.
#include <map>
#include <set>
#include <sstream>
#include <stdexcept>

#include "../util/json.h"
#include "grammar.h"

namespace b200 {
namespace so {

const char* const kJsonGbnf =
    "value ::= object | array | string | number | \"true\" | \"false\" | \"null\"\n"
    "object ::= \"{\" ws ( string ws \":\" ws value ( ws \",\" ws string ws \":\" ws value )* )? ws \"}\"\n"
    "array ::= \"[\" ws ( value ( ws \",\" ws value )* )? ws \"]\"\n"
    "string ::= \"\\\"\" char* \"\\\"\"\n"
    "char ::= [^\"\\\\\\x00-\\x1F] | \"\\\\\" ( [\"\\\\/bfnrt] | \"u\" hex hex hex hex )\n"
    "hex ::= [0-9a-fA-F]\n"
    "number ::= integer ( \".\" [0-9]+ )? ( [eE] [-+]? [0-9]+ )?\n"
    "integer ::= \"-\"? ( \"0\" | [1-9] [0-9]* )\n"
    "boolean ::= \"true\" | \"false\"\n"
    "ws ::= [ \\t\\n]{0,8}\n";

namespace {

std::string literal(const std::string& s) {
  std::string out;
  Json::escape(s, out);
  return out;
}

class SchemaConverter {
 public:
  explicit SchemaConverter(const Json& root) : root_(root) {}

  std::string run() {
    const std::string top = visit(root_, "root-value");
    std::ostringstream o;
    o << "root ::= " << top << "\n";
    for (const auto& r : rules_) o << r.first << " ::= " << r.second << "\n";
    o << kJsonGbnf;
    return o.str();
  }

 private:
  std::string add(const std::string& name, const std::string& body) {
    std::string n = name;
    int k = 0;
    while (rules_map_.count(n) && rules_map_[n] != body) n = name + "-" + std::to_string(++k);
    if (!rules_map_.count(n)) {
      rules_map_[n] = body;
      rules_.emplace_back(n, body);
    }
    return n;
  }
  static std::string sanitize(const std::string& s) {
    std::string o;
    for (char c : s) o.push_back(((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9')) ? c : '-');
    return o.empty() ? "x" : o;
  }
  const Json& resolve(const std::string& ref) {
    if (ref.rfind("#/", 0) != 0) throw std::runtime_error("unsupported $ref: " + ref);
    const Json* cur = &root_;
    size_t pos = 2;
    while (pos <= ref.size()) {
      size_t next = ref.find('/', pos);
      if (next == std::string::npos) next = ref.size();
      const std::string key = ref.substr(pos, next - pos);
      cur = cur->find(key);
      if (!cur) throw std::runtime_error("unresolved $ref: " + ref);
      pos = next + 1;
    }
    return *cur;
  }
  std::string const_value(const Json& v) { return literal(v.dump()); }

  std::string visit(const Json& s, const std::string& name) {
    if (s.is_bool()) return "value";
    if (!s.is_object() || s.size() == 0) return "value";
    if (s.contains("$ref")) {
      const std::string& ref = s["$ref"].as_string();
      const std::string rn = "ref-" + sanitize(ref);
      if (!in_progress_.count(ref) && !rules_map_.count(rn)) {
        in_progress_.insert(ref);
        rules_map_[rn] = "";                       // reserve (recursive schemas)
        rules_.emplace_back(rn, "");
        const std::string body = visit(resolve(ref), rn + "-body");
        rules_map_[rn] = body;
        for (auto& r : rules_) if (r.first == rn) r.second = body;
        in_progress_.erase(ref);
      }
      return rn;
    }
    if (s.contains("const")) return add(name, const_value(s["const"]));
    if (s.contains("enum")) {
      std::string body;
      for (const Json& v : s["enum"].items()) {
        if (!body.empty()) body += " | ";
        body += const_value(v);
      }
      return add(name, body);
    }
    for (const char* key : {"anyOf", "oneOf"}) {
      if (s.contains(key)) {
        std::string body;
        int i = 0;
        for (const Json& v : s[key].items()) {
          if (!body.empty()) body += " | ";
          body += visit(v, name + "-" + std::to_string(i++));
        }
        return add(name, body);
      }
    }
    if (s.contains("allOf") && s["allOf"].size() == 1) return visit(s["allOf"][(size_t)0], name);
    const Json& type = s["type"];
    if (type.is_array()) {
      std::string body;
      for (const Json& t : type.items()) {
        Json sub = s;
        sub["type"] = t;
        if (!body.empty()) body += " | ";
        body += visit(sub, name + "-" + t.as_string());
      }
      return add(name, body);
    }
    const std::string t = type.as_string();
    if (t == "string") {
      if (s.contains("minLength") || s.contains("maxLength")) {
        const int lo = (int)s["minLength"].as_int(0);
        const int hi = s.contains("maxLength") ? (int)s["maxLength"].as_int(0) : -1;
        return add(name, "\"\\\"\" char{" + std::to_string(lo) + "," + (hi >= 0 ? std::to_string(hi) : "") + "} \"\\\"\"");
      }
      if (s.contains("pattern")) {
        // the regex constrains the string's content between the quotes
        std::string sub = regex_to_gbnf(s["pattern"].as_string());
        // rename its rules into this grammar's namespace
        const std::string pre = sanitize(name) + "-re";
        std::istringstream in(sub);
        std::string line, rootname;
        std::vector<std::pair<std::string, std::string>> defs;
        while (std::getline(in, line)) {
          const size_t p = line.find(" ::= ");
          if (p == std::string::npos) continue;
          defs.emplace_back(line.substr(0, p), line.substr(p + 5));
        }
        auto rename = [&](std::string body) {
          for (auto& d : defs) {
            size_t at = 0;
            while ((at = body.find(d.first, at)) != std::string::npos) {
              const bool lb = at == 0 || !(isalnum((unsigned char)body[at - 1]) || body[at - 1] == '-' || body[at - 1] == '$');
              const size_t end = at + d.first.size();
              const bool rb = end >= body.size() || !(isalnum((unsigned char)body[end]) || body[end] == '-' || body[end] == '$');
              if (lb && rb) { body.replace(at, d.first.size(), pre + "-" + d.first); at += pre.size() + 1 + d.first.size(); }
              else at = end;
            }
          }
          return body;
        };
        for (auto& d : defs) add(pre + "-" + d.first, rename(d.second));
        return add(name, "\"\\\"\" " + pre + "-root \"\\\"\"");
      }
      return "string";
    }
    if (t == "integer") return "integer";
    if (t == "number") return "number";
    if (t == "boolean") return "boolean";
    if (t == "null") return add(name, "\"null\"");
    if (t == "array") {
      const std::string item = s.contains("items") ? visit(s["items"], name + "-item") : "value";
      const int lo = (int)s["minItems"].as_int(0);
      const int hi = s.contains("maxItems") ? (int)s["maxItems"].as_int(0) : -1;
      std::string body = "\"[\" ws ";
      if (hi == 0) {
        body += "\"]\"";
      } else if (lo == 0) {
        body += "( " + item + " ( ws \",\" ws " + item + " )" +
                (hi > 0 ? "{0," + std::to_string(hi - 1) + "}" : "*") + " )? ws \"]\"";
      } else {
        body += item + " ( ws \",\" ws " + item + " ){" + std::to_string(lo - 1) + "," +
                (hi > 0 ? std::to_string(hi - 1) : "") + "} ws \"]\"";
      }
      return add(name, body);
    }
    if (t == "object" || s.contains("properties")) {
      const Json& props = s["properties"];
      if (!props.is_object() || props.size() == 0) return "object";
      std::set<std::string> required;
      for (const Json& r : s["required"].items()) required.insert(r.as_string());
      // properties in declaration order; optional ones may be skipped
      std::vector<std::pair<std::string, bool>> kv;   // (rule producing "key": value, required)
      for (const auto& p : props.members()) {
        const std::string vr = visit(p.second, name + "-" + sanitize(p.first));
        const std::string kvr = add(name + "-" + sanitize(p.first) + "-kv",
                                    literal("\"" + p.first + "\"") + " ws \":\" ws " + vr);
        kv.emplace_back(kvr, required.count(p.first) > 0);
      }
      // body(i, need_comma): members i.. given whether one was already emitted
      std::string body = "\"{\" ws " + members(kv, 0, false, name) + " ws \"}\"";
      return add(name, body);
    }
    return "value";
  }

  // Builds the rule for properties [i, n) ; `comma` = a member precedes them.
  std::string members(const std::vector<std::pair<std::string, bool>>& kv, size_t i, bool comma,
                      const std::string& name) {
    if (i >= kv.size()) return "\"\"";
    const std::string key = name + "-m" + std::to_string(i) + (comma ? "c" : "n");
    if (rules_map_.count(key)) return key;
    rules_map_[key] = "";
    rules_.emplace_back(key, "");
    const std::string sep = comma ? "ws \",\" ws " : "";
    std::string with = sep + kv[i].first;
    if (i + 1 < kv.size()) with += " " + members(kv, i + 1, true, name);
    std::string body = with;
    if (!kv[i].second) {
      const std::string without = i + 1 < kv.size() ? members(kv, i + 1, comma, name) : "\"\"";
      body += " | " + without;
    }
    rules_map_[key] = body;
    for (auto& r : rules_) if (r.first == key) r.second = body;
    return key;
  }

  const Json& root_;
  std::vector<std::pair<std::string, std::string>> rules_;
  std::map<std::string, std::string> rules_map_;
  std::set<std::string> in_progress_;
};

// ------------------------------------------------------------------------------ regex
class RegexConverter {
 public:
  explicit RegexConverter(const std::string& p) : s_(p) {}
  std::string run() {
    if (!s_.empty() && s_[0] == '^') ++pos_;
    const std::string top = alternation();
    if (pos_ < s_.size() && s_[pos_] != '$') throw std::runtime_error("regex: unexpected ')' or trailing input");
    std::ostringstream o;
    o << "root ::= " << top << "\n";
    for (auto& r : rules_) o << r.first << " ::= " << r.second << "\n";
    return o.str();
  }

 private:
  std::string fresh(const std::string& body) {
    const std::string n = "r" + std::to_string(rules_.size());
    rules_.emplace_back(n, body);
    return n;
  }
  static std::string cls_char(uint32_t c) {
    char b[16];
    if (c == '\\' || c == ']' || c == '[' || c == '^' || c == '-' || c == '"') { snprintf(b, sizeof b, "\\%c", (char)c); return b; }
    if (c < 0x20 || c == 0x7F) { snprintf(b, sizeof b, "\\x%02X", c); return b; }
    return std::string(1, (char)c);
  }
  std::string alternation() {
    std::string out = sequence();
    while (pos_ < s_.size() && s_[pos_] == '|') {
      ++pos_;
      out += " | " + sequence();
    }
    return out;
  }
  std::string sequence() {
    std::string out;
    while (pos_ < s_.size() && s_[pos_] != '|' && s_[pos_] != ')') {
      if (s_[pos_] == '$' && pos_ + 1 == s_.size()) break;
      std::string a = atom();
      // quantifier
      if (pos_ < s_.size()) {
        const char q = s_[pos_];
        if (q == '*' || q == '+' || q == '?') {
          ++pos_;
          if (pos_ < s_.size() && (s_[pos_] == '?' || s_[pos_] == '+')) ++pos_;   // lazy / possessive: same language
          a = a + q;
        } else if (q == '{') {
          const size_t close = s_.find('}', pos_);
          if (close != std::string::npos) {
            a = a + s_.substr(pos_, close - pos_ + 1);
            pos_ = close + 1;
          }
        }
      }
      out += (out.empty() ? "" : " ") + a;
    }
    return out.empty() ? "\"\"" : out;
  }
  std::string escape_class(char e) {
    switch (e) {
      case 'd': return "[0-9]";
      case 'D': return "[^0-9]";
      case 'w': return "[a-zA-Z0-9_]";
      case 'W': return "[^a-zA-Z0-9_]";
      case 's': return "[ \\t\\n\\r]";
      case 'S': return "[^ \\t\\n\\r]";
      default: return "";
    }
  }
  std::string atom() {
    const char c = s_[pos_];
    if (c == '(') {
      ++pos_;
      if (s_.compare(pos_, 2, "?:") == 0) pos_ += 2;
      const std::string inner = alternation();
      if (pos_ >= s_.size() || s_[pos_] != ')') throw std::runtime_error("regex: missing )");
      ++pos_;
      return fresh(inner);
    }
    if (c == '[') {
      std::string out = "[";
      ++pos_;
      if (pos_ < s_.size() && s_[pos_] == '^') { out += '^'; ++pos_; }
      bool first = true;
      while (pos_ < s_.size() && (s_[pos_] != ']' || first)) {
        first = false;
        if (s_[pos_] == '\\' && pos_ + 1 < s_.size()) {
          const char e = s_[pos_ + 1];
          pos_ += 2;
          const std::string k = escape_class(e);
          if (!k.empty()) out += k.substr(k[1] == '^' ? 2 : 1, k.size() - (k[1] == '^' ? 3 : 2));
          else if (e == 'n') out += "\\n";
          else if (e == 't') out += "\\t";
          else if (e == 'r') out += "\\r";
          else out += cls_char((unsigned char)e);
        } else if (s_[pos_] == '-' ) {
          out += (out.size() > 1 && out.back() != '^' && pos_ + 1 < s_.size() && s_[pos_ + 1] != ']') ? "-" : "\\-";
          ++pos_;
        } else {
          out += cls_char((unsigned char)s_[pos_++]);
        }
      }
      if (pos_ >= s_.size()) throw std::runtime_error("regex: missing ]");
      ++pos_;
      return out + "]";
    }
    if (c == '.') { ++pos_; return "[^\\n]"; }
    if (c == '\\') {
      if (pos_ + 1 >= s_.size()) throw std::runtime_error("regex: dangling backslash");
      const char e = s_[pos_ + 1];
      pos_ += 2;
      const std::string k = escape_class(e);
      if (!k.empty()) return k;
      if (e == 'n') return "\"\\n\"";
      if (e == 't') return "\"\\t\"";
      if (e == 'r') return "\"\\r\"";
      return literal(std::string(1, e));
    }
    // literal run of one UTF-8 character
    size_t n = 1;
    const unsigned char u = (unsigned char)c;
    if (u >= 0xF0) n = 4; else if (u >= 0xE0) n = 3; else if (u >= 0xC0) n = 2;
    const std::string ch = s_.substr(pos_, n);
    pos_ += n;
    return literal(ch);
  }

  const std::string& s_;
  size_t pos_ = 0;
  std::vector<std::pair<std::string, std::string>> rules_;
};

}  // namespace

std::string json_schema_to_gbnf(const Json& schema) { return SchemaConverter(schema).run(); }
std::string regex_to_gbnf(const std::string& pattern) { return RegexConverter(pattern).run(); }

std::shared_ptr<Grammar> Grammar::from_json_schema(const Json& schema) {
  return from_gbnf(json_schema_to_gbnf(schema));
}
std::shared_ptr<Grammar> Grammar::from_json_schema_text(const std::string& text) {
  return from_json_schema(Json::parse(text));
}
std::shared_ptr<Grammar> Grammar::any_json_object() {
  return from_gbnf(std::string("root ::= object\n") + kJsonGbnf);
}
std::shared_ptr<Grammar> Grammar::from_regex(const std::string& pattern) {
  return from_gbnf(regex_to_gbnf(pattern));
}

}  // namespace so
}  // namespace b200
