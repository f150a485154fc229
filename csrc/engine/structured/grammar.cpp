// GBNF parser, push-down matcher and token-trie mask fill.
#include "grammar.h"

#include <algorithm>
#include <map>
#include <sstream>
#include <stdexcept>

#include "../util/json.h"

namespace b200 {
namespace so {

bool Element::matches(uint32_t cp) const {
  bool hit = false;
  for (const auto& r : ranges)
    if (cp >= r.first && cp <= r.second) { hit = true; break; }
  return hit != negate;
}

// ------------------------------------------------------------------------------ parser
class GbnfParser {
 public:
  GbnfParser(const std::string& text, Grammar* g) : s_(text), g_(g) {}

  void parse(const std::string& root) {
    skip_ws(true);
    while (pos_ < s_.size()) {
      parse_rule();
      skip_ws(true);
    }
    for (const auto& r : g_->rules_)
      if (r.alts.empty()) fail("rule '" + r.name + "' is referenced but never defined");
    auto it = ids_.find(root);
    if (it == ids_.end()) fail("no '" + root + "' rule");
    g_->root_ = it->second;
  }

 private:
  [[noreturn]] void fail(const std::string& msg) const {
    throw std::runtime_error("grammar error at offset " + std::to_string(pos_) + ": " + msg);
  }
  int rule_id(const std::string& name) {
    auto it = ids_.find(name);
    if (it != ids_.end()) return it->second;
    const int id = (int)g_->rules_.size();
    g_->rules_.push_back(Rule{name, {}});
    ids_[name] = id;
    return id;
  }
  int fresh_rule(const std::string& base) {
    return rule_id(base + "$" + std::to_string(counter_++));
  }
  void skip_ws(bool newlines) {
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (c == '#') { while (pos_ < s_.size() && s_[pos_] != '\n') ++pos_; }
      else if (c == ' ' || c == '\t' || (newlines && (c == '\n' || c == '\r'))) ++pos_;
      else break;
    }
  }
  static bool name_char(char c) {
    return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '-' || c == '_';
  }
  std::string parse_name() {
    const size_t b = pos_;
    while (pos_ < s_.size() && name_char(s_[pos_])) ++pos_;
    if (pos_ == b) fail("expected a rule name");
    return s_.substr(b, pos_ - b);
  }
  uint32_t utf8_cp() {
    const unsigned char c = (unsigned char)s_[pos_];
    int n = c < 0x80 ? 1 : c < 0xE0 ? 2 : c < 0xF0 ? 3 : 4;
    uint32_t cp = n == 1 ? c : c & (0xFF >> (n + 1));
    for (int i = 1; i < n && pos_ + i < s_.size(); ++i) cp = (cp << 6) | ((unsigned char)s_[pos_ + i] & 0x3F);
    pos_ += n;
    return cp;
  }
  uint32_t parse_char() {   // one (possibly escaped) character inside "..." or [...]
    if (pos_ >= s_.size()) fail("unexpected end");
    if (s_[pos_] != '\\') return utf8_cp();
    ++pos_;
    if (pos_ >= s_.size()) fail("dangling escape");
    const char e = s_[pos_++];
    auto hex = [&](int n) {
      uint32_t v = 0;
      for (int i = 0; i < n; ++i) {
        if (pos_ >= s_.size()) fail("short hex escape");
        const char c = s_[pos_++];
        v <<= 4;
        if (c >= '0' && c <= '9') v |= c - '0';
        else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
        else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
        else fail("bad hex digit");
      }
      return v;
    };
    switch (e) {
      case 'n': return '\n'; case 'r': return '\r'; case 't': return '\t';
      case 'x': return hex(2); case 'u': return hex(4); case 'U': return hex(8);
      default: return (unsigned char)e;   // \" \\ \[ \] \- ...
    }
  }
  void parse_rule() {
    const std::string name = parse_name();
    skip_ws(false);
    if (s_.compare(pos_, 3, "::=") != 0) fail("expected ::=");
    pos_ += 3;
    skip_ws(true);
    const int id = rule_id(name);
    if (!g_->rules_[id].alts.empty()) fail("rule '" + name + "' defined twice");
    std::vector<Sequence> alts = parse_alternatives(name, false);
    g_->rules_[id].alts = std::move(alts);
  }
  std::vector<Sequence> parse_alternatives(const std::string& base, bool nested) {
    std::vector<Sequence> alts;
    alts.push_back(parse_sequence(base, nested));
    while (pos_ < s_.size() && s_[pos_] == '|') {
      ++pos_;
      skip_ws(true);
      alts.push_back(parse_sequence(base, nested));
    }
    return alts;
  }
  // item{m,n} on the last `count` elements of seq
  void apply_repeat(const std::string& base, Sequence* seq, size_t start, int lo, int hi) {
    Sequence item(seq->begin() + (long)start, seq->end());
    seq->resize(start);
    // sub: item as its own rule when it is more than one element
    auto ref = [&](int rid) { Element e; e.kind = Element::kRule; e.rule = rid; return e; };
    Element unit;
    if (item.size() == 1) unit = item[0];
    else {
      const int rid = fresh_rule(base);
      g_->rules_[rid].alts = {item};
      unit = ref(rid);
    }
    for (int i = 0; i < lo; ++i) seq->push_back(unit);
    if (hi < 0) {          // unbounded tail: star ::= unit star | (empty)
      const int star = fresh_rule(base);
      g_->rules_[star].alts = {Sequence{unit, ref(star)}, Sequence{}};
      seq->push_back(ref(star));
    } else if (hi > lo) {  // up to hi-lo optional copies, nested so that they stay ordered
      int next = -1;
      for (int i = 0; i < hi - lo; ++i) {
        const int opt = fresh_rule(base);
        Sequence with{unit};
        if (next >= 0) with.push_back(ref(next));
        g_->rules_[opt].alts = {with, Sequence{}};
        next = opt;
      }
      seq->push_back(ref(next));
    }
  }
  Sequence parse_sequence(const std::string& base, bool nested) {
    Sequence seq;
    size_t last_start = 0;
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (c == '"') {
        ++pos_;
        last_start = seq.size();
        while (pos_ < s_.size() && s_[pos_] != '"') {
          const uint32_t cp = parse_char();
          Element e;
          e.ranges.push_back({cp, cp});
          seq.push_back(e);
        }
        if (pos_ >= s_.size()) fail("unterminated string literal");
        ++pos_;
        skip_ws(nested);
      } else if (c == '[') {
        ++pos_;
        Element e;
        if (pos_ < s_.size() && s_[pos_] == '^') { e.negate = true; ++pos_; }
        while (pos_ < s_.size() && s_[pos_] != ']') {
          const uint32_t lo = parse_char();
          uint32_t hi = lo;
          if (pos_ + 1 < s_.size() && s_[pos_] == '-' && s_[pos_ + 1] != ']') {
            ++pos_;
            hi = parse_char();
          }
          e.ranges.push_back({lo, hi});
        }
        if (pos_ >= s_.size()) fail("unterminated character class");
        ++pos_;
        last_start = seq.size();
        seq.push_back(e);
        skip_ws(nested);
      } else if (c == '.') {
        ++pos_;
        Element e;
        e.negate = true;                 // anything
        last_start = seq.size();
        seq.push_back(e);
        skip_ws(nested);
      } else if (c == '(') {
        ++pos_;
        skip_ws(true);
        const int rid = fresh_rule(base);
        std::vector<Sequence> alts = parse_alternatives(base, true);
        g_->rules_[rid].alts = std::move(alts);
        if (pos_ >= s_.size() || s_[pos_] != ')') fail("expected )");
        ++pos_;
        Element e;
        e.kind = Element::kRule;
        e.rule = rid;
        last_start = seq.size();
        seq.push_back(e);
        skip_ws(nested);
      } else if (name_char(c)) {
        // a name followed by ::= starts the next rule
        const size_t save = pos_;
        const std::string name = parse_name();
        size_t look = pos_;
        while (look < s_.size() && (s_[look] == ' ' || s_[look] == '\t')) ++look;
        if (s_.compare(look, 3, "::=") == 0) { pos_ = save; break; }
        Element e;
        e.kind = Element::kRule;
        e.rule = rule_id(name);
        last_start = seq.size();
        seq.push_back(e);
        skip_ws(nested);
      } else if (c == '*' || c == '+' || c == '?') {
        if (seq.size() == last_start) fail("nothing to repeat");
        ++pos_;
        apply_repeat(base, &seq, last_start, c == '+' ? 1 : 0, c == '?' ? 1 : -1);
        last_start = seq.size();
        skip_ws(nested);
      } else if (c == '{') {
        if (seq.size() == last_start) fail("nothing to repeat");
        ++pos_;
        auto num = [&]() {
          int v = 0;
          bool any = false;
          while (pos_ < s_.size() && s_[pos_] >= '0' && s_[pos_] <= '9') { v = v * 10 + (s_[pos_++] - '0'); any = true; }
          return any ? v : -1;
        };
        int lo = num(), hi = lo;
        if (lo < 0) fail("expected a repeat count");
        if (pos_ < s_.size() && s_[pos_] == ',') { ++pos_; hi = num(); }
        if (pos_ >= s_.size() || s_[pos_] != '}') fail("expected }");
        ++pos_;
        if (hi >= 0 && hi < lo) fail("bad repeat range");
        apply_repeat(base, &seq, last_start, lo, hi);
        last_start = seq.size();
        skip_ws(nested);
      } else if (c == '\n' || c == '\r') {
        // a newline ends the rule unless the next line continues with '|'
        const size_t save = pos_;
        skip_ws(true);
        if (pos_ < s_.size() && s_[pos_] == '|') continue;
        if (nested) continue;
        pos_ = save;
        skip_ws(true);
        break;
      } else {
        break;   // ')' or '|' or end
      }
    }
    return seq;
  }

  const std::string& s_;
  Grammar* g_;
  size_t pos_ = 0;
  int counter_ = 0;
  std::map<std::string, int> ids_;
};

std::shared_ptr<Grammar> Grammar::from_gbnf(const std::string& text, const std::string& root) {
  auto g = std::make_shared<Grammar>();
  GbnfParser(text, g.get()).parse(root);
  return g;
}

static void write_cp(std::ostringstream& o, uint32_t cp) {
  if (cp == '\n') o << "\\n";
  else if (cp == '\r') o << "\\r";
  else if (cp == '\t') o << "\\t";
  else if (cp == '"' || cp == '\\' || cp == '[' || cp == ']' || cp == '-' || cp == '^') o << '\\' << (char)cp;
  else if (cp >= 0x20 && cp < 0x7F) o << (char)cp;
  else { char b[16]; snprintf(b, sizeof b, cp > 0xFFFF ? "\\U%08X" : "\\u%04X", cp); o << b; }
}

std::string Grammar::to_gbnf() const {
  std::ostringstream o;
  for (const Rule& r : rules_) {
    o << r.name << " ::= ";
    for (size_t a = 0; a < r.alts.size(); ++a) {
      if (a) o << " | ";
      if (r.alts[a].empty()) o << "\"\"";
      for (size_t i = 0; i < r.alts[a].size(); ++i) {
        const Element& e = r.alts[a][i];
        if (i) o << ' ';
        if (e.kind == Element::kRule) o << rules_[e.rule].name;
        else {
          o << '[' << (e.negate ? "^" : "");
          for (auto& rg : e.ranges) {
            write_cp(o, rg.first);
            if (rg.second != rg.first) { o << '-'; write_cp(o, rg.second); }
          }
          o << ']';
        }
      }
    }
    o << "\n";
  }
  return o.str();
}

std::shared_ptr<Grammar> Grammar::from_choices(const std::vector<std::string>& choices) {
  std::string text = "root ::= ";
  for (size_t i = 0; i < choices.size(); ++i) {
    if (i) text += " | ";
    std::string lit;
    Json::escape(choices[i], lit);   // JSON string escaping is a valid GBNF literal
    text += lit;
  }
  return from_gbnf(text);
}

// ------------------------------------------------------------------------------ matcher
Matcher::Matcher(std::shared_ptr<const Grammar> g) : g_(std::move(g)) { reset(); }

void Matcher::reset() {
  stacks_.clear();
  history_.clear();
  partial_cp_ = 0;
  partial_left_ = 0;
  const Rule& root = g_->rules()[g_->root()];
  for (int a = 0; a < (int)root.alts.size(); ++a) {
    Stack st;
    st.push_back(Pos{g_->root(), a, 0});
    expand(st, &stacks_);
  }
}

// Resolves the top of `st` until it points at a character element (or the stack is empty) and
// appends the resulting stacks (one per alternative taken) to `out`, without duplicates.
void Matcher::expand(const Stack& st, std::vector<Stack>* out) const {
  if (st.empty()) {
    if (std::find(out->begin(), out->end(), st) == out->end()) out->push_back(st);
    return;
  }
  const Pos top = st.back();
  const Sequence& seq = g_->rules()[top.rule].alts[top.alt];
  if (top.idx >= (int)seq.size()) {           // alternative finished: pop
    Stack rest(st.begin(), st.end() - 1);
    expand(rest, out);
    return;
  }
  const Element& e = seq[top.idx];
  if (e.kind == Element::kChar) {
    if (std::find(out->begin(), out->end(), st) == out->end()) out->push_back(st);
    return;
  }
  // rule reference: continue after it once the referenced rule completes
  Stack base(st.begin(), st.end() - 1);
  base.push_back(Pos{top.rule, top.alt, top.idx + 1});
  if (base.size() > 512) return;              // runaway left recursion
  const Rule& r = g_->rules()[e.rule];
  for (int a = 0; a < (int)r.alts.size(); ++a) {
    Stack next = base;
    next.push_back(Pos{e.rule, a, 0});
    expand(next, out);
  }
}

void Matcher::advance_cp(const std::vector<Stack>& in, uint32_t cp, std::vector<Stack>* out) const {
  for (const Stack& st : in) {
    if (st.empty()) continue;
    const Pos top = st.back();
    const Element& e = g_->rules()[top.rule].alts[top.alt][top.idx];
    if (!e.matches(cp)) continue;
    Stack next = st;
    next.back().idx++;
    expand(next, out);
  }
}

// Can some stack still match a code point in [lo, hi]? Used for unfinished UTF-8 sequences,
// so that a lead byte is only allowed where a character of its range is.
bool Matcher::feasible(const State& s, uint32_t lo, uint32_t hi) const {
  for (const Stack& st : s.stacks) {
    if (st.empty()) continue;
    const Pos top = st.back();
    const Element& e = g_->rules()[top.rule].alts[top.alt][top.idx];
    if (!e.negate) {
      for (const auto& r : e.ranges)
        if (r.first <= hi && r.second >= lo) return true;
    } else {
      bool covered = false;   // excluded entirely only if one range spans the whole interval
      for (const auto& r : e.ranges)
        if (r.first <= lo && r.second >= hi) { covered = true; break; }
      if (!covered) return true;
    }
  }
  return false;
}

bool Matcher::advance(State* s, uint8_t byte) const {
  auto partial_ok = [&]() {
    const int sh = 6 * s->partial_left;
    uint32_t lo = s->partial_cp << sh;
    const uint32_t hi = lo | ((1u << sh) - 1);
    if (lo < s->partial_min) lo = s->partial_min;     // overlong encodings are not characters
    return hi >= lo && feasible(*s, lo, hi);
  };
  if (s->partial_left > 0) {
    if ((byte & 0xC0) != 0x80) return false;
    s->partial_cp = (s->partial_cp << 6) | (byte & 0x3F);
    if (--s->partial_left > 0) return partial_ok();
  } else if (byte < 0x80) {
    s->partial_cp = byte;
    s->partial_min = 0;
  } else if (byte >= 0xC2 && byte <= 0xDF) {
    s->partial_cp = byte & 0x1F; s->partial_left = 1; s->partial_min = 0x80; return partial_ok();
  } else if (byte >= 0xE0 && byte <= 0xEF) {
    s->partial_cp = byte & 0x0F; s->partial_left = 2; s->partial_min = 0x800; return partial_ok();
  } else if (byte >= 0xF0 && byte <= 0xF4) {
    s->partial_cp = byte & 0x07; s->partial_left = 3; s->partial_min = 0x10000; return partial_ok();
  } else {
    return false;
  }
  if (s->partial_cp < s->partial_min && s->partial_cp >= 0x80) return false;
  std::vector<Stack> next;
  advance_cp(s->stacks, s->partial_cp, &next);
  s->stacks.swap(next);
  s->partial_cp = 0;
  return !s->stacks.empty();
}

bool Matcher::accept_bytes(const std::string& bytes) {
  State s = state();
  for (unsigned char b : bytes)
    if (!advance(&s, b)) return false;
  stacks_.swap(s.stacks);
  partial_cp_ = s.partial_cp;
  partial_left_ = s.partial_left;
  partial_min_ = s.partial_min;
  return true;
}

bool Matcher::can_terminate() const {
  if (partial_left_ > 0) return false;
  for (const Stack& s : stacks_)
    if (s.empty()) return true;
  return false;
}

void Matcher::push_checkpoint() {
  history_.push_back(state());
  if (history_.size() > 64) history_.erase(history_.begin());
}

void Matcher::rollback(int tokens) {
  // history_[k] is the state AFTER token k was accepted; undoing n tokens restores the state
  // before them, i.e. the checkpoint n+1 from the end (or the start state).
  if (tokens <= 0) return;
  if ((size_t)tokens >= history_.size()) {
    const bool had = !history_.empty();
    reset();
    (void)had;
    return;
  }
  history_.resize(history_.size() - (size_t)tokens);
  const State& s = history_.back();
  stacks_ = s.stacks;
  partial_cp_ = s.partial_cp;
  partial_left_ = s.partial_left;
  partial_min_ = s.partial_min;
}

// ------------------------------------------------------------------------------ trie
TokenTrie::TokenTrie(const std::vector<std::string>& tokens) : vocab_((int)tokens.size()) {
  nodes_.push_back(Node{});
  for (int id = 0; id < (int)tokens.size(); ++id) {
    const std::string& t = tokens[id];
    if (t.empty()) continue;
    int cur = 0;
    for (unsigned char b : t) {
      int child = nodes_[cur].first_child;
      while (child >= 0 && nodes_[child].byte != b) child = nodes_[child].next_sibling;
      if (child < 0) {
        child = (int)nodes_.size();
        Node n;
        n.byte = b;
        n.next_sibling = nodes_[cur].first_child;
        nodes_.push_back(n);
        nodes_[cur].first_child = child;
      }
      cur = child;
    }
    nodes_[cur].tokens.push_back(id);
  }
}

void TokenTrie::dfs(const Matcher& m, int node, const Matcher::State& st, uint32_t* mask) const {
  for (int child = nodes_[node].first_child; child >= 0; child = nodes_[child].next_sibling) {
    Matcher::State next = st;
    if (!m.advance(&next, nodes_[child].byte)) continue;
    for (int id : nodes_[child].tokens) mask[id >> 5] |= 1u << (id & 31);
    if (nodes_[child].first_child >= 0) dfs(m, child, next, mask);
  }
}

void TokenTrie::fill_mask(const Matcher& m, uint32_t* mask_words) const {
  dfs(m, 0, m.state(), mask_words);
}

}  // namespace so
}  // namespace b200
