// Native structured-output engine: a GBNF-style grammar compiled to a rule table over Unicode
// code points, matched by a set of push-down stacks, with a token trie walked depth-first to
// fill per-step token bitmasks. Front ends: GBNF text, JSON schema, "any JSON object", a regex
// subset, literal choices, and lazy (trigger-activated) structural tags for tool calls.
//
// Reference counterparts: src/vllm/v1/structured_output/{manager,backend_native,gbnf_parser,
// json_schema_to_gbnf,regex_to_gbnf}.cpp.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace b200 {
class Json;
namespace so {

// One grammar element. kChar matches one code point against `ranges` (inclusive pairs,
// negated when `negate`); kRule refers to rules[rule].
struct Element {
  enum Kind : uint8_t { kChar, kRule } kind = kChar;
  bool negate = false;
  int rule = -1;
  std::vector<std::pair<uint32_t, uint32_t>> ranges;
  bool matches(uint32_t cp) const;
};
using Sequence = std::vector<Element>;
struct Rule {
  std::string name;
  std::vector<Sequence> alts;
};

class Grammar {
 public:
  // Throws std::runtime_error with a position on malformed input.
  static std::shared_ptr<Grammar> from_gbnf(const std::string& text, const std::string& root = "root");
  static std::shared_ptr<Grammar> from_json_schema(const Json& schema);
  static std::shared_ptr<Grammar> from_json_schema_text(const std::string& schema_json);
  static std::shared_ptr<Grammar> any_json_object();
  static std::shared_ptr<Grammar> from_regex(const std::string& pattern);
  static std::shared_ptr<Grammar> from_choices(const std::vector<std::string>& choices);

  const std::vector<Rule>& rules() const { return rules_; }
  int root() const { return root_; }
  std::string to_gbnf() const;   // normalised text form (for caching keys and tests)

 private:
  friend class GbnfParser;
  std::vector<Rule> rules_;
  int root_ = 0;
};

// Converters exposed for tests and for composing structural tags.
std::string json_schema_to_gbnf(const Json& schema);
std::string regex_to_gbnf(const std::string& pattern);
extern const char* const kJsonGbnf;   // value / object / array / string / number rules

// Position inside an alternative: (rule, alt, index). A stack is the list of positions still
// to be matched, innermost last. An empty stack means the root rule is complete.
struct Pos {
  int rule, alt, idx;
  bool operator==(const Pos& o) const { return rule == o.rule && alt == o.alt && idx == o.idx; }
};
using Stack = std::vector<Pos>;

class Matcher {
 public:
  explicit Matcher(std::shared_ptr<const Grammar> g);
  // Feeds raw bytes (a token's text). Returns false (state unchanged) if they do not fit.
  bool accept_bytes(const std::string& bytes);
  bool can_terminate() const;        // some stack is empty: the root rule may end here
  bool is_dead() const { return stacks_.empty(); }
  void reset();
  // Snapshots for rollback: push after every accepted token, pop to undo.
  void push_checkpoint();
  void rollback(int tokens);
  size_t checkpoints() const { return history_.size(); }

  // --- used by the mask filler (works on a copy of the state) ---
  struct State {
    std::vector<Stack> stacks;
    uint32_t partial_cp = 0;   // bits of an unfinished UTF-8 sequence
    int partial_left = 0;
    uint32_t partial_min = 0;  // smallest code point a sequence of this length may encode
  };
  const State state() const { return State{stacks_, partial_cp_, partial_left_, partial_min_}; }
  // Advance `s` by one byte; returns false if no stack survives.
  bool advance(State* s, uint8_t byte) const;
  bool feasible(const State& s, uint32_t lo, uint32_t hi) const;

 private:
  void expand(const Stack& st, std::vector<Stack>* out) const;
  void advance_cp(const std::vector<Stack>& in, uint32_t cp, std::vector<Stack>* out) const;
  std::shared_ptr<const Grammar> g_;
  std::vector<Stack> stacks_;
  uint32_t partial_cp_ = 0;
  int partial_left_ = 0;
  uint32_t partial_min_ = 0;
  std::vector<State> history_;
};

// Vocabulary trie over token bytes, shared by every request of an engine.
class TokenTrie {
 public:
  // tokens[id] = raw bytes (empty = never allowed, e.g. special tokens).
  explicit TokenTrie(const std::vector<std::string>& tokens);
  // Sets bit id for every token whose bytes are accepted from the matcher's current state.
  void fill_mask(const Matcher& m, uint32_t* mask_words) const;
  int vocab_size() const { return vocab_; }

 private:
  struct Node {
    int first_child = -1, next_sibling = -1;
    uint8_t byte = 0;
    std::vector<int> tokens;   // ids ending here
  };
  void dfs(const Matcher& m, int node, const Matcher::State& st, uint32_t* mask) const;
  std::vector<Node> nodes_;
  int vocab_ = 0;
};

}  // namespace so
}  // namespace b200
