// Structured-output manager: compiles each request's constraint into a grammar (cached by its
// text), keeps one matcher per request, advances it with the sampled tokens and fills the
// per-step token bitmasks the sampler applies. Lazy "structural tags" constrain only the
// spans that follow a trigger string (tool calls inside free text).
//
// Reference: src/vllm/v1/structured_output/manager.cpp (grammar_init, grammar_bitmask,
// should_advance), backend_native.cpp.
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../core/scheduler.h"
#include "grammar.h"

namespace b200 {
namespace so {

struct Structure {   // one entry of a structural tag
  std::string begin, end;
  std::shared_ptr<Grammar> body;   // grammar of the span between begin and end
  std::string body_gbnf;
};

struct RequestGrammar {
  std::shared_ptr<Grammar> grammar;       // eager constraint (null for lazy requests)
  std::unique_ptr<Matcher> matcher;       // null while a lazy request is in free text
  bool terminated = false;
  bool invalid = false;                   // the constraint failed to compile
  std::string error;
  // lazy mode
  bool lazy = false;
  std::vector<std::string> triggers;
  std::vector<Structure> structures;
  std::string tail;                       // recent free text (for trigger detection)
  std::vector<bool> free_history;         // per accepted token: was it consumed in free text
};

class StructuredOutputManager : public StructuredOutputHook {
 public:
  // token_bytes[id]: the bytes a token contributes (empty for special / unused ids);
  // vocab_size: width of the model's logits (>= token_bytes.size()).
  StructuredOutputManager(std::vector<std::string> token_bytes, int vocab_size, std::vector<int> eos_ids);

  bool grammar_ready(Request& req) override;
  bool accept_tokens(Request& req, const std::vector<int32_t>& tokens) override;
  void rollback(Request& req, int num_tokens) override;
  GrammarOutput grammar_bitmask(const std::vector<RequestPtr>& reqs,
                                const std::map<std::string, std::vector<int32_t>>& spec) override;
  void release(Request& req) override;
  bool is_terminated(Request& req) override;

  // Compiles a constraint without a request (validation at the API boundary). Throws.
  std::shared_ptr<Grammar> compile(const StructuredOutputsParams& p);
  // Stand-alone helpers for tests / tools.
  std::vector<uint32_t> mask_for(RequestGrammar& st);
  std::unique_ptr<RequestGrammar> make_state(const StructuredOutputsParams& p);
  bool accept(RequestGrammar& st, int32_t token);
  int words_per_row() const { return (vocab_ + 31) / 32; }

 private:
  RequestGrammar* state_of(Request& req);
  void enter_structure(RequestGrammar& st, const std::string& trigger, const std::string& after);
  std::vector<std::string> tokens_;
  int vocab_;
  std::vector<int> eos_;
  TokenTrie trie_;
  std::mutex mu_;
  std::map<std::string, std::shared_ptr<Grammar>> cache_;
  std::map<std::string, std::unique_ptr<RequestGrammar>> states_;
};

}  // namespace so
}  // namespace b200
