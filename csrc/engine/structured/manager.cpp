#include "manager.h"

#include <algorithm>
#include <stdexcept>

#include "../util/json.h"

namespace b200 {
namespace so {

StructuredOutputManager::StructuredOutputManager(std::vector<std::string> token_bytes, int vocab_size,
                                                 std::vector<int> eos_ids)
    : tokens_(std::move(token_bytes)), vocab_(std::max(vocab_size, (int)tokens_.size())),
      eos_(std::move(eos_ids)), trie_(tokens_) {}

std::shared_ptr<Grammar> StructuredOutputManager::compile(const StructuredOutputsParams& p) {
  std::string key;
  if (p.json) key = "json:" + *p.json;
  else if (p.regex) key = "regex:" + *p.regex;
  else if (p.grammar) key = "gbnf:" + *p.grammar;
  else if (p.choice) { key = "choice:"; for (auto& c : *p.choice) { key += c; key.push_back('\x1f'); } }
  else if (p.json_object) key = "json_object";
  else throw std::runtime_error("no structured-output constraint given");
  {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = cache_.find(key);
    if (it != cache_.end()) return it->second;
  }
  std::shared_ptr<Grammar> g;
  if (p.json) g = Grammar::from_json_schema_text(*p.json);
  else if (p.regex) g = Grammar::from_regex(*p.regex);
  else if (p.grammar) g = Grammar::from_gbnf(*p.grammar);
  else if (p.choice) g = Grammar::from_choices(*p.choice);
  else g = Grammar::any_json_object();
  std::lock_guard<std::mutex> lock(mu_);
  if (cache_.size() > 256) cache_.clear();
  cache_[key] = g;
  return g;
}

std::unique_ptr<RequestGrammar> StructuredOutputManager::make_state(const StructuredOutputsParams& p) {
  auto st = std::make_unique<RequestGrammar>();
  try {
    if (p.structural_tag) {
      // {"structures": [{"begin": s, "schema": {...} | "grammar": gbnf, "end": s}], "triggers": [s]}
      Json tag = Json::parse(*p.structural_tag);
      st->lazy = true;
      for (const Json& t : tag["triggers"].items()) st->triggers.push_back(t.as_string());
      for (const Json& s : tag["structures"].items()) {
        Structure sx;
        sx.begin = s["begin"].as_string();
        sx.end = s["end"].as_string();
        if (s.contains("grammar")) sx.body_gbnf = s["grammar"].as_string();
        else sx.body_gbnf = json_schema_to_gbnf(s["schema"]);
        sx.body = Grammar::from_gbnf(sx.body_gbnf);   // validates
        st->structures.push_back(std::move(sx));
      }
      if (st->triggers.empty())
        for (auto& sx : st->structures) st->triggers.push_back(sx.begin);
    } else {
      st->grammar = compile(p);
      st->matcher = std::make_unique<Matcher>(st->grammar);
    }
  } catch (const std::exception& e) {
    st->invalid = true;
    st->error = e.what();
  }
  return st;
}

RequestGrammar* StructuredOutputManager::state_of(Request& req) {
  return reinterpret_cast<RequestGrammar*>(req.structured_state);
}

bool StructuredOutputManager::grammar_ready(Request& req) {
  if (req.structured_state) return true;
  if (!req.sampling_params.structured_outputs) return true;
  auto st = make_state(*req.sampling_params.structured_outputs);
  req.structured_state = st.get();
  std::lock_guard<std::mutex> lock(mu_);
  states_[req.request_id] = std::move(st);
  return true;
}

// The structure(s) whose `begin` starts with `trigger` become the active grammar:
// root ::= (rest-of-begin body end) | ...
void StructuredOutputManager::enter_structure(RequestGrammar& st, const std::string& trigger,
                                              const std::string& after) {
  std::string text = "root ::= ";
  std::string bodies;
  int n = 0;
  for (size_t i = 0; i < st.structures.size(); ++i) {
    const Structure& sx = st.structures[i];
    if (sx.begin.compare(0, trigger.size(), trigger) != 0) continue;
    std::string rest, end;
    Json::escape(sx.begin.substr(trigger.size()), rest);
    Json::escape(sx.end, end);
    if (n++) text += " | ";
    const std::string pre = "s" + std::to_string(i) + "-";
    text += rest + " " + pre + "root " + end;
    // prefix the body's rule names
    std::string body = sx.body_gbnf;
    std::vector<std::string> names;
    size_t pos = 0;
    while (pos < body.size()) {
      size_t eol = body.find('\n', pos);
      if (eol == std::string::npos) eol = body.size();
      const size_t def = body.find(" ::= ", pos);
      if (def != std::string::npos && def < eol) names.push_back(body.substr(pos, def - pos));
      pos = eol + 1;
    }
    std::sort(names.begin(), names.end(), [](const std::string& a, const std::string& b) { return a.size() > b.size(); });
    auto is_name = [](char c) { return isalnum((unsigned char)c) || c == '-' || c == '_' || c == '$'; };
    std::string out;
    for (size_t at = 0; at < body.size();) {
      bool rep = false;
      // only outside string literals / classes: cheap check by scanning state
      for (const std::string& nm : names) {
        if (body.compare(at, nm.size(), nm) == 0 && (at == 0 || !is_name(body[at - 1])) &&
            (at + nm.size() >= body.size() || !is_name(body[at + nm.size()]))) {
          // skip matches inside a quoted literal
          size_t q = 0;
          const size_t line = body.rfind('\n', at) == std::string::npos ? 0 : body.rfind('\n', at) + 1;
          bool in_str = false, in_cls = false;
          for (q = line; q < at; ++q) {
            if (body[q] == '\\') { ++q; continue; }
            if (!in_cls && body[q] == '"') in_str = !in_str;
            else if (!in_str && body[q] == '[') in_cls = true;
            else if (!in_str && body[q] == ']') in_cls = false;
          }
          if (in_str || in_cls) break;
          out += pre + nm;
          at += nm.size();
          rep = true;
          break;
        }
      }
      if (!rep) out.push_back(body[at++]);
    }
    bodies += out;
    if (bodies.empty() || bodies.back() != '\n') bodies.push_back('\n');
  }
  if (n == 0) return;
  text += "\n" + bodies;
  st.grammar = Grammar::from_gbnf(text);
  st.matcher = std::make_unique<Matcher>(st.grammar);
  if (!after.empty() && !st.matcher->accept_bytes(after)) {
    // the token ran past the trigger with text the structure does not allow: stay free
    st.matcher.reset();
    st.grammar.reset();
  }
}

bool StructuredOutputManager::accept(RequestGrammar& st, int32_t token) {
  if (st.invalid || st.terminated) return true;
  if (std::find(eos_.begin(), eos_.end(), token) != eos_.end()) {
    st.terminated = true;
    return true;
  }
  const std::string& bytes = (token >= 0 && token < (int)tokens_.size()) ? tokens_[token] : std::string();
  if (st.lazy && !st.matcher) {
    st.tail += bytes;
    st.free_history.push_back(true);
    for (const std::string& trg : st.triggers) {
      const size_t at = st.tail.rfind(trg);
      // the trigger must end inside the bytes just added (older text was checked before)
      if (at != std::string::npos && at + trg.size() > st.tail.size() - bytes.size()) {
        enter_structure(st, trg, st.tail.substr(at + trg.size()));
        st.tail.clear();
        break;
      }
    }
    if (st.tail.size() > 256) st.tail.erase(0, st.tail.size() - 128);
    return true;
  }
  if (!st.matcher) return true;
  if (!st.matcher->accept_bytes(bytes)) return false;
  st.matcher->push_checkpoint();
  if (st.lazy) {
    st.free_history.push_back(false);
    // structure complete and nothing more can follow: back to free text
    if (st.matcher->can_terminate()) {
      Matcher::State s = st.matcher->state();
      bool only_empty = true;
      for (auto& stack : s.stacks) if (!stack.empty()) { only_empty = false; break; }
      if (only_empty) { st.matcher.reset(); st.grammar.reset(); }
    }
  }
  return true;
}

bool StructuredOutputManager::accept_tokens(Request& req, const std::vector<int32_t>& tokens) {
  RequestGrammar* st = state_of(req);
  if (!st) return true;
  for (int32_t t : tokens)
    if (!accept(*st, t)) return false;
  return true;
}

void StructuredOutputManager::rollback(Request& req, int num_tokens) {
  RequestGrammar* st = state_of(req);
  if (!st || num_tokens <= 0 || !st->matcher) return;
  st->matcher->rollback(num_tokens);
  st->terminated = false;
}

std::vector<uint32_t> StructuredOutputManager::mask_for(RequestGrammar& st) {
  const int words = words_per_row();
  std::vector<uint32_t> row((size_t)words, 0u);
  auto allow_eos = [&]() { for (int e : eos_) if (e >= 0 && e < vocab_) row[e >> 5] |= 1u << (e & 31); };
  if (st.invalid || st.terminated) { allow_eos(); return row; }
  if (!st.matcher) {                       // free text
    std::fill(row.begin(), row.end(), 0xffffffffu);
    return row;
  }
  trie_.fill_mask(*st.matcher, row.data());
  if (st.matcher->can_terminate() || st.matcher->is_dead()) {
    if (st.lazy) {
      // a finished structure may be followed by anything
      if (st.matcher->can_terminate()) std::fill(row.begin(), row.end(), 0xffffffffu);
    }
    allow_eos();
  }
  return row;
}

GrammarOutput StructuredOutputManager::grammar_bitmask(const std::vector<RequestPtr>& reqs,
                                                       const std::map<std::string, std::vector<int32_t>>&) {
  GrammarOutput g;
  g.words_per_row = words_per_row();
  for (const RequestPtr& r : reqs) {
    RequestGrammar* st = state_of(*r);
    if (!st) continue;
    g.structured_output_request_ids.push_back(r->request_id);
    std::vector<uint32_t> row = mask_for(*st);
    for (uint32_t w : row) g.bitmask.push_back((int32_t)w);
  }
  return g;
}

void StructuredOutputManager::release(Request& req) {
  req.structured_state = nullptr;
  std::lock_guard<std::mutex> lock(mu_);
  states_.erase(req.request_id);
}

bool StructuredOutputManager::is_terminated(Request& req) {
  RequestGrammar* st = state_of(req);
  return st && st->terminated;
}

}  // namespace so
}  // namespace b200
