// Tokenizer construction (tokenizer.json / GGUF), BPE merging, encode and decode.
#include "tokenizer.h"

#include <algorithm>
#include <fstream>
#include <queue>
#include <sstream>
#include <stdexcept>

#include "../util/json.h"

namespace b200 {
namespace tok {

namespace {
const char kMeta[] = "\xE2\x96\x81";  // U+2581, the SentencePiece space marker

std::string read_file(const std::string& path, bool required) {
  std::ifstream f(path, std::ios::binary);
  if (!f) {
    if (required) throw std::runtime_error("cannot open " + path);
    return "";
  }
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

void replace_all(std::string* s, const std::string& from, const std::string& to) {
  if (from.empty()) return;
  size_t pos = 0;
  while ((pos = s->find(from, pos)) != std::string::npos) {
    s->replace(pos, from.size(), to);
    pos += to.size();
  }
}

// Collects every Split regex source and the component types below a pre_tokenizer node.
void walk_pretokenizer(const Json& node, std::string* patterns, bool* byte_level, bool* bl_regex,
                       bool* metaspace, bool* digits, bool* bl_prefix_space) {
  if (!node.is_object()) return;
  const std::string& type = node["type"].as_string();
  if (type == "Sequence") {
    for (const Json& c : node["pretokenizers"].items())
      walk_pretokenizer(c, patterns, byte_level, bl_regex, metaspace, digits, bl_prefix_space);
  } else if (type == "Split") {
    const Json& pat = node["pattern"];
    const std::string& re = pat["Regex"].as_string();
    *patterns += re.empty() ? pat["String"].as_string() : re;
    *patterns += "\n";
  } else if (type == "ByteLevel") {
    *byte_level = true;
    if (node["use_regex"].as_bool(true)) *bl_regex = true;
    if (node["add_prefix_space"].as_bool(false)) *bl_prefix_space = true;
  } else if (type == "Metaspace") {
    *metaspace = true;
  } else if (type == "Digits") {
    *digits = true;
  }
}

std::string token_name(const Json& v) {
  if (v.is_string()) return v.as_string();
  if (v.is_object()) return v["content"].as_string();
  return "";
}
}  // namespace

// --------------------------------------------------------------------------- building
std::unique_ptr<Tokenizer> Tokenizer::from_dir(const std::string& dir) {
  return from_hf_json(read_file(dir + "/tokenizer.json", true),
                      read_file(dir + "/tokenizer_config.json", false));
}

std::unique_ptr<Tokenizer> Tokenizer::from_hf_json(const std::string& tokenizer_json,
                                                   const std::string& config_json) {
  Json root = Json::parse(tokenizer_json);
  const Json& model = root["model"];
  const std::string& mtype = model["type"].as_string();
  if (!mtype.empty() && mtype != "BPE")
    throw std::runtime_error("tokenizer model type '" + mtype + "' is not supported (BPE only)");
  std::unique_ptr<Tokenizer> t(new Tokenizer());

  // vocabulary
  int max_id = -1;
  for (const auto& kv : model["vocab"].members()) max_id = std::max(max_id, (int)kv.second.as_int(-1));
  for (const Json& a : root["added_tokens"].items()) max_id = std::max(max_id, (int)a["id"].as_int(-1));
  t->id_to_token_.assign((size_t)max_id + 1, std::string());
  t->token_to_id_.reserve((size_t)max_id * 2 + 16);
  for (const auto& kv : model["vocab"].members()) {
    const int id = (int)kv.second.as_int(-1);
    if (id < 0) continue;
    t->id_to_token_[id] = kv.first;
    t->token_to_id_[kv.first] = id;
  }
  t->special_.assign((size_t)max_id + 1, 0);
  t->is_added_.assign((size_t)max_id + 1, 0);
  for (const Json& a : root["added_tokens"].items()) {
    AddedToken at;
    at.content = a["content"].as_string();
    at.id = (int)a["id"].as_int(-1);
    at.special = a["special"].as_bool(false);
    at.lstrip = a["lstrip"].as_bool(false);
    at.rstrip = a["rstrip"].as_bool(false);
    at.single_word = a["single_word"].as_bool(false);
    at.normalized = a["normalized"].as_bool(false);
    if (at.id < 0 || at.content.empty()) continue;
    t->id_to_token_[at.id] = at.content;
    t->token_to_id_[at.content] = at.id;
    t->special_[at.id] = at.special;
    t->is_added_[at.id] = 1;
    t->added_.push_back(std::move(at));
  }

  // merges: "a b" strings or [a, b] pairs; rank = position
  int rank = 0;
  for (const Json& m : model["merges"].items()) {
    std::string a, b;
    if (m.is_string()) {
      const std::string& s = m.as_string();
      const size_t sp = s.find(' ');
      if (sp == std::string::npos) { ++rank; continue; }
      a = s.substr(0, sp);
      b = s.substr(sp + 1);
    } else {
      a = m[(size_t)0].as_string();
      b = m[(size_t)1].as_string();
    }
    auto ia = t->token_to_id_.find(a), ib = t->token_to_id_.find(b), im = t->token_to_id_.find(a + b);
    if (ia != t->token_to_id_.end() && ib != t->token_to_id_.end() && im != t->token_to_id_.end())
      t->merges_.emplace(std::make_pair(ia->second, ib->second), std::make_pair(rank, im->second));
    ++rank;
  }
  t->byte_fallback_ = model["byte_fallback"].as_bool(false);
  t->ignore_merges_ = model["ignore_merges"].as_bool(false);
  if (model["unk_token"].is_string()) t->unk_id_ = t->token_to_id(model["unk_token"].as_string());

  // pre-tokenizer
  std::string patterns;
  bool bl = false, bl_regex = false, metaspace = false, digits = false, bl_prefix = false;
  walk_pretokenizer(root["pre_tokenizer"], &patterns, &bl, &bl_regex, &metaspace, &digits, &bl_prefix);
  t->byte_level_ = bl;
  t->byte_level_prefix_space_ = bl_prefix;
  t->sp_metaspace_ = metaspace;
  if (!patterns.empty()) t->family_ = family_from_pattern(patterns);
  else if (bl && bl_regex) t->family_ = PreFamily::kGpt2;
  else t->family_ = PreFamily::kNone;
  if (metaspace) {
    const Json& pt = root["pre_tokenizer"];
    // Metaspace both replaces spaces and (unless prepend_scheme == "never") prepends the marker
    t->sp_replace_space_ = true;
    const std::string& scheme = pt["prepend_scheme"].as_string();
    t->sp_prepend_ = scheme.empty() ? pt["add_prefix_space"].as_bool(true) : (scheme != "never");
    t->sp_prepend_first_only_ = (scheme == "first");
    t->sp_metaspace_split_ = pt["split"].as_bool(true);
  }

  // normalizer
  std::vector<const Json*> norms;
  const Json& norm = root["normalizer"];
  if (norm["type"].as_string() == "Sequence") for (const Json& c : norm["normalizers"].items()) norms.push_back(&c);
  else if (norm.is_object()) norms.push_back(&norm);
  for (const Json* c : norms) {
    const std::string& ty = (*c)["type"].as_string();
    if (ty == "Prepend" && (*c)["prepend"].as_string() == kMeta) t->sp_prepend_ = true;
    else if (ty == "Replace" && (*c)["pattern"]["String"].as_string() == " " && (*c)["content"].as_string() == kMeta)
      t->sp_replace_space_ = true;
    else if (ty == "NFC") t->nfc_ = true;
  }

  // decoder
  std::vector<const Json*> decs;
  const Json& dec = root["decoder"];
  if (dec["type"].as_string() == "Sequence") for (const Json& c : dec["decoders"].items()) decs.push_back(&c);
  else if (dec.is_object()) decs.push_back(&dec);
  for (const Json* c : decs) {
    const std::string& ty = (*c)["type"].as_string();
    if (ty == "ByteLevel") t->byte_level_ = true;
    else if (ty == "Strip" && (*c)["content"].as_string() == " " && (*c)["start"].as_int(0) >= 1)
      t->dec_strip_leading_space_ = true;
    else if (ty == "Metaspace") {
      const std::string& scheme = (*c)["prepend_scheme"].as_string();
      t->dec_strip_leading_space_ = scheme.empty() ? (*c)["add_prefix_space"].as_bool(true) : (scheme != "never");
    }
  }

  // post-processor: the "single" template gives the ids added around one sequence
  std::vector<const Json*> posts;
  const Json& post = root["post_processor"];
  if (post["type"].as_string() == "Sequence") for (const Json& c : post["processors"].items()) posts.push_back(&c);
  else if (post.is_object()) posts.push_back(&post);
  for (const Json* c : posts) {
    if ((*c)["type"].as_string() != "TemplateProcessing") continue;
    bool seen_seq = false;
    for (const Json& piece : (*c)["single"].items()) {
      if (piece.contains("Sequence")) { seen_seq = true; continue; }
      const int id = t->token_to_id(piece["SpecialToken"]["id"].as_string());
      if (id < 0) continue;
      (seen_seq ? t->suffix_ids_ : t->prefix_ids_).push_back(id);
    }
  }

  // tokenizer_config.json overrides
  if (!config_json.empty()) {
    Json cfg;
    if (Json::try_parse(config_json, &cfg)) {
      const std::string bos = token_name(cfg["bos_token"]), eos = token_name(cfg["eos_token"]);
      const std::string pad = token_name(cfg["pad_token"]), unk = token_name(cfg["unk_token"]);
      if (!bos.empty()) t->bos_id_ = t->token_to_id(bos);
      if (!eos.empty()) t->eos_id_ = t->token_to_id(eos);
      if (!pad.empty()) t->pad_id_ = t->token_to_id(pad);
      if (!unk.empty() && t->unk_id_ < 0) t->unk_id_ = t->token_to_id(unk);
      if (cfg["chat_template"].is_string()) t->chat_template_ = cfg["chat_template"].as_string();
      // Llama-style fast tokenizers rebuild the template from these flags
      if (cfg.contains("add_bos_token") && posts.empty()) {
        if (cfg["add_bos_token"].as_bool(false) && t->bos_id_ >= 0) t->prefix_ids_ = {t->bos_id_};
      }
      if (cfg.contains("add_bos_token") && !cfg["add_bos_token"].as_bool(true)) t->prefix_ids_.clear();
      if (cfg["add_eos_token"].as_bool(false) && t->eos_id_ >= 0 && t->suffix_ids_.empty())
        t->suffix_ids_ = {t->eos_id_};
    }
  }
  if (t->bos_id_ < 0 && !t->prefix_ids_.empty()) t->bos_id_ = t->prefix_ids_[0];
  t->finish_setup();
  return t;
}

std::unique_ptr<Tokenizer> Tokenizer::from_gguf(const std::string& model, const std::string& pre,
                                                const std::vector<std::string>& tokens,
                                                const std::vector<std::string>& merges,
                                                const std::vector<int>& token_types, int bos_id,
                                                int eos_id, bool add_bos, bool add_eos) {
  std::unique_ptr<Tokenizer> t(new Tokenizer());
  const size_t n = tokens.size();
  t->id_to_token_ = tokens;
  t->special_.assign(n, 0);
  t->is_added_.assign(n, 0);
  t->token_to_id_.reserve(n * 2);
  for (size_t i = 0; i < n; ++i) t->token_to_id_.emplace(tokens[i], (int)i);
  for (size_t i = 0; i < n && i < token_types.size(); ++i) {
    const int ty = token_types[i];
    if (ty == 3 || ty == 4) {   // control / user defined: matched verbatim in the text
      AddedToken at;
      at.content = tokens[i];
      at.id = (int)i;
      at.special = (ty == 3);
      t->special_[i] = at.special;
      t->is_added_[i] = 1;
      t->added_.push_back(std::move(at));
    }
  }
  if (model == "gpt2") {
    t->byte_level_ = true;
    t->family_ = family_from_gguf_pre(pre);
    t->ignore_merges_ = (t->family_ == PreFamily::kLlama3);
  } else {   // "llama": SentencePiece-style vocabulary with <0xXX> byte pieces
    t->byte_fallback_ = true;
    t->sp_prepend_ = true;
    t->sp_replace_space_ = true;
    t->dec_strip_leading_space_ = true;
    t->family_ = PreFamily::kNone;
    for (size_t i = 0; i < n && i < token_types.size(); ++i)
      if (token_types[i] == 2 && t->unk_id_ < 0) t->unk_id_ = (int)i;
  }
  int rank = 0;
  for (const std::string& s : merges) {
    const size_t sp = s.find(' ', 1);   // a merge's left side is never empty
    if (sp != std::string::npos) {
      auto ia = t->token_to_id_.find(s.substr(0, sp)), ib = t->token_to_id_.find(s.substr(sp + 1));
      auto im = t->token_to_id_.find(s.substr(0, sp) + s.substr(sp + 1));
      if (ia != t->token_to_id_.end() && ib != t->token_to_id_.end() && im != t->token_to_id_.end())
        t->merges_.emplace(std::make_pair(ia->second, ib->second), std::make_pair(rank, im->second));
    }
    ++rank;
  }
  t->bos_id_ = bos_id;
  t->eos_id_ = eos_id;
  if (add_bos && bos_id >= 0) t->prefix_ids_ = {bos_id};
  if (add_eos && eos_id >= 0) t->suffix_ids_ = {eos_id};
  t->finish_setup();
  return t;
}

void Tokenizer::finish_setup() {
  if (byte_fallback_) {
    byte_token_.assign(256, -1);
    static const char* hex = "0123456789ABCDEF";
    for (int b = 0; b < 256; ++b) {
      std::string name = "<0x";
      name.push_back(hex[b >> 4]);
      name.push_back(hex[b & 15]);
      name.push_back('>');
      byte_token_[b] = token_to_id(name);
    }
  }
  // longest content first so that the scan in encode() prefers the longest added token
  std::stable_sort(added_.begin(), added_.end(), [](const AddedToken& a, const AddedToken& b) {
    return a.content.size() > b.content.size();
  });
}

const std::string& Tokenizer::id_to_token(int id) const {
  static const std::string kEmpty;
  return (id >= 0 && id < (int)id_to_token_.size()) ? id_to_token_[id] : kEmpty;
}

int Tokenizer::token_to_id(const std::string& t) const {
  auto it = token_to_id_.find(t);
  return it == token_to_id_.end() ? -1 : it->second;
}

}  // namespace tok
}  // namespace b200
