// Tokenizer: byte-level BPE (GPT-2 / Qwen / Llama-3 / DeepSeek / OLMo families) and
// SentencePiece-style BPE with byte fallback (Llama-2 / Mistral / Gemma), built from a Hugging
// Face `tokenizer.json` or from GGUF vocabulary arrays, plus the incremental detokenizer the
// engine streams text with.
//
// The reference project covers the same ground in `src/vllm/tokenizer/{tokenizer,pretokenizer,
// bpe,unicode_data}.cpp` and `src/vllm/v1/engine/detokenizer.cpp`. The pre-tokenizer here is a
// set of hand-written scanners, one per regex family, over generated Unicode range tables.
#pragma once
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace b200 {
class Json;
namespace tok {

// Which split pattern the checkpoint's pre-tokenizer uses.
enum class PreFamily {
  kNone,        // no regex split (SentencePiece-style models)
  kGpt2,        // 's|'t|... | ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
  kLlama3,      // cl100k-like, case-insensitive contractions, \p{N}{1,3}
  kQwen2,       // cl100k-like with single-digit \p{N}
  kQwen35,      // Qwen2 pattern with combining marks counted as letters
  kDeepseekV3,  // \p{N}{1,3} | CJK runs | cl100k-like tail with [!-/:-~...] punctuation class
  kDeepseekV2,  // sequence of five splits ([\r\n], letters, punctuation, \s+$, CJK, \p{N}+)
};

struct AddedToken {
  std::string content;
  int id = -1;
  bool special = false;
  bool lstrip = false, rstrip = false;
  bool single_word = false;
  bool normalized = false;
};

// Splits `text` (UTF-8) into the pieces the family's regex would produce.
std::vector<std::string> pretokenize(PreFamily family, const std::string& text);
// Guesses the family from the regex source(s) found in tokenizer.json.
PreFamily family_from_pattern(const std::string& pattern);
// The GGUF `tokenizer.ggml.pre` name -> family.
PreFamily family_from_gguf_pre(const std::string& pre);

// GPT-2 byte <-> printable code point table.
uint32_t byte_to_codepoint(uint8_t b);
int codepoint_to_byte(uint32_t cp);  // -1 when cp is not in the table

// UTF-8 helpers shared with the detokenizer and the grammar engine.
uint32_t utf8_next(const std::string& s, size_t* pos);  // U+FFFD on malformed input
void utf8_append(uint32_t cp, std::string* out);
size_t utf8_incomplete_tail(const std::string& s);      // bytes of an unfinished sequence at the end

class Tokenizer {
 public:
  // `tokenizer_json` is the text of tokenizer.json; `config_json` (may be empty) the text of
  // tokenizer_config.json, which supplies add_bos_token/bos/eos/chat_template overrides.
  static std::unique_ptr<Tokenizer> from_hf_json(const std::string& tokenizer_json,
                                                 const std::string& config_json = "");
  // Reads <dir>/tokenizer.json (+ tokenizer_config.json when present).
  static std::unique_ptr<Tokenizer> from_dir(const std::string& dir);
  // GGUF vocabulary: `model` is tokenizer.ggml.model ("gpt2" = byte-level BPE, "llama" =
  // SentencePiece-style), `token_types` follow llama.cpp (3 = control, 4 = user defined,
  // 6 = byte).
  static std::unique_ptr<Tokenizer> from_gguf(const std::string& model, const std::string& pre,
                                              const std::vector<std::string>& tokens,
                                              const std::vector<std::string>& merges,
                                              const std::vector<int>& token_types, int bos_id,
                                              int eos_id, bool add_bos, bool add_eos);

  std::vector<int> encode(const std::string& text, bool add_special_tokens = true) const;
  // Encodes without looking for added/special tokens inside `text`.
  std::vector<int> encode_ordinary(const std::string& text) const;
  std::string decode(const std::vector<int>& ids, bool skip_special_tokens = true) const;

  // Text of tokens[first:last) the way the model's decoder chain produces it (malformed UTF-8
  // becomes U+FFFD, SentencePiece-style decoders drop one leading space): the detokenizer's
  // building block.
  std::string tokens_to_string(const std::vector<int>& ids, size_t first, size_t last,
                               bool skip_special_tokens) const;
  // The raw bytes one token contributes to the output (byte-level and byte-fallback aware).
  std::string token_bytes(int id) const;

  int vocab_size() const { return (int)id_to_token_.size(); }
  const std::string& id_to_token(int id) const;
  int token_to_id(const std::string& t) const;
  bool is_special(int id) const { return id >= 0 && id < (int)special_.size() && special_[id]; }
  int bos_id() const { return bos_id_; }
  int eos_id() const { return eos_id_; }
  int pad_id() const { return pad_id_; }
  int unk_id() const { return unk_id_; }
  bool adds_bos() const { return !prefix_ids_.empty(); }
  bool byte_level() const { return byte_level_; }
  PreFamily family() const { return family_; }
  const std::string& chat_template() const { return chat_template_; }
  const std::vector<AddedToken>& added_tokens() const { return added_; }
  std::vector<std::string> pretokenize_text(const std::string& text) const;

 private:
  Tokenizer() = default;
  void finish_setup();
  void bpe_word(const std::string& word, std::vector<int>* out) const;
  void encode_segment(const std::string& text, bool first_segment, std::vector<int>* out) const;
  std::string normalize(const std::string& text, bool first_segment) const;

  struct PairHash {
    size_t operator()(const std::pair<int, int>& p) const {
      return ((size_t)(uint32_t)p.first << 32 | (uint32_t)p.second) * 0x9e3779b97f4a7c15ull;
    }
  };

  std::vector<std::string> id_to_token_;
  std::unordered_map<std::string, int> token_to_id_;
  std::unordered_map<std::pair<int, int>, std::pair<int, int>, PairHash> merges_;  // -> (rank, id)
  std::vector<AddedToken> added_;
  std::vector<uint8_t> special_;
  std::vector<uint8_t> is_added_;
  std::vector<int> byte_token_;       // byte-fallback: <0xXX> ids (256) or empty
  std::vector<int> prefix_ids_, suffix_ids_;
  PreFamily family_ = PreFamily::kNone;
  bool byte_level_ = false;           // ByteLevel pre-tokenizer/decoder
  bool byte_fallback_ = false;
  bool ignore_merges_ = false;
  bool sp_prepend_ = false;           // normalizer prepends U+2581 to the text
  bool sp_replace_space_ = false;     // normalizer maps ' ' to U+2581
  bool sp_metaspace_ = false;         // Metaspace pre-tokenizer (split on U+2581)
  bool sp_metaspace_split_ = true;    // "split": false keeps the text whole, so merges may span markers
  bool sp_prepend_first_only_ = false;  // marker only before the first segment of the text
  bool dec_strip_leading_space_ = false;
  bool nfc_ = false;
  bool byte_level_prefix_space_ = false;
  int bos_id_ = -1, eos_id_ = -1, pad_id_ = -1, unk_id_ = -1;
  std::string chat_template_;
  mutable std::unordered_map<std::string, std::vector<int>> cache_;   // word -> ids
  mutable std::mutex cache_mu_;
};

// Incremental detokenizer with the semantics of vLLM's slow path: text is re-derived from a
// short window of trailing tokens; output that ends in an incomplete UTF-8 sequence (it would
// render as U+FFFD) is held back until the next token completes it; stop strings are searched
// in the newly produced characters and text that could still become a stop string is held
// back from streaming.
class IncrementalDetokenizer {
 public:
  IncrementalDetokenizer(const Tokenizer* tok, const std::vector<int>& prompt_ids,
                         bool skip_special_tokens, std::vector<std::string> stop,
                         bool include_stop_str_in_output, int min_tokens = 0);
  // Appends tokens; returns true (and sets *stop_str) when a stop string matched. When
  // `stop_terminated` the last token is an EOS/stop token and is not turned into text.
  bool update(const std::vector<int>& new_ids, bool stop_terminated, std::string* stop_str);
  // Cumulative or delta text available for the client; when not finished the tail that could
  // still be the start of a stop string stays hidden.
  std::string get_next_output_text(bool finished, bool delta);
  const std::string& output_text() const { return output_text_; }
  const std::vector<int>& token_ids() const { return token_ids_; }
  size_t num_output_tokens() const { return token_ids_.size() - prompt_len_; }

 private:
  std::string decode_next(int id);
  const Tokenizer* tok_;
  std::vector<int> token_ids_;
  std::vector<int> window_;   // trailing prompt tokens + generated tokens that produce text
  size_t prompt_len_;
  size_t prefix_offset_, read_offset_;
  bool skip_special_;
  std::vector<std::string> stop_;
  bool include_stop_;
  int min_tokens_;
  size_t stop_buffer_len_ = 0;
  std::string output_text_;
  size_t last_output_len_ = 0;
};

}  // namespace tok
}  // namespace b200
