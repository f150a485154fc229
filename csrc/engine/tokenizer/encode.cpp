// BPE merging, text -> ids, ids -> text and the incremental detokenizer.
#include <algorithm>
#include <queue>

#include "tokenizer.h"
#include "unicode_ranges.h"

namespace b200 {
namespace tok {

namespace {
const char kMeta[] = "\xE2\x96\x81";
const char kReplacement[] = "\xEF\xBF\xBD";

// Replaces every malformed UTF-8 sequence with U+FFFD (what a lossy decode shows the user).
std::string lossy_utf8(const std::string& s) {
  bool clean = true;
  for (size_t i = 0; i < s.size();) {
    size_t j = i;
    const uint32_t cp = utf8_next(s, &j);
    if (cp == 0xFFFD && !(j - i == 3)) { clean = false; break; }
    i = j;
  }
  if (clean) return s;
  std::string o;
  o.reserve(s.size() + 8);
  for (size_t i = 0; i < s.size();) {
    size_t j = i;
    const uint32_t cp = utf8_next(s, &j);
    if (cp == 0xFFFD && j - i != 3) o += kReplacement;
    else o.append(s, i, j - i);
    i = j;
  }
  return o;
}

bool ends_with(const std::string& s, const char* tail) {
  const size_t n = std::char_traits<char>::length(tail);
  return s.size() >= n && s.compare(s.size() - n, n, tail) == 0;
}
}  // namespace

// ------------------------------------------------------------------------------ BPE
void Tokenizer::bpe_word(const std::string& word, std::vector<int>* out) const {
  if (word.empty()) return;
  if (ignore_merges_) {
    auto it = token_to_id_.find(word);
    if (it != token_to_id_.end()) { out->push_back(it->second); return; }
  }
  {
    std::lock_guard<std::mutex> lock(cache_mu_);
    auto hit = cache_.find(word);
    if (hit != cache_.end()) {
      out->insert(out->end(), hit->second.begin(), hit->second.end());
      return;
    }
  }
  // initial symbols: one per code point (bytes of unknown characters when byte fallback is on)
  std::vector<int> sym;
  for (size_t i = 0; i < word.size();) {
    size_t j = i;
    utf8_next(word, &j);
    auto it = token_to_id_.find(word.substr(i, j - i));
    if (it != token_to_id_.end()) {
      sym.push_back(it->second);
    } else if (byte_fallback_) {
      for (size_t b = i; b < j; ++b) {
        const int id = byte_token_[(uint8_t)word[b]];
        if (id >= 0) sym.push_back(id);
        else if (unk_id_ >= 0) sym.push_back(unk_id_);
      }
    } else if (unk_id_ >= 0) {
      if (sym.empty() || sym.back() != unk_id_) sym.push_back(unk_id_);
    }
    i = j;
  }
  const int n = (int)sym.size();
  if (n > 1) {
    std::vector<int> prev(n), next(n);
    for (int i = 0; i < n; ++i) { prev[i] = i - 1; next[i] = i + 1 < n ? i + 1 : -1; }
    struct Cand { int rank, pos, left, right, merged; };
    auto worse = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.pos > b.pos; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(worse)> heap(worse);
    auto push = [&](int i) {
      const int j = next[i];
      if (i < 0 || j < 0) return;
      auto m = merges_.find(std::make_pair(sym[i], sym[j]));
      if (m != merges_.end()) heap.push(Cand{m->second.first, i, sym[i], sym[j], m->second.second});
    };
    for (int i = 0; i + 1 < n; ++i) push(i);
    while (!heap.empty()) {
      const Cand c = heap.top();
      heap.pop();
      const int i = c.pos, j = next[i];
      if (sym[i] != c.left || j < 0 || sym[j] != c.right) continue;   // stale entry
      sym[i] = c.merged;
      sym[j] = -1;
      next[i] = next[j];
      if (next[j] >= 0) prev[next[j]] = i;
      if (prev[i] >= 0) push(prev[i]);
      push(i);
    }
  }
  std::vector<int> ids;
  for (int s : sym) if (s >= 0) ids.push_back(s);
  out->insert(out->end(), ids.begin(), ids.end());
  if (word.size() <= 64) {
    std::lock_guard<std::mutex> lock(cache_mu_);
    if (cache_.size() > 200000) cache_.clear();
    cache_.emplace(word, std::move(ids));
  }
}

std::string Tokenizer::normalize(const std::string& text, bool first_segment) const {
  if (!sp_prepend_ && !sp_replace_space_) return text;
  std::string s;
  if (sp_prepend_ && !text.empty() && (first_segment || !sp_prepend_first_only_) &&
      text.compare(0, 3, kMeta) != 0 && !(sp_metaspace_ && text[0] == ' '))
    s = kMeta;   // Metaspace adds its marker only where the text does not already start with one
  if (sp_replace_space_) {
    for (char c : text) {
      if (c == ' ') s += kMeta; else s.push_back(c);
    }
  } else {
    s += text;
  }
  return s;
}

std::vector<std::string> Tokenizer::pretokenize_text(const std::string& text) const {
  return pretokenize(family_, text);
}

void Tokenizer::encode_segment(const std::string& text, bool first_segment, std::vector<int>* out) const {
  if (text.empty()) return;
  if (byte_level_) {
    std::string t = text;
    if (byte_level_prefix_space_ && t[0] != ' ') t.insert(t.begin(), ' ');
    for (const std::string& piece : pretokenize(family_, t)) {
      std::string mapped;
      mapped.reserve(piece.size() * 2);
      for (unsigned char b : piece) utf8_append(byte_to_codepoint(b), &mapped);
      bpe_word(mapped, out);
    }
    return;
  }
  const std::string norm = normalize(text, first_segment);
  if (sp_metaspace_ && !sp_metaspace_split_) {
    bpe_word(norm, out);        // one piece: runs of markers merge ("▁▁", "▁▁▁" are vocabulary entries)
  } else if (sp_metaspace_) {
    // split before every marker; the marker stays with the piece that follows it
    size_t start = 0;
    for (size_t pos = norm.find(kMeta, 1); pos != std::string::npos; pos = norm.find(kMeta, pos + 3)) {
      if (pos > start) bpe_word(norm.substr(start, pos - start), out);
      start = pos;
    }
    bpe_word(norm.substr(start), out);
  } else if (family_ != PreFamily::kNone) {
    for (const std::string& piece : pretokenize(family_, norm)) bpe_word(piece, out);
  } else {
    bpe_word(norm, out);
  }
}

std::vector<int> Tokenizer::encode_ordinary(const std::string& text) const {
  std::vector<int> out;
  encode_segment(text, true, &out);
  return out;
}

std::vector<int> Tokenizer::encode(const std::string& text, bool add_special_tokens) const {
  std::vector<int> out;
  if (add_special_tokens) out = prefix_ids_;
  size_t seg_start = 0, i = 0;
  bool first = true;
  const size_t n = text.size();
  auto flush = [&](size_t end) {
    if (end > seg_start) {
      encode_segment(text.substr(seg_start, end - seg_start), first, &out);
      first = false;
    }
  };
  while (i < n && !added_.empty()) {
    const AddedToken* hit = nullptr;
    for (const AddedToken& a : added_) {   // sorted longest first
      if (a.content[0] == text[i] && text.compare(i, a.content.size(), a.content) == 0) {
        if (a.single_word) {
          auto word_char = [&](size_t k) {
            const unsigned char ch = (unsigned char)text[k];
            return ch >= 0x80 || (ch >= '0' && ch <= '9') || (ch >= 'A' && ch <= 'Z') ||
                   (ch >= 'a' && ch <= 'z') || ch == '_';
          };
          if ((i > 0 && word_char(i - 1)) || (i + a.content.size() < n && word_char(i + a.content.size())))
            continue;
        }
        hit = &a;
        break;
      }
    }
    if (!hit) { ++i; continue; }
    size_t left = i, right = i + hit->content.size();
    if (hit->lstrip) while (left > seg_start && (text[left - 1] == ' ' || text[left - 1] == '\t' || text[left - 1] == '\n')) --left;
    if (hit->rstrip) while (right < n && (text[right] == ' ' || text[right] == '\t' || text[right] == '\n')) ++right;
    flush(left);
    first = false;
    out.push_back(hit->id);
    seg_start = i = right;
  }
  flush(n);
  if (add_special_tokens) out.insert(out.end(), suffix_ids_.begin(), suffix_ids_.end());
  return out;
}

// --------------------------------------------------------------------------- decoding
std::string Tokenizer::token_bytes(int id) const {
  const std::string& t = id_to_token(id);
  if (t.empty()) return t;
  if (id < (int)is_added_.size() && is_added_[id]) return t;
  if (byte_level_) {
    std::string o;
    for (size_t i = 0; i < t.size();) {
      const size_t at = i;
      const uint32_t cp = utf8_next(t, &i);
      const int b = codepoint_to_byte(cp);
      if (b >= 0) o.push_back((char)b);
      else o.append(t, at, i - at);   // not a byte-table character: keep as written
    }
    return o;
  }
  if (byte_fallback_ && t.size() == 6 && t[0] == '<' && t[1] == '0' && t[2] == 'x' && t[5] == '>') {
    auto hv = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'A' && c <= 'F' ? c - 'A' + 10 : c >= 'a' && c <= 'f' ? c - 'a' + 10 : -1; };
    const int hi = hv(t[3]), lo = hv(t[4]);
    if (hi >= 0 && lo >= 0) return std::string(1, (char)(hi * 16 + lo));
  }
  if (sp_replace_space_ || sp_metaspace_) {
    std::string o = t;
    size_t pos = 0;
    while ((pos = o.find(kMeta, pos)) != std::string::npos) o.replace(pos, 3, " ");
    return o;
  }
  return t;
}

std::string Tokenizer::tokens_to_string(const std::vector<int>& ids, size_t first, size_t last,
                                        bool skip_special_tokens) const {
  std::string raw;
  last = std::min(last, ids.size());
  for (size_t i = first; i < last; ++i) {
    if (skip_special_tokens && is_special(ids[i])) continue;
    raw += token_bytes(ids[i]);
  }
  std::string s = lossy_utf8(raw);
  if (dec_strip_leading_space_ && !s.empty() && s[0] == ' ') s.erase(0, 1);
  return s;
}

std::string Tokenizer::decode(const std::vector<int>& ids, bool skip_special_tokens) const {
  return tokens_to_string(ids, 0, ids.size(), skip_special_tokens);
}

// ------------------------------------------------------------------------ detokenizer
namespace {
constexpr size_t kInitialOffset = 5;   // tokens of context kept before the read position

// Byte position that leaves `chars` code points after it (clamped to 0).
size_t back_chars(const std::string& s, size_t chars) {
  size_t pos = s.size();
  while (chars > 0 && pos > 0) {
    --pos;
    while (pos > 0 && ((uint8_t)s[pos] & 0xC0) == 0x80) --pos;
    --chars;
  }
  return pos;
}
size_t count_chars(const std::string& s) {
  size_t n = 0;
  for (unsigned char c : s) if ((c & 0xC0) != 0x80) ++n;
  return n;
}
}  // namespace

IncrementalDetokenizer::IncrementalDetokenizer(const Tokenizer* tok, const std::vector<int>& prompt_ids,
                                               bool skip_special_tokens, std::vector<std::string> stop,
                                               bool include_stop_str_in_output, int min_tokens)
    : tok_(tok), token_ids_(prompt_ids), prompt_len_(prompt_ids.size()), skip_special_(skip_special_tokens),
      stop_(std::move(stop)), include_stop_(include_stop_str_in_output), min_tokens_(min_tokens) {
  const size_t keep = kInitialOffset + 2;
  const size_t from = prompt_ids.size() > keep ? prompt_ids.size() - keep : 0;
  for (size_t i = from; i < prompt_ids.size(); ++i)
    if (!(skip_special_ && tok_ && tok_->is_special(prompt_ids[i]))) window_.push_back(prompt_ids[i]);
  read_offset_ = window_.size();
  prefix_offset_ = read_offset_ > kInitialOffset ? read_offset_ - kInitialOffset : 0;
  if (!stop_.empty() && !include_stop_) {
    size_t longest = 0;
    for (const std::string& s : stop_) longest = std::max(longest, count_chars(s));
    stop_buffer_len_ = longest > 0 ? longest - 1 : 0;
  }
}

std::string IncrementalDetokenizer::decode_next(int id) {
  if (!tok_) return "";
  if (skip_special_ && tok_->is_special(id)) return "";
  window_.push_back(id);
  const std::string prefix_text = tok_->tokens_to_string(window_, prefix_offset_, read_offset_, false);
  std::string new_text = tok_->tokens_to_string(window_, prefix_offset_, window_.size(), false);
  if (new_text.size() <= prefix_text.size() || ends_with(new_text, kReplacement)) return "";
  prefix_offset_ = read_offset_;
  read_offset_ = window_.size();
  // bound the window: everything before the prefix offset is never read again
  if (prefix_offset_ > 64) {
    window_.erase(window_.begin(), window_.begin() + (long)prefix_offset_);
    read_offset_ -= prefix_offset_;
    prefix_offset_ = 0;
  }
  return new_text.substr(prefix_text.size());
}

bool IncrementalDetokenizer::update(const std::vector<int>& new_ids, bool stop_terminated,
                                    std::string* stop_str) {
  if (new_ids.empty()) return false;
  size_t n = new_ids.size();
  int skipped = -1;
  if (stop_terminated && !include_stop_) { skipped = new_ids[n - 1]; --n; }
  size_t stop_check_offset = output_text_.size();
  for (size_t i = 0; i < n; ++i) {
    token_ids_.push_back(new_ids[i]);
    output_text_ += decode_next(new_ids[i]);
    if (min_tokens_ > 0 && (int)num_output_tokens() <= min_tokens_) stop_check_offset = output_text_.size();
  }
  if (skipped >= 0) token_ids_.push_back(skipped);
  if (stop_.empty() || (int)num_output_tokens() <= min_tokens_) return false;
  const size_t new_bytes = output_text_.size() - stop_check_offset;
  if (new_bytes == 0) return false;
  for (const std::string& s : stop_) {
    if (s.empty()) continue;
    // a match must end inside the new text, so it cannot start before this position
    const size_t window = new_bytes + s.size() - 1;
    const size_t start = output_text_.size() > window ? output_text_.size() - window : 0;
    size_t idx = output_text_.find(s, start);
    if (idx == std::string::npos) continue;
    if (include_stop_) {
      idx += s.size();
      if (idx < output_text_.size()) output_text_.resize(idx);
    } else {
      output_text_.resize(idx);
    }
    if (stop_str) *stop_str = s;
    return true;
  }
  return false;
}

std::string IncrementalDetokenizer::get_next_output_text(bool finished, bool delta) {
  const size_t hold = finished ? 0 : stop_buffer_len_;
  const size_t length = hold ? back_chars(output_text_, hold) : output_text_.size();
  if (!delta) return output_text_.substr(0, length);
  if (last_output_len_ < length) {
    std::string piece = output_text_.substr(last_output_len_, length - last_output_len_);
    last_output_len_ = length;
    return piece;
  }
  return "";
}

}  // namespace tok
}  // namespace b200
