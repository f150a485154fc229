// Hand-written scanners for the split regexes of the supported tokenizer families. Each
// scanner answers "how many code points does the pattern match at position i" with the
// leftmost-alternative, greedy-with-backtracking semantics of the regex it stands for.
#include <algorithm>
#include <cstring>

#include "tokenizer.h"
#include "unicode_ranges.h"

namespace b200 {
namespace tok {

using unicode::is_cased;
using unicode::is_letter;
using unicode::is_mark;
using unicode::is_number;
using unicode::is_punct;
using unicode::is_space;

// ------------------------------------------------------------------------------- UTF-8
uint32_t utf8_next(const std::string& s, size_t* pos) {
  const size_t n = s.size();
  size_t i = *pos;
  const uint8_t c = (uint8_t)s[i];
  auto cont = [&](size_t k) { return k < n && ((uint8_t)s[k] & 0xC0) == 0x80; };
  if (c < 0x80) { *pos = i + 1; return c; }
  if (c >= 0xC2 && c <= 0xDF && cont(i + 1)) {
    *pos = i + 2;
    return ((c & 0x1F) << 6) | ((uint8_t)s[i + 1] & 0x3F);
  }
  if (c >= 0xE0 && c <= 0xEF && cont(i + 1) && cont(i + 2)) {
    uint32_t cp = ((c & 0x0F) << 12) | (((uint8_t)s[i + 1] & 0x3F) << 6) | ((uint8_t)s[i + 2] & 0x3F);
    if (cp >= 0x800 && !(cp >= 0xD800 && cp <= 0xDFFF)) { *pos = i + 3; return cp; }
  }
  if (c >= 0xF0 && c <= 0xF4 && cont(i + 1) && cont(i + 2) && cont(i + 3)) {
    uint32_t cp = ((c & 0x07) << 18) | (((uint8_t)s[i + 1] & 0x3F) << 12) |
                  (((uint8_t)s[i + 2] & 0x3F) << 6) | ((uint8_t)s[i + 3] & 0x3F);
    if (cp >= 0x10000 && cp <= 0x10FFFF) { *pos = i + 4; return cp; }
  }
  *pos = i + 1;
  return 0xFFFD;
}

void utf8_append(uint32_t cp, std::string* o) {
  if (cp < 0x80) o->push_back((char)cp);
  else if (cp < 0x800) { o->push_back((char)(0xC0 | (cp >> 6))); o->push_back((char)(0x80 | (cp & 63))); }
  else if (cp < 0x10000) {
    o->push_back((char)(0xE0 | (cp >> 12)));
    o->push_back((char)(0x80 | ((cp >> 6) & 63)));
    o->push_back((char)(0x80 | (cp & 63)));
  } else {
    o->push_back((char)(0xF0 | (cp >> 18)));
    o->push_back((char)(0x80 | ((cp >> 12) & 63)));
    o->push_back((char)(0x80 | ((cp >> 6) & 63)));
    o->push_back((char)(0x80 | (cp & 63)));
  }
}

size_t utf8_incomplete_tail(const std::string& s) {
  // Looks at up to the last three bytes for a lead byte whose sequence is not complete yet.
  const size_t n = s.size();
  for (size_t back = 1; back <= 3 && back <= n; ++back) {
    const uint8_t c = (uint8_t)s[n - back];
    if ((c & 0xC0) == 0x80) continue;           // continuation byte: keep looking for its lead
    size_t need = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
    return need > back ? back : 0;
  }
  return 0;
}

// ------------------------------------------------------------------------ byte <-> char
static const uint32_t* byte_table() {
  static uint32_t table[256];
  static bool init = false;
  if (!init) {
    int extra = 0;
    for (int b = 0; b < 256; ++b) {
      const bool printable = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      table[b] = printable ? (uint32_t)b : (uint32_t)(256 + extra++);
    }
    init = true;
  }
  return table;
}
uint32_t byte_to_codepoint(uint8_t b) { return byte_table()[b]; }
int codepoint_to_byte(uint32_t cp) {
  static int inv[512];
  static bool init = false;
  if (!init) {
    for (int i = 0; i < 512; ++i) inv[i] = -1;
    for (int b = 0; b < 256; ++b) inv[byte_table()[b]] = b;
    init = true;
  }
  return cp < 512 ? inv[cp] : -1;
}

// --------------------------------------------------------------------------- scanners
namespace {

struct Cps {
  std::vector<uint32_t> cp;
  std::vector<uint32_t> off;  // byte offset of each code point; off[n] = text size
  explicit Cps(const std::string& s) {
    size_t i = 0;
    while (i < s.size()) {
      off.push_back((uint32_t)i);
      cp.push_back(utf8_next(s, &i));
    }
    off.push_back((uint32_t)s.size());
  }
};

inline bool is_nl(uint32_t x) { return x == '\r' || x == '\n'; }

inline uint32_t fold(uint32_t x) {
  if (x >= 'A' && x <= 'Z') return x + 32;
  if (x == 0x17F) return 's';   // LATIN SMALL LETTER LONG S case-folds to 's'
  if (x == 0x212A) return 'k';
  return x;
}

// 's|'t|'re|'ve|'m|'ll|'d at position i (after the apostrophe check)
size_t contraction(const std::vector<uint32_t>& c, size_t i, size_t n, bool icase) {
  if (c[i] != '\'' || i + 1 >= n) return 0;
  auto at = [&](size_t k) { return icase ? fold(c[k]) : c[k]; };
  const uint32_t a = at(i + 1);
  if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
  if (i + 2 < n) {
    const uint32_t b = at(i + 2);
    if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
  }
  return 0;
}

// The three whitespace alternatives shared by every family: \s*[\r\n]+ (when `newline_alt`),
// \s+(?!\S), \s+.
size_t whitespace_tail(const std::vector<uint32_t>& c, size_t i, size_t n, bool newline_alt) {
  size_t e = i;
  while (e < n && is_space(c[e])) ++e;
  if (e == i) return 0;
  if (newline_alt) {
    for (size_t k = e; k > i; --k)
      if (is_nl(c[k - 1])) return k - i;
  }
  if (e == n) return e - i;
  if (e - i >= 2) return e - i - 1;
  return e - i;
}

size_t match_gpt2(const std::vector<uint32_t>& c, size_t i, size_t n) {
  if (size_t m = contraction(c, i, n, false)) return m;
  const size_t j = (c[i] == ' ' && i + 1 < n) ? i + 1 : i;
  size_t k = j;
  if (is_letter(c[j])) {
    while (k < n && is_letter(c[k])) ++k;
    return k - i;
  }
  if (is_number(c[j])) {
    while (k < n && is_number(c[k])) ++k;
    return k - i;
  }
  if (!is_space(c[j])) {
    while (k < n && !is_space(c[k]) && !is_letter(c[k]) && !is_number(c[k])) ++k;
    return k - i;
  }
  return whitespace_tail(c, i, n, false);
}

// cl100k-shaped pattern; max_digits = digits per number piece; marks = \p{M} joins \p{L}.
size_t match_cl100k(const std::vector<uint32_t>& c, size_t i, size_t n, int max_digits, bool marks) {
  auto L = [&](uint32_t x) { return is_letter(x) || (marks && is_mark(x)); };
  if (size_t m = contraction(c, i, n, true)) return m;
  const uint32_t x = c[i];
  {  // [^\r\n\p{L}\p{N}]?\p{L}+
    const size_t j = (!is_nl(x) && !is_letter(x) && !is_number(x)) ? i + 1 : i;
    size_t k = j;
    while (k < n && L(c[k])) ++k;
    if (k > j) return k - i;
    if (j != i) {
      k = i;
      while (k < n && L(c[k])) ++k;
      if (k > i) return k - i;
    }
  }
  if (is_number(x)) {
    size_t k = i;
    while (k < n && (int)(k - i) < max_digits && is_number(c[k])) ++k;
    return k - i;
  }
  {  //  ?[^\s\p{L}\p{N}]+[\r\n]*
    const size_t j = (x == ' ') ? i + 1 : i;
    size_t k = j;
    while (k < n && !is_space(c[k]) && !L(c[k]) && !is_number(c[k])) ++k;
    if (k > j) {
      while (k < n && is_nl(c[k])) ++k;
      return k - i;
    }
  }
  if (size_t m = whitespace_tail(c, i, n, true)) return m;
  return 1;
}

inline bool ascii_punct(uint32_t x) {
  return (x >= '!' && x <= '/') || (x >= ':' && x <= '@') || (x >= '[' && x <= '`') || (x >= '{' && x <= '~');
}
inline bool ascii_alpha(uint32_t x) { return (x >= 'A' && x <= 'Z') || (x >= 'a' && x <= 'z'); }

// DeepSeek-V3 main pattern. Returns 0 where nothing matches (the caller keeps such code
// points as a gap piece).
size_t match_deepseek3(const std::vector<uint32_t>& c, size_t i, size_t n) {
  const uint32_t x = c[i];
  auto LM = [&](uint32_t y) { return is_letter(y) || is_mark(y); };
  if (ascii_punct(x) && i + 1 < n && ascii_alpha(c[i + 1])) {
    size_t k = i + 1;
    while (k < n && ascii_alpha(c[k])) ++k;
    return k - i;
  }
  {  // [^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+
    const size_t j = (!is_nl(x) && !is_letter(x) && !is_punct(x)) ? i + 1 : i;
    size_t k = j;
    while (k < n && LM(c[k])) ++k;
    if (k > j) return k - i;
    if (j != i) {
      k = i;
      while (k < n && LM(c[k])) ++k;
      if (k > i) return k - i;
    }
  }
  {  //  ?[\p{P}\p{S}]+[\r\n]*
    const size_t j = (x == ' ') ? i + 1 : i;
    size_t k = j;
    while (k < n && is_punct(c[k])) ++k;
    if (k > j) {
      while (k < n && is_nl(c[k])) ++k;
      return k - i;
    }
  }
  return whitespace_tail(c, i, n, true);
}

inline bool cjk_v3(uint32_t x) { return (x >= 0x4E00 && x <= 0x9FA5) || (x >= 0x3040 && x <= 0x30FF); }
inline bool cjk_v2(uint32_t x) { return (x >= 0x0800 && x <= 0x9FA5) || (x >= 0xAC00 && x <= 0xD7FF); }
inline bool punct_v2(uint32_t x) {
  return (x >= 0x21 && x <= 0x2F) || (x >= 0x3A && x <= 0x7E) || (x >= 0xFF01 && x <= 0xFF0F) ||
         (x >= 0xFF1A && x <= 0xFF5E) || (x >= 0x2018 && x <= 0x201F) || (x >= 0x3000 && x <= 0x3002);
}

using Span = std::pair<size_t, size_t>;  // [first, second) in code points

// Applies one "isolated" split: every match becomes its own piece, text between matches is
// kept as pieces too. `m(c, i, end)` gives the match length at i within [i, end).
template <class Matcher>
std::vector<Span> split_isolated(const std::vector<uint32_t>& c, const std::vector<Span>& in, Matcher m) {
  std::vector<Span> out;
  for (const Span& s : in) {
    size_t gap = s.first, i = s.first;
    while (i < s.second) {
      const size_t len = m(c, i, s.second);
      if (len == 0) { ++i; continue; }
      if (gap < i) out.emplace_back(gap, i);
      out.emplace_back(i, i + len);
      i += len;
      gap = i;
    }
    if (gap < s.second) out.emplace_back(gap, s.second);
  }
  return out;
}

size_t run_of(const std::vector<uint32_t>& c, size_t i, size_t n, bool (*pred)(uint32_t), size_t max_len) {
  size_t k = i;
  while (k < n && k - i < max_len && pred(c[k])) ++k;
  return k - i;
}

}  // namespace

std::vector<std::string> pretokenize(PreFamily family, const std::string& text) {
  std::vector<std::string> out;
  if (text.empty()) return out;
  if (family == PreFamily::kNone) {
    out.push_back(text);
    return out;
  }
  Cps t(text);
  const std::vector<uint32_t>& c = t.cp;
  const size_t n = c.size();
  auto emit = [&](size_t a, size_t b) { out.emplace_back(text, t.off[a], t.off[b] - t.off[a]); };

  if (family == PreFamily::kDeepseekV3 || family == PreFamily::kDeepseekV2) {
    std::vector<Span> spans{{0, n}};
    if (family == PreFamily::kDeepseekV3) {
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t e) {
        return run_of(v, i, e, [](uint32_t x) { return is_number(x); }, 3);
      });
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t e) {
        return run_of(v, i, e, cjk_v3, (size_t)-1);
      });
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t e) {
        return match_deepseek3(v, i, e);
      });
    } else {
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t) {
        return (size_t)(is_nl(v[i]) ? 1 : 0);
      });
      // \s?<cased letters>+
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t e) {
        size_t j = (is_space(v[i]) && i + 1 < e) ? i + 1 : i;
        size_t len = run_of(v, j, e, [](uint32_t x) { return is_cased(x); }, (size_t)-1);
        if (len) return j - i + len;
        return j != i ? run_of(v, i, e, [](uint32_t x) { return is_cased(x); }, (size_t)-1) : (size_t)0;
      });
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t e) {
        size_t j = (is_space(v[i]) && i + 1 < e) ? i + 1 : i;
        size_t len = run_of(v, j, e, punct_v2, (size_t)-1);
        if (len) return j - i + len;
        return j != i ? run_of(v, i, e, punct_v2, (size_t)-1) : (size_t)0;
      });
      // \s+$ : only at the very end of the whole text
      spans = split_isolated(c, spans, [n](const std::vector<uint32_t>& v, size_t i, size_t e) {
        if (e != n || !is_space(v[i])) return (size_t)0;
        size_t k = i;
        while (k < e && is_space(v[k])) ++k;
        return k == n ? k - i : (size_t)0;
      });
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t e) {
        return run_of(v, i, e, cjk_v2, (size_t)-1);
      });
      spans = split_isolated(c, spans, [](const std::vector<uint32_t>& v, size_t i, size_t) {
        return (size_t)(is_number(v[i]) ? 1 : 0);   // individual digits
      });
    }
    for (const Span& s : spans) emit(s.first, s.second);
    return out;
  }

  size_t i = 0;
  while (i < n) {
    size_t len;
    switch (family) {
      case PreFamily::kGpt2: len = match_gpt2(c, i, n); break;
      case PreFamily::kLlama3: len = match_cl100k(c, i, n, 3, false); break;
      case PreFamily::kQwen2: len = match_cl100k(c, i, n, 1, false); break;
      default: len = match_cl100k(c, i, n, 1, true); break;
    }
    if (len == 0) len = 1;
    emit(i, i + len);
    i += len;
  }
  return out;
}

PreFamily family_from_pattern(const std::string& p) {
  auto has = [&](const char* s) { return p.find(s) != std::string::npos; };
  if (has("A-Za-z\xC2\xB5")) return PreFamily::kDeepseekV2;                   // A-Za-zµ...
  if (has("\\p{N}{1,3}") && has("\xE4\xB8\x80-\xE9\xBE\xA5")) return PreFamily::kDeepseekV3;  // 一-龥
  if (has("\\p{N}{1,3}")) return PreFamily::kLlama3;
  if (has("(?i:") && has("[\\p{L}\\p{M}]+")) return PreFamily::kQwen35;
  if (has("(?i:")) return PreFamily::kQwen2;
  if (has("'s|'t|'re")) return PreFamily::kGpt2;
  return PreFamily::kGpt2;
}

PreFamily family_from_gguf_pre(const std::string& pre) {
  if (pre == "llama3" || pre == "llama-bpe" || pre == "llama-v3" || pre == "smaug-bpe") return PreFamily::kLlama3;
  if (pre == "qwen2" || pre == "deepseek-r1-qwen" || pre == "megrez") return PreFamily::kQwen2;
  if (pre == "qwen35" || pre == "qwen3.5") return PreFamily::kQwen35;
  if (pre == "deepseek-v3") return PreFamily::kDeepseekV3;
  if (pre == "deepseek-llm" || pre == "deepseek-v2") return PreFamily::kDeepseekV2;
  return PreFamily::kGpt2;   // gpt-2, olmo, dbrx, default
}

}  // namespace tok
}  // namespace b200
