// Byte-level BPE tokenizer for the Qwen family (GPT-2 byte alphabet, ranked merges, special-token
// matching, Qwen2 / Qwen3.5 pre-tokenisation rules), built from the arrays a GGUF file carries:
// tokenizer.ggml.tokens / merges / token_type / pre.
//
// Behaviour to match (reference: common/bpe_tokenizer.h:28-50 API, :642-775 pre-tokeniser, :868-989 merge
// loop, :1027-1078 encode): text is first cut at special tokens (longest match, token types 3 and 4), the
// pieces are split by the pre-tokeniser pattern
//   (?i:'s|'t|'re|'ve|'m|'ll|'d) | [^\r\n\p{L}\p{N}]?\p{L}+ | \p{N} | ?[^\s\p{L}\p{N}]+[\r\n]* | \s*[\r\n]+ | \s+(?!\S) | \s+
// ("qwen35" lets combining marks \p{M} join letters), every word is mapped byte -> printable code point and
// merged greedily by ascending merge rank.  Decoding maps the code points back to bytes.
#include "common.h"
#include "unicode_ranges.inc"
#include <string.h>
#include <algorithm>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

namespace gbh {

// ------------------------------------------------------------------------------------------ unicode helpers
enum : uint8_t { F_LETTER = 1, F_NUMBER = 2, F_MARK = 4, F_SPACE = 8, F_OTHER = 16 };

template <size_t N>
static bool in_ranges(const uint32_t (&r)[N][2], uint32_t cp) {
  size_t lo = 0, hi = N;
  while (lo < hi) {
    const size_t mid = (lo + hi) / 2;
    if (cp < r[mid][0]) hi = mid; else if (cp > r[mid][1]) lo = mid + 1; else return true;
  }
  return false;
}
static bool is_space(uint32_t c) {
  return (c >= 0x09 && c <= 0x0D) || c == 0x20 || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 ||
         c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
static uint8_t cp_flags(uint32_t c) {
  if (c == 0xFFFFFFFFu) return 0;
  if (is_space(c)) return F_SPACE;
  if (in_ranges(k_letter_ranges, c)) return F_LETTER;
  if (in_ranges(k_number_ranges, c)) return F_NUMBER;
  if (in_ranges(k_mark_ranges, c)) return F_MARK;
  return F_OTHER;
}
static uint32_t cp_lower(uint32_t c) {
  if (c < 128) return (c >= 'A' && c <= 'Z') ? c + 32 : c;
  const size_t n = sizeof(k_lower_pairs) / sizeof(k_lower_pairs[0]);
  size_t lo = 0, hi = n;
  while (lo < hi) { const size_t mid = (lo + hi) / 2; if (k_lower_pairs[mid][0] < c) lo = mid + 1; else hi = mid; }
  return (lo < n && k_lower_pairs[lo][0] == c) ? k_lower_pairs[lo][1] : c;
}
// Decodes one UTF-8 sequence (invalid bytes decode as themselves, one at a time).
static uint32_t utf8_next(const uint8_t* s, size_t n, size_t* adv) {
  const uint8_t c = s[0];
  if (c < 0x80) { *adv = 1; return c; }
  int len = (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 0;
  if (len == 0 || (size_t)len > n) { *adv = 1; return c; }
  uint32_t cp = c & (0xFF >> (len + 1));
  for (int i = 1; i < len; ++i) { if ((s[i] & 0xC0) != 0x80) { *adv = 1; return c; } cp = (cp << 6) | (s[i] & 0x3F); }
  *adv = (size_t)len;
  return cp;
}
static void utf8_put(std::string& out, uint32_t cp) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
}

// ------------------------------------------------------------------------------------------ tokenizer
struct Tokenizer {
  std::vector<std::string> tokens;
  std::vector<int> types;
  std::unordered_map<std::string, int> vocab;
  std::unordered_map<std::string, int> merge_rank;     // "left right" -> rank
  std::vector<std::pair<std::string, int>> specials;   // sorted by descending length
  uint32_t byte_to_cp[256];
  std::unordered_map<uint32_t, uint8_t> cp_to_byte;
  bool marks_with_letters = false;
  bool spm_style = false;                              // "gemma4": spaces become U+2581, split at newlines

  void init_byte_map() {
    // GPT-2 alphabet: printable Latin-1 bytes map to themselves, the others to U+0100 upwards in byte order.
    int n = 0;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      byte_to_cp[b] = keep ? (uint32_t)b : (uint32_t)(256 + n++);
    }
    for (int b = 0; b < 256; ++b) cp_to_byte[byte_to_cp[b]] = (uint8_t)b;
  }

  // pre-tokeniser: byte ranges of the words of text[0, n)
  void split_words(const uint8_t* text, size_t n, std::vector<std::pair<size_t, size_t>>& words) const {
    std::vector<uint32_t> cps; std::vector<size_t> off;
    for (size_t i = 0; i < n;) { size_t adv; cps.push_back(utf8_next(text + i, n - i, &adv)); off.push_back(i); i += adv; }
    off.push_back(n);
    const int m = (int)cps.size();
    auto CP = [&](int p) -> uint32_t { return (p >= 0 && p < m) ? cps[p] : 0xFFFFFFFFu; };
    auto FL = [&](int p) -> uint8_t { return (p >= 0 && p < m) ? cp_flags(cps[p]) : 0; };
    const uint8_t lm_mask = (uint8_t)(F_LETTER | (marks_with_letters ? F_MARK : 0));
    int prev = 0;
    auto emit = [&](int end) { if (end > prev) words.emplace_back(off[prev], off[end] - off[prev]); prev = end; };
    for (int pos = 0; pos < m;) {
      const uint32_t c = CP(pos);
      const uint8_t f = FL(pos);
      if (c == '\'' && pos + 1 < m) {                      // English contractions, case-insensitive
        const uint32_t c1 = cp_lower(CP(pos + 1));
        if (c1 == 's' || c1 == 't' || c1 == 'm' || c1 == 'd') { emit(pos + 2); pos += 2; continue; }
        if (pos + 2 < m) {
          const uint32_t c2 = cp_lower(CP(pos + 2));
          if ((c1 == 'r' && c2 == 'e') || (c1 == 'v' && c2 == 'e') || (c1 == 'l' && c2 == 'l')) { emit(pos + 3); pos += 3; continue; }
        }
      }
      if (!(c == '\r' || c == '\n' || (f & F_NUMBER))) {    // optional lead character + run of letters
        if ((f & lm_mask) || (FL(pos + 1) & lm_mask)) {
          int p = pos + 1;
          while (FL(p) & lm_mask) ++p;
          emit(p); pos = p; continue;
        }
      }
      if (f & F_NUMBER) { emit(pos + 1); ++pos; continue; }  // one digit at a time
      {                                                     // optional space + run of punctuation/symbols + newlines
        const uint8_t f2 = (c == ' ') ? FL(pos + 1) : f;
        if (f2 && !(f2 & (F_SPACE | lm_mask | F_NUMBER))) {
          int p = pos + (c == ' ' ? 1 : 0);
          while (p < m) { const uint8_t ff = FL(p); if (!ff || (ff & (F_SPACE | lm_mask | F_NUMBER))) break; ++p; }
          while (p < m && (CP(p) == '\r' || CP(p) == '\n')) ++p;
          emit(p); pos = p; continue;
        }
      }
      {                                                     // whitespace rules
        int ws = 0, last_nl = 0;
        while (FL(pos + ws) & F_SPACE) { const uint32_t c2 = CP(pos + ws); if (c2 == '\r' || c2 == '\n') last_nl = pos + ws + 1; ++ws; }
        if (last_nl > 0) { emit(last_nl); pos = last_nl; continue; }
        if (ws > 1 && CP(pos + ws) != 0xFFFFFFFFu) { emit(pos + ws - 1); pos += ws - 1; continue; }
        if (ws > 0) { emit(pos + ws); pos += ws; continue; }
      }
      emit(pos + 1); ++pos;
    }
  }

  // BPE of one word (already in the byte-level alphabet, UTF-8): merges by ascending rank.
  void bpe_word(const std::string& w, std::vector<int>& out) const {
    struct Sym { int prev, next; size_t start, len; };
    std::vector<Sym> syms;
    for (size_t i = 0; i < w.size();) {
      size_t adv; utf8_next((const uint8_t*)w.data() + i, w.size() - i, &adv);
      syms.push_back({(int)syms.size() - 1, (int)syms.size() + 1, i, adv});
      i += adv;
    }
    if (syms.empty()) return;
    syms.back().next = -1;
    struct Cand { int rank, left, right; size_t len; };
    auto cmp = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.left > b.left; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> pq(cmp);
    std::string key;
    auto try_add = [&](int l, int r) {
      if (l < 0 || r < 0) return;
      key.assign(w, syms[l].start, syms[l].len); key.push_back(' '); key.append(w, syms[r].start, syms[r].len);
      auto it = merge_rank.find(key);
      if (it != merge_rank.end()) pq.push({it->second, l, r, syms[l].len + syms[r].len});
    };
    for (int i = 0; i + 1 < (int)syms.size(); ++i) try_add(i, i + 1);
    while (!pq.empty()) {
      const Cand c = pq.top(); pq.pop();
      Sym& l = syms[c.left]; Sym& r = syms[c.right];
      if (l.len == 0 || r.len == 0 || l.next != c.right || l.len + r.len != c.len) continue;   // stale candidate
      l.len += r.len; r.len = 0;
      l.next = r.next;
      if (r.next >= 0) syms[r.next].prev = c.left;
      try_add(l.prev, c.left);
      try_add(c.left, l.next);
    }
    for (int i = 0; i >= 0; i = syms[i].next) {
      key.assign(w, syms[i].start, syms[i].len);
      auto it = vocab.find(key);
      if (it != vocab.end()) { out.push_back(it->second); continue; }
      // unknown piece: fall back to its single characters, then to <0xXX> byte tokens
      for (size_t p = 0; p < key.size();) {
        size_t adv; const uint32_t cp = utf8_next((const uint8_t*)key.data() + p, key.size() - p, &adv);
        auto it2 = vocab.find(key.substr(p, adv));
        if (it2 != vocab.end()) out.push_back(it2->second);
        else {
          auto bt = cp_to_byte.find(cp);
          char buf[8]; snprintf(buf, sizeof(buf), "<0x%02X>", bt != cp_to_byte.end() ? bt->second : (unsigned)(cp & 0xFF));
          auto it3 = vocab.find(buf);
          if (it3 != vocab.end()) out.push_back(it3->second);
        }
        p += adv;
      }
    }
  }

  void encode_plain(const uint8_t* text, size_t n, std::vector<int>& out) const {
    std::vector<std::pair<size_t, size_t>> words;
    std::string norm;
    if (spm_style) {
      for (size_t i = 0; i < n; ++i) { if (text[i] == ' ') norm += "\xE2\x96\x81"; else norm.push_back((char)text[i]); }
      size_t start = 0;
      for (size_t i = 0; i < norm.size(); ++i)
        if (norm[i] == '\n') { if (i > start) words.emplace_back(start, i - start); words.emplace_back(i, 1); start = i + 1; }
      if (start < norm.size()) words.emplace_back(start, norm.size() - start);
      for (auto& w : words) bpe_word(norm.substr(w.first, w.second), out);
      return;
    }
    split_words(text, n, words);
    std::string mapped;
    for (auto& w : words) {
      mapped.clear();
      for (size_t i = 0; i < w.second; ++i) utf8_put(mapped, byte_to_cp[text[w.first + i]]);
      bpe_word(mapped, out);
    }
  }

  void encode(const uint8_t* text, size_t n, bool parse_special, std::vector<int>& out) const {
    if (!parse_special || specials.empty()) { encode_plain(text, n, out); return; }
    size_t start = 0, i = 0;
    while (i < n) {
      int hit = -1; size_t hit_len = 0;
      for (auto& sp : specials) {
        const std::string& s = sp.first;
        if (s.size() <= n - i && memcmp(text + i, s.data(), s.size()) == 0) { hit = sp.second; hit_len = s.size(); break; }   // longest first
      }
      if (hit >= 0) {
        if (i > start) encode_plain(text + start, i - start, out);
        out.push_back(hit);
        i += hit_len; start = i;
      } else ++i;
    }
    if (n > start) encode_plain(text + start, n - start, out);
  }

  void piece_bytes(int id, std::string& out) const {
    if (id < 0 || id >= (int)tokens.size()) return;
    const std::string& t = tokens[id];
    if (types.size() == tokens.size() && (types[id] == 3 || types[id] == 4)) { out += t; return; }     // specials are literal text
    if (t.size() == 6 && t[0] == '<' && t[1] == '0' && t[2] == 'x' && t[5] == '>') {                    // <0xXX> byte token
      unsigned v = 0;
      if (sscanf(t.c_str(), "<0x%02X>", &v) == 1) { out.push_back((char)v); return; }
    }
    if (spm_style) {
      for (size_t i = 0; i < t.size();) {
        if (i + 2 < t.size() && (uint8_t)t[i] == 0xE2 && (uint8_t)t[i + 1] == 0x96 && (uint8_t)t[i + 2] == 0x81) { out.push_back(' '); i += 3; }
        else out.push_back(t[i++]);
      }
      return;
    }
    for (size_t i = 0; i < t.size();) {
      size_t adv; const uint32_t cp = utf8_next((const uint8_t*)t.data() + i, t.size() - i, &adv);
      auto it = cp_to_byte.find(cp);
      if (it != cp_to_byte.end()) out.push_back((char)it->second); else out.append(t, i, adv);
      i += adv;
    }
  }
};

}  // namespace gbh

using namespace gbh;

// tokens / merges: concatenated bytes with per-item lengths.  types may be null.  pre: "qwen2" (default), "qwen35", "gemma4".
GBH_API void* gbh_tok_create(const char* token_bytes, const uint64_t* token_lens, long n_tokens, const char* merge_bytes,
                             const uint64_t* merge_lens, long n_merges, const int* types, const char* pre) {
  auto* t = new Tokenizer();
  t->init_byte_map();
  t->tokens.reserve(n_tokens);
  const char* p = token_bytes;
  for (long i = 0; i < n_tokens; ++i) { t->tokens.emplace_back(p, token_lens[i]); p += token_lens[i]; t->vocab.emplace(t->tokens.back(), (int)i); }
  p = merge_bytes;
  for (long i = 0; i < n_merges; ++i) { t->merge_rank.emplace(std::string(p, merge_lens[i]), (int)i); p += merge_lens[i]; }
  if (types) {
    t->types.assign(types, types + n_tokens);
    for (long i = 0; i < n_tokens; ++i) if ((types[i] == 3 || types[i] == 4) && !t->tokens[i].empty()) t->specials.emplace_back(t->tokens[i], (int)i);
    std::stable_sort(t->specials.begin(), t->specials.end(), [](const std::pair<std::string, int>& a, const std::pair<std::string, int>& b) { return a.first.size() > b.first.size(); });
  }
  if (pre && strcmp(pre, "qwen35") == 0) t->marks_with_letters = true;
  if (pre && strcmp(pre, "gemma4") == 0) t->spm_style = true;
  return t;
}
GBH_API void gbh_tok_free(void* h) { delete (Tokenizer*)h; }
GBH_API long gbh_tok_vocab_size(void* h) { return (long)((Tokenizer*)h)->tokens.size(); }
// Returns the number of ids (may exceed cap: call again with a larger buffer).
GBH_API long gbh_tok_encode(void* h, const char* text, long len, int parse_special, int* out, long cap) {
  std::vector<int> ids;
  ((Tokenizer*)h)->encode((const uint8_t*)text, (size_t)len, parse_special != 0, ids);
  for (long i = 0; i < (long)ids.size() && i < cap; ++i) out[i] = ids[i];
  return (long)ids.size();
}
// Bytes of the decoded text (may exceed cap).
GBH_API long gbh_tok_decode(void* h, const int* ids, long n, char* out, long cap) {
  std::string s;
  for (long i = 0; i < n; ++i) ((Tokenizer*)h)->piece_bytes(ids[i], s);
  const long m = std::min<long>((long)s.size(), cap);
  if (m > 0) memcpy(out, s.data(), (size_t)m);
  return (long)s.size();
}
GBH_API int gbh_tok_find(void* h, const char* token, long len) {
  auto* t = (Tokenizer*)h; auto it = t->vocab.find(std::string(token, (size_t)len));
  return it == t->vocab.end() ? -1 : it->second;
}
