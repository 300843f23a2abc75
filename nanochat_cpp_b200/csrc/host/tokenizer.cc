// Byte-level BPE tokenizer: the fixed nanochat split pattern (hand-written scanner), greedy lowest-rank merging,
// NCTOKEN1 artefacts, lossy UTF-8 decoding, and the BPE trainer.
#include <algorithm>
#include <cstring>
#include <fstream>
#include <unordered_map>

#include "core.h"

namespace ncb {

namespace {

struct CodeRange {
  std::uint32_t lo, hi;
};
#include "unicode_tables.inc"

template <std::size_t N>
bool InRanges(const CodeRange (&table)[N], std::uint32_t cp) {
  std::size_t lo = 0, hi = N;
  while (lo < hi) {
    const std::size_t mid = (lo + hi) / 2;
    if (cp < table[mid].lo) {
      hi = mid;
    } else if (cp > table[mid].hi) {
      lo = mid + 1;
    } else {
      return true;
    }
  }
  return false;
}

// Decodes one code point at `pos`; malformed bytes decode as themselves (one byte, value >= 0x110000 marker
// is avoided by mapping to U+FFFD semantics: neither letter, number nor whitespace).
std::uint32_t DecodeAt(std::string_view s, std::size_t pos, std::size_t* len) {
  const auto b0 = static_cast<unsigned char>(s[pos]);
  auto cont = [&](std::size_t i) {
    return pos + i < s.size() && (static_cast<unsigned char>(s[pos + i]) & 0xC0) == 0x80;
  };
  if (b0 < 0x80) {
    *len = 1;
    return b0;
  }
  if ((b0 & 0xE0) == 0xC0 && cont(1)) {
    *len = 2;
    return ((b0 & 0x1Fu) << 6) | (static_cast<unsigned char>(s[pos + 1]) & 0x3Fu);
  }
  if ((b0 & 0xF0) == 0xE0 && cont(1) && cont(2)) {
    *len = 3;
    return ((b0 & 0x0Fu) << 12) | ((static_cast<unsigned char>(s[pos + 1]) & 0x3Fu) << 6) |
           (static_cast<unsigned char>(s[pos + 2]) & 0x3Fu);
  }
  if ((b0 & 0xF8) == 0xF0 && cont(1) && cont(2) && cont(3)) {
    *len = 4;
    return ((b0 & 0x07u) << 18) | ((static_cast<unsigned char>(s[pos + 1]) & 0x3Fu) << 12) |
           ((static_cast<unsigned char>(s[pos + 2]) & 0x3Fu) << 6) | (static_cast<unsigned char>(s[pos + 3]) & 0x3Fu);
  }
  *len = 1;
  return 0xFFFD;
}

struct Cp {
  std::uint32_t value;
  std::uint32_t begin, end;  // byte span
};

inline bool IsNewline(std::uint32_t c) { return c == '\r' || c == '\n'; }

// Tries the seven alternatives of the pattern at code-point index i; returns the index one past the match.
std::size_t MatchAt(const std::vector<Cp>& cps, std::size_t i) {
  const std::size_t n = cps.size();
  auto L = [&](std::size_t k) { return k < n && IsUnicodeLetter(cps[k].value); };
  auto N = [&](std::size_t k) { return k < n && IsUnicodeNumber(cps[k].value); };
  auto S = [&](std::size_t k) { return k < n && IsUnicodeWhitespace(cps[k].value); };
  auto lower = [&](std::size_t k) -> std::uint32_t {
    if (k >= n) return 0;
    const std::uint32_t c = cps[k].value;
    return (c >= 'A' && c <= 'Z') ? c + 32 : c;
  };
  // 1. '(?i:[sdmt]|ll|ve|re)
  if (cps[i].value == '\'') {
    const std::uint32_t a = lower(i + 1), b = lower(i + 2);
    if (a == 's' || a == 'd' || a == 'm' || a == 't') return i + 2;
    if ((a == 'l' && b == 'l') || (a == 'v' && b == 'e') || (a == 'r' && b == 'e')) return i + 3;
  }
  // 2. [^\r\n\p{L}\p{N}]?+\p{L}+   (possessive optional prefix)
  {
    std::size_t k = i;
    const std::uint32_t c = cps[k].value;
    if (!IsNewline(c) && !L(k) && !N(k)) ++k;
    if (L(k)) {
      while (L(k)) ++k;
      return k;
    }
  }
  // 3. \p{N}{1,2}
  if (N(i)) return N(i + 1) ? i + 2 : i + 1;
  // 4.  ?[^\s\p{L}\p{N}]++[\r\n]*
  {
    std::size_t k = i;
    if (cps[k].value == ' ' && k + 1 < n && !S(k + 1) && !L(k + 1) && !N(k + 1)) ++k;
    if (k < n && !S(k) && !L(k) && !N(k)) {
      while (k < n && !S(k) && !L(k) && !N(k)) ++k;
      while (k < n && IsNewline(cps[k].value)) ++k;
      return k;
    }
  }
  if (S(i)) {
    std::size_t run = i;
    while (S(run)) ++run;
    // 5. \s*[\r\n] : the longest prefix of the whitespace run that ends in a newline
    for (std::size_t k = run; k > i; --k)
      if (IsNewline(cps[k - 1].value)) return k;
    // 6. \s+(?!\S) : the run minus its last character when a non-space follows, the whole run at the end
    if (run == n) return run;
    if (run - i >= 2) return run - 1;
    // 7. \s+
    return run;
  }
  return i + 1;  // defensive: every code point is matched by one of the alternatives above
}

}  // namespace

bool IsUnicodeLetter(std::uint32_t cp) { return InRanges(kLetterRanges, cp); }
bool IsUnicodeNumber(std::uint32_t cp) { return InRanges(kNumberRanges, cp); }
bool IsUnicodeWhitespace(std::uint32_t cp) {
  return (cp >= 9 && cp <= 13) || cp == 32 || cp == 0x85 || cp == 0xA0 || cp == 0x1680 ||
         (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 || cp == 0x2029 || cp == 0x202F || cp == 0x205F ||
         cp == 0x3000;
}

std::string NanochatSplitPattern() {
  return "'(?i:[sdmt]|ll|ve|re)|[^\\r\\n\\p{L}\\p{N}]?+\\p{L}+|\\p{N}{1,2}| ?[^\\s\\p{L}\\p{N}]++[\\r\\n]*|"
         "\\s*[\\r\\n]|\\s+(?!\\S)|\\s+";
}

std::vector<std::string_view> SplitPattern(std::string_view text) {
  std::vector<Cp> cps;
  cps.reserve(text.size());
  for (std::size_t pos = 0; pos < text.size();) {
    std::size_t len = 1;
    const std::uint32_t v = DecodeAt(text, pos, &len);
    cps.push_back({v, static_cast<std::uint32_t>(pos), static_cast<std::uint32_t>(pos + len)});
    pos += len;
  }
  std::vector<std::string_view> pieces;
  for (std::size_t i = 0; i < cps.size();) {
    std::size_t j = MatchAt(cps, i);
    if (j <= i) j = i + 1;
    pieces.push_back(text.substr(cps[i].begin, cps[j - 1].end - cps[i].begin));
    i = j;
  }
  return pieces;
}

std::string SanitizeUtf8(std::string_view bytes) {
  // "replace" decoding with the maximal-subpart rule: a truncated but so-far-valid sequence becomes ONE U+FFFD,
  // any other offending byte becomes one U+FFFD of its own.
  std::string out;
  out.reserve(bytes.size());
  const std::size_t n = bytes.size();
  for (std::size_t pos = 0; pos < n;) {
    const auto b0 = static_cast<unsigned char>(bytes[pos]);
    if (b0 < 0x80) {
      out.push_back(static_cast<char>(b0));
      ++pos;
      continue;
    }
    int need = 0;
    unsigned char lo = 0x80, hi = 0xBF;  // allowed range of the first continuation byte
    if (b0 >= 0xC2 && b0 <= 0xDF) need = 1;
    else if (b0 == 0xE0) need = 2, lo = 0xA0;
    else if ((b0 >= 0xE1 && b0 <= 0xEC) || b0 == 0xEE || b0 == 0xEF) need = 2;
    else if (b0 == 0xED) need = 2, hi = 0x9F;
    else if (b0 == 0xF0) need = 3, lo = 0x90;
    else if (b0 >= 0xF1 && b0 <= 0xF3) need = 3;
    else if (b0 == 0xF4) need = 3, hi = 0x8F;
    if (need == 0) {
      out.append("\xEF\xBF\xBD");
      ++pos;
      continue;
    }
    std::size_t got = 0;
    while (got < static_cast<std::size_t>(need) && pos + 1 + got < n) {
      const auto c = static_cast<unsigned char>(bytes[pos + 1 + got]);
      const unsigned char l = got == 0 ? lo : 0x80, h = got == 0 ? hi : 0xBF;
      if (c < l || c > h) break;
      ++got;
    }
    if (got == static_cast<std::size_t>(need)) {
      out.append(bytes.substr(pos, 1 + got));
    } else {
      out.append("\xEF\xBF\xBD");
    }
    pos += 1 + got;
  }
  return out;
}

const std::vector<std::string>& DefaultSpecialTokens() {
  static const std::vector<std::string> k = {"<|bos|>",          "<|user_start|>",  "<|user_end|>",
                                             "<|assistant_start|>", "<|assistant_end|>", "<|python_start|>",
                                             "<|python_end|>",   "<|output_start|>", "<|output_end|>"};
  return k;
}

// ------------------------------------------------------------------ Tokenizer
Tokenizer::Tokenizer(std::vector<std::pair<std::uint32_t, std::uint32_t>> merges,
                     std::vector<std::pair<std::string, std::uint32_t>> specials)
    : merges_(std::move(merges)), specials_(std::move(specials)) {
  const std::size_t base = 256 + merges_.size();
  bytes_of_.resize(base);
  for (int b = 0; b < 256; ++b) bytes_of_[b] = std::string(1, static_cast<char>(b));
  for (std::size_t i = 0; i < merges_.size(); ++i) {
    const auto [l, r] = merges_[i];
    if (l < 256 + i && r < 256 + i) bytes_of_[256 + i] = bytes_of_[l] + bytes_of_[r];
    rank_[(static_cast<std::uint64_t>(l) << 32) | r] = static_cast<std::uint32_t>(i);
  }
  for (std::size_t i = 0; i < base; ++i) by_bytes_.emplace(bytes_of_[i], static_cast<std::uint32_t>(i));
  std::size_t vocab = base;
  for (const auto& sp : specials_) vocab = std::max<std::size_t>(vocab, sp.second + 1);
  vocab_size_ = static_cast<int>(vocab);
  token_bytes_.assign(vocab, 0);
  for (std::size_t i = 0; i < base; ++i) token_bytes_[i] = static_cast<std::uint8_t>(std::min<std::size_t>(bytes_of_[i].size(), 255));
}

int Tokenizer::SpecialId(std::string_view name) const {
  for (const auto& sp : specials_)
    if (sp.first == name) return static_cast<int>(sp.second);
  return -1;
}
bool Tokenizer::IsSpecial(int id) const {
  for (const auto& sp : specials_)
    if (static_cast<int>(sp.second) == id) return true;
  return false;
}

void Tokenizer::EncodePiece(std::string_view piece, std::vector<int>* out) const {
  // tiktoken's rule: adjacent parts merge when their concatenated BYTES are a vocabulary entry, lowest id first
  // (not only when that exact pair was merged during training).
  std::vector<std::uint32_t> bounds(piece.size() + 1);
  for (std::size_t i = 0; i <= piece.size(); ++i) bounds[i] = static_cast<std::uint32_t>(i);
  auto rank_of = [&](std::size_t i) -> std::uint32_t {  // rank of parts i and i+1 joined
    const auto it = by_bytes_.find(std::string(piece.substr(bounds[i], bounds[i + 2] - bounds[i])));
    return it == by_bytes_.end() ? UINT32_MAX : it->second;
  };
  while (bounds.size() > 2) {
    std::uint32_t best = UINT32_MAX;
    std::size_t at = 0;
    for (std::size_t i = 0; i + 2 < bounds.size(); ++i) {
      const std::uint32_t r = rank_of(i);
      if (r < best) {
        best = r;
        at = i;
      }
    }
    if (best == UINT32_MAX) break;
    bounds.erase(bounds.begin() + static_cast<std::ptrdiff_t>(at) + 1);
  }
  for (std::size_t i = 0; i + 1 < bounds.size(); ++i) {
    const auto it = by_bytes_.find(std::string(piece.substr(bounds[i], bounds[i + 1] - bounds[i])));
    out->push_back(it != by_bytes_.end() ? static_cast<int>(it->second) : static_cast<unsigned char>(piece[bounds[i]]));
  }
}

std::vector<int> Tokenizer::Encode(std::string_view text, int prepend, int append) const {
  std::vector<int> out;
  if (prepend >= 0) out.push_back(prepend);
  for (std::string_view piece : SplitPattern(text)) EncodePiece(piece, &out);
  if (append >= 0) out.push_back(append);
  return out;
}

bool Tokenizer::AppendTokenBytes(int id, std::string* out) const {
  if (id >= 0 && static_cast<std::size_t>(id) < bytes_of_.size()) {
    out->append(bytes_of_[id]);
    return true;
  }
  for (const auto& sp : specials_) {
    if (static_cast<int>(sp.second) == id) {
      out->append(sp.first);
      return true;
    }
  }
  return false;
}

std::string Tokenizer::Decode(const int* ids, int count) const {
  std::string raw;
  for (int i = 0; i < count; ++i) AppendTokenBytes(ids[i], &raw);
  return SanitizeUtf8(raw);
}

std::unique_ptr<Tokenizer> Tokenizer::Load(const std::string& path, std::string* error) {
  auto fail = [&](const char* m) -> std::unique_ptr<Tokenizer> {
    if (error != nullptr) *error = std::string(m) + ": " + path;
    return nullptr;
  };
  std::ifstream f(path, std::ios::binary);
  if (!f) return fail("cannot open tokenizer");
  std::string data((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  std::size_t off = 0;
  auto u32 = [&](std::uint32_t* v) {
    if (off + 4 > data.size()) return false;
    std::memcpy(v, data.data() + off, 4);
    off += 4;
    return true;
  };
  if (data.size() < 8 || data.compare(0, 8, "NCTOKEN1") != 0) return fail("not an NCTOKEN1 artefact");
  off = 8;
  std::uint32_t version = 0, plen = 0, nmerge = 0, nspecial = 0;
  if (!u32(&version) || version != 1) return fail("unsupported tokenizer version");
  if (!u32(&plen) || off + plen > data.size()) return fail("truncated tokenizer pattern");
  if (data.substr(off, plen) != NanochatSplitPattern()) return fail("tokenizer split pattern differs from the built-in one");
  off += plen;
  if (!u32(&nmerge) || nmerge > (1u << 24)) return fail("truncated tokenizer merges");
  std::vector<std::pair<std::uint32_t, std::uint32_t>> merges(nmerge);
  for (auto& m : merges)
    if (!u32(&m.first) || !u32(&m.second)) return fail("truncated tokenizer merges");
  if (!u32(&nspecial) || nspecial > 4096) return fail("truncated tokenizer specials");
  std::vector<std::pair<std::string, std::uint32_t>> specials(nspecial);
  for (auto& sp : specials) {
    std::uint32_t n = 0;
    if (!u32(&n) || off + n > data.size()) return fail("truncated tokenizer specials");
    sp.first = data.substr(off, n);
    off += n;
    if (!u32(&sp.second)) return fail("truncated tokenizer specials");
  }
  return std::make_unique<Tokenizer>(std::move(merges), std::move(specials));
}

bool Tokenizer::Save(const std::string& path) const {
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  if (!out) return false;
  auto u32 = [&](std::uint32_t v) { out.write(reinterpret_cast<const char*>(&v), 4); };
  out.write("NCTOKEN1", 8);
  u32(1);
  const std::string pattern = NanochatSplitPattern();
  u32(static_cast<std::uint32_t>(pattern.size()));
  out.write(pattern.data(), static_cast<std::streamsize>(pattern.size()));
  u32(static_cast<std::uint32_t>(merges_.size()));
  for (const auto& m : merges_) {
    u32(m.first);
    u32(m.second);
  }
  u32(static_cast<std::uint32_t>(specials_.size()));
  for (const auto& sp : specials_) {
    u32(static_cast<std::uint32_t>(sp.first.size()));
    out.write(sp.first.data(), static_cast<std::streamsize>(sp.first.size()));
    u32(sp.second);
  }
  return static_cast<bool>(out);
}

// ------------------------------------------------------------------ BPE trainer
// Classic incremental BPE over unique pre-tokenised words: counts of adjacent pairs are kept up to date as merges
// are applied, and the next merge is the most frequent pair (ties: the numerically smaller pair).
std::unique_ptr<Tokenizer> TrainBpe(const std::function<bool(std::string*)>& next_document,
                                    const BpeTrainerConfig& config) {
  std::unordered_map<std::string, std::int64_t> word_counts;
  std::string doc;
  std::int64_t total = 0;
  while (next_document(&doc)) {
    std::string_view view(doc);
    if (config.doc_cap > 0 && static_cast<std::int64_t>(view.size()) > config.doc_cap) view = view.substr(0, config.doc_cap);
    if (config.max_chars > 0 && total + static_cast<std::int64_t>(view.size()) > config.max_chars) {
      view = view.substr(0, static_cast<std::size_t>(std::max<std::int64_t>(0, config.max_chars - total)));
    }
    total += static_cast<std::int64_t>(view.size());
    for (std::string_view piece : SplitPattern(view)) ++word_counts[std::string(piece)];
    if (config.max_chars > 0 && total >= config.max_chars) break;
  }
  struct Word {
    std::vector<std::uint32_t> ids;
    std::int64_t count;
  };
  std::vector<Word> words;
  words.reserve(word_counts.size());
  for (auto& kv : word_counts) {
    Word w;
    w.count = kv.second;
    for (unsigned char c : kv.first) w.ids.push_back(c);
    words.push_back(std::move(w));
  }
  std::sort(words.begin(), words.end(), [](const Word& a, const Word& b) { return a.ids < b.ids; });  // deterministic
  const int num_specials = static_cast<int>(DefaultSpecialTokens().size());
  const int num_merges = std::max(0, config.vocab_size - 256 - num_specials);
  auto key = [](std::uint32_t a, std::uint32_t b) { return (static_cast<std::uint64_t>(a) << 32) | b; };
  std::unordered_map<std::uint64_t, std::int64_t> pair_count;
  std::unordered_map<std::uint64_t, std::vector<std::uint32_t>> where;  // pair -> word indices (may hold stale entries)
  for (std::uint32_t wi = 0; wi < words.size(); ++wi) {
    const Word& w = words[wi];
    for (std::size_t i = 0; i + 1 < w.ids.size(); ++i) {
      const std::uint64_t k = key(w.ids[i], w.ids[i + 1]);
      pair_count[k] += w.count;
      where[k].push_back(wi);
    }
  }
  std::vector<std::pair<std::uint32_t, std::uint32_t>> merges;
  for (int m = 0; m < num_merges; ++m) {
    std::uint64_t best_key = 0;
    std::int64_t best = 0;
    for (const auto& kv : pair_count) {
      if (kv.second > best || (kv.second == best && best > 0 && kv.first < best_key)) {
        best = kv.second;
        best_key = kv.first;
      }
    }
    if (best <= 0) break;
    const std::uint32_t a = static_cast<std::uint32_t>(best_key >> 32), b = static_cast<std::uint32_t>(best_key);
    const std::uint32_t new_id = 256 + static_cast<std::uint32_t>(merges.size());
    merges.emplace_back(a, b);
    std::vector<std::uint32_t> touched = std::move(where[best_key]);
    where.erase(best_key);
    std::sort(touched.begin(), touched.end());
    touched.erase(std::unique(touched.begin(), touched.end()), touched.end());
    for (std::uint32_t wi : touched) {
      Word& w = words[wi];
      std::vector<std::uint32_t> out;
      out.reserve(w.ids.size());
      bool changed = false;
      for (std::size_t i = 0; i < w.ids.size();) {
        if (i + 1 < w.ids.size() && w.ids[i] == a && w.ids[i + 1] == b) {
          out.push_back(new_id);
          i += 2;
          changed = true;
        } else {
          out.push_back(w.ids[i]);
          ++i;
        }
      }
      if (!changed) continue;
      for (std::size_t i = 0; i + 1 < w.ids.size(); ++i) pair_count[key(w.ids[i], w.ids[i + 1])] -= w.count;
      w.ids = std::move(out);
      for (std::size_t i = 0; i + 1 < w.ids.size(); ++i) {
        const std::uint64_t k = key(w.ids[i], w.ids[i + 1]);
        pair_count[k] += w.count;
        where[k].push_back(wi);
      }
    }
    pair_count.erase(best_key);
  }
  std::vector<std::pair<std::string, std::uint32_t>> specials;
  std::uint32_t id = 256 + static_cast<std::uint32_t>(merges.size());
  for (const std::string& name : DefaultSpecialTokens()) specials.emplace_back(name, id++);
  return std::make_unique<Tokenizer>(std::move(merges), std::move(specials));
}

}  // namespace ncb
