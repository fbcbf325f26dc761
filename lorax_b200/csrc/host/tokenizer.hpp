// The router's own tokenizer: reads a HuggingFace `tokenizer.json` and turns request text into token ids on a pool of worker
// threads, so that validation (input length, truncation, token budget) does not cost a round trip to a shard.  The reference
// router does the same with the Rust `tokenizers` crate on `validation_workers` threads (router/src/validation.rs:44-118,
// tokenizer_worker / prepare_input); no such library exists for C++ here, so the pipeline is implemented from the file format:
//
//   added tokens -> normalizer -> pre-tokenizer -> model (BPE, WordPiece, WordLevel, Unigram) -> post-processor
//
// Only ids are produced (offsets stay with the shard's `/tokenize` helper).  A file that uses a component outside what is
// implemented (an unknown regex construct, a model type such as an n-gram language model ...) makes `load` fail with the reason,
// and the router keeps asking shard 0 for that model.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <fstream>
#include <functional>
#include <future>
#include <limits>
#include <memory>
#include <mutex>
#include <optional>
#include <queue>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "json.hpp"
#include "mini_regex.hpp"
#include "unicode.hpp"

namespace lx {
namespace tok {

using uni::Text;
using json::Value;

struct Unsupported : std::runtime_error { using std::runtime_error::runtime_error; };

inline Text text_of(const std::string& s) { return uni::from_utf8(s); }

// GPT-2's byte <-> printable code point table.
inline const uint32_t* byte_to_char() {
  static uint32_t table[256];
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
      table[b] = keep ? (uint32_t)b : (uint32_t)(256 + n++);
    }
  });
  return table;
}
// ------------------------------------------------------------------------------------------------ normalizers
struct Normalizer {
  virtual ~Normalizer() = default;
  virtual Text apply(const Text& t) const = 0;
};
using NormP = std::unique_ptr<Normalizer>;

struct SeqNorm : Normalizer {
  std::vector<NormP> parts;
  Text apply(const Text& t) const override { Text cur = t; for (auto& p : parts) cur = p->apply(cur); return cur; }
};
struct FormNorm : Normalizer {
  uni::Form form;
  explicit FormNorm(uni::Form f) : form(f) {}
  Text apply(const Text& t) const override { return uni::normalize(t, form); }
};
struct LowerNorm : Normalizer { Text apply(const Text& t) const override { return uni::lowercase(t); } };
struct PrependNorm : Normalizer {
  Text what;
  Text apply(const Text& t) const override {
    if (t.empty()) return t;
    Text out = what;
    out.insert(out.end(), t.begin(), t.end());
    return out;
  }
};
struct StripNorm : Normalizer {
  bool left = true, right = true;
  Text apply(const Text& t) const override {
    size_t b = 0, e = t.size();
    if (left) while (b < e && uni::is_space(t[b])) ++b;
    if (right) while (e > b && uni::is_space(t[e - 1])) --e;
    return Text(t.begin() + (long)b, t.begin() + (long)e);
  }
};
struct StripAccentsNorm : Normalizer {
  Text apply(const Text& t) const override { Text out; for (uint32_t c : t) if (!uni::is_mark(c)) out.push_back(c); return out; }
};
struct ReplaceNorm : Normalizer {
  Text literal;                              // String pattern
  std::unique_ptr<MiniRegex> re;             // Regex pattern
  Text content;
  Text apply(const Text& t) const override {
    Text out;
    if (!re) {
      if (literal.empty()) return t;
      for (size_t i = 0; i < t.size();) {
        if (i + literal.size() <= t.size() && std::equal(literal.begin(), literal.end(), t.begin() + (long)i)) {
          out.insert(out.end(), content.begin(), content.end());
          i += literal.size();
        } else {
          out.push_back(t[i++]);
        }
      }
      return out;
    }
    size_t at = 0;
    while (at <= t.size()) {
      size_t b, e;
      if (!re->search(t.data(), t.size(), at, &b, &e)) break;
      out.insert(out.end(), t.begin() + (long)at, t.begin() + (long)b);
      out.insert(out.end(), content.begin(), content.end());
      if (e == b) { if (b < t.size()) out.push_back(t[b]); at = b + 1; } else at = e;
    }
    if (at < t.size()) out.insert(out.end(), t.begin() + (long)at, t.end());
    return out;
  }
};
struct ByteLevelNorm : Normalizer {            // every byte of the text as its printable stand-in (the byte-level alphabet)
  Text apply(const Text& t) const override {
    const std::string bytes = uni::to_utf8(t);
    const uint32_t* map = byte_to_char();
    Text out;
    out.reserve(bytes.size());
    for (unsigned char b : bytes) out.push_back(map[b]);
    return out;
  }
};
struct NmtNorm : Normalizer {                 // the clean-up in front of NMT models: control characters out, odd spaces to ' '
  Text apply(const Text& t) const override {
    Text out;
    out.reserve(t.size());
    for (uint32_t c : t) {
      if ((c >= 1 && c <= 8) || c == 0xB || (c >= 0xE && c <= 0x1F) || c == 0x7F || c == 0x8F || c == 0x9F) continue;
      const bool space = c == 9 || c == 0xA || c == 0xC || c == 0xD || c == 0x1680 || (c >= 0x200B && c <= 0x200F) || c == 0x2028 || c == 0x2029 ||
                         c == 0x2581 || c == 0xFEFF || c == 0xFFFD;
      out.push_back(space ? ' ' : c);
    }
    return out;
  }
};
struct BertNorm : Normalizer {
  bool clean = true, chinese = true, strip_accents = true, lower = true;
  static bool cjk(uint32_t c) {
    return (c >= 0x4E00 && c <= 0x9FFF) || (c >= 0x3400 && c <= 0x4DBF) || (c >= 0x20000 && c <= 0x2A6DF) || (c >= 0x2A700 && c <= 0x2B73F) ||
           (c >= 0x2B740 && c <= 0x2B81F) || (c >= 0x2B920 && c <= 0x2CEAF) || (c >= 0xF900 && c <= 0xFAFF) || (c >= 0x2F800 && c <= 0x2FA1F);
  }
  Text apply(const Text& t) const override {
    Text cur;
    if (clean) {
      for (uint32_t c : t) {
        const bool ws = c == ' ' || c == '\t' || c == '\n' || c == '\r' || uni::is_space(c);
        const bool ctl = !(c == '\t' || c == '\n' || c == '\r') && uni::is_other(c);
        if (c == 0 || c == 0xFFFD || ctl) continue;
        cur.push_back(ws ? ' ' : c);
      }
    } else {
      cur = t;
    }
    if (chinese) {
      Text o;
      for (uint32_t c : cur) { if (cjk(c)) { o.push_back(' '); o.push_back(c); o.push_back(' '); } else o.push_back(c); }
      cur.swap(o);
    }
    if (strip_accents) {
      Text d = uni::normalize(cur, uni::Form::NFD), o;
      for (uint32_t c : d) if (!uni::is_nonspacing_mark(c)) o.push_back(c);
      cur.swap(o);
    }
    if (lower) cur = uni::lowercase(cur);
    return cur;
  }
};

// SentencePiece's compiled character map (`Precompiled`): a double-array trie from byte strings to offsets into a pool of
// replacement strings, applied grapheme cluster by grapheme cluster the way the `tokenizers` library does it (a cluster shorter than
// six bytes is looked up as a whole and replaced by what its shortest matching prefix maps to; otherwise, and when nothing
// matches, its characters are looked up one by one).
struct PrecompiledNorm : Normalizer {
  std::vector<uint32_t> trie;
  std::string pool;

  static std::string base64(const std::string& in) {
    std::string out;
    uint32_t acc = 0;
    int bits = 0;
    for (unsigned char c : in) {
      int v;
      if (c >= 'A' && c <= 'Z') v = c - 'A';
      else if (c >= 'a' && c <= 'z') v = c - 'a' + 26;
      else if (c >= '0' && c <= '9') v = c - '0' + 52;
      else if (c == '+' || c == '-') v = 62;
      else if (c == '/' || c == '_') v = 63;
      else continue;                                   // padding, line breaks
      acc = (acc << 6) | (uint32_t)v;
      bits += 6;
      if (bits >= 8) { bits -= 8; out.push_back((char)((acc >> bits) & 0xFF)); }
    }
    return out;
  }
  explicit PrecompiledNorm(const std::string& b64) {
    if (!uni::kHasGcb) throw Unsupported("Precompiled normalizer (built without the grapheme break tables)");
    const std::string blob = base64(b64);
    if (blob.size() < 4) throw Unsupported("Precompiled normalizer with an empty character map");
    uint32_t trie_bytes;
    std::memcpy(&trie_bytes, blob.data(), 4);
    if (trie_bytes % 4 != 0 || 4 + (size_t)trie_bytes > blob.size()) throw std::runtime_error("Precompiled character map: bad trie size");
    trie.resize(trie_bytes / 4);
    if (trie_bytes) std::memcpy(trie.data(), blob.data() + 4, trie_bytes);
    pool.assign(blob.data() + 4 + trie_bytes, blob.size() - 4 - trie_bytes);
  }
  static size_t offset_of(uint32_t u) { return (size_t)(u >> 10) << ((u & (1u << 9)) >> 6); }
  // What the shortest prefix of `key` that the map knows is replaced by; false when no prefix is in the map.
  bool transform(const std::string& key, std::string* out) const {
    if (trie.empty()) return false;
    size_t node = 0;
    uint32_t unit = trie[0];
    node ^= offset_of(unit);
    for (unsigned char c : key) {
      if (c == 0) break;
      node ^= c;
      if (node >= trie.size()) return false;
      unit = trie[node];
      if ((unit & ((1u << 31) | 0xFFu)) != c) return false;
      node ^= offset_of(unit);
      if (node >= trie.size()) return false;
      if ((unit >> 8) & 1) {
        const size_t at = trie[node] & ((1u << 31) - 1);
        if (at > pool.size()) return false;
        size_t end = at;
        while (end < pool.size() && pool[end] != 0) ++end;
        out->assign(pool, at, end - at);
        return true;
      }
    }
    return false;
  }
  Text apply(const Text& t) const override {
    Text out;
    out.reserve(t.size());
    std::string key, repl;
    size_t b = 0;
    for (size_t e : uni::grapheme_ends(t)) {
      key = uni::to_utf8(t.data() + b, e - b);
      bool done = false;
      if (key.size() < 6 && transform(key, &repl)) {
        const Text r = uni::from_utf8(repl);
        out.insert(out.end(), r.begin(), r.end());
        done = true;
      }
      for (size_t i = b; !done && i < e; ++i) {
        key.clear();
        uni::append_utf8(key, t[i]);
        if (transform(key, &repl)) {
          const Text r = uni::from_utf8(repl);
          out.insert(out.end(), r.begin(), r.end());
        } else {
          out.push_back(t[i]);
        }
      }
      b = e;
    }
    return out;
  }
};

inline std::unique_ptr<MiniRegex> compile_or_throw(const std::string& pattern) {
  std::string err;
  auto re = MiniRegex::compile(pattern, &err);
  if (!re) throw Unsupported("regex `" + pattern + "`: " + err);
  return re;
}

inline NormP make_normalizer(const Value& v) {
  if (v.is_null()) return nullptr;
  const std::string& type = v["type"].as_string();
  if (type == "Sequence") {
    auto s = std::make_unique<SeqNorm>();
    for (auto& p : v["normalizers"].items()) if (auto n = make_normalizer(p)) s->parts.push_back(std::move(n));
    return s;
  }
  if (type == "NFC") return std::make_unique<FormNorm>(uni::Form::NFC);
  if (type == "NFD") return std::make_unique<FormNorm>(uni::Form::NFD);
  if (type == "NFKC") return std::make_unique<FormNorm>(uni::Form::NFKC);
  if (type == "NFKD") return std::make_unique<FormNorm>(uni::Form::NFKD);
  if (type == "Lowercase") return std::make_unique<LowerNorm>();
  if (type == "StripAccents") return std::make_unique<StripAccentsNorm>();
  if (type == "Prepend") { auto p = std::make_unique<PrependNorm>(); p->what = text_of(v["prepend"].as_string()); return p; }
  if (type == "Strip") {
    auto s = std::make_unique<StripNorm>();
    s->left = v["strip_left"].as_bool(true); s->right = v["strip_right"].as_bool(true);
    return s;
  }
  if (type == "Replace") {
    auto r = std::make_unique<ReplaceNorm>();
    r->content = text_of(v["content"].as_string());
    if (v["pattern"]["String"].is_string()) r->literal = text_of(v["pattern"]["String"].as_string());
    else if (v["pattern"]["Regex"].is_string()) r->re = compile_or_throw(v["pattern"]["Regex"].as_string());
    else throw Unsupported("Replace normalizer without a pattern");
    return r;
  }
  if (type == "BertNormalizer") {
    auto b = std::make_unique<BertNorm>();
    b->clean = v["clean_text"].as_bool(true);
    b->chinese = v["handle_chinese_chars"].as_bool(true);
    b->lower = v["lowercase"].as_bool(true);
    b->strip_accents = v["strip_accents"].is_bool() ? v["strip_accents"].as_bool() : b->lower;
    return b;
  }
  if (type == "Nmt") return std::make_unique<NmtNorm>();
  if (type == "ByteLevel") return std::make_unique<ByteLevelNorm>();
  if (type == "Precompiled") return std::make_unique<PrecompiledNorm>(v["precompiled_charsmap"].as_string());
  throw Unsupported("normalizer " + type);
}

// ------------------------------------------------------------------------------------------------ pre-tokenizers
// A pre-tokenizer maps one piece of text to pieces.  `at_start` says that the piece begins the request text (Metaspace's
// "first" scheme prepends only there).
struct PreTokenizer {
  virtual ~PreTokenizer() = default;
  virtual void apply(const Text& t, bool at_start, std::vector<Text>& out) const = 0;
};
using PreP = std::unique_ptr<PreTokenizer>;

enum class Behavior { Removed, Isolated, MergedWithPrevious, MergedWithNext, Contiguous };
inline Behavior behavior_of(const std::string& s) {
  if (s == "Removed") return Behavior::Removed;
  if (s == "Isolated") return Behavior::Isolated;
  if (s == "MergedWithPrevious") return Behavior::MergedWithPrevious;
  if (s == "MergedWithNext") return Behavior::MergedWithNext;
  if (s == "Contiguous") return Behavior::Contiguous;
  throw Unsupported("split behavior " + s);
}

// Spans [b, e) with a flag "is a delimiter match", covering the text; then the behaviour decides what becomes a piece.
struct Span { size_t b, e; bool match; };
inline void split_spans(const Text& t, const std::vector<Span>& spans, Behavior how, std::vector<Text>& out) {
  std::vector<std::pair<size_t, size_t>> pieces;
  switch (how) {
    case Behavior::Removed:
      for (auto& s : spans) if (!s.match) pieces.push_back({s.b, s.e});
      break;
    case Behavior::Isolated:
      for (auto& s : spans) pieces.push_back({s.b, s.e});
      break;
    case Behavior::MergedWithPrevious: {
      bool prev_match = false;
      for (auto& s : spans) {
        if (s.match && !prev_match && !pieces.empty()) pieces.back().second = s.e;
        else pieces.push_back({s.b, s.e});
        prev_match = s.match;
      }
      break;
    }
    case Behavior::MergedWithNext: {
      bool prev_match = false;
      std::vector<std::pair<size_t, size_t>> rev;
      for (size_t i = spans.size(); i-- > 0;) {
        const Span& s = spans[i];
        if (s.match && !prev_match && !rev.empty()) rev.back().first = s.b;
        else rev.push_back({s.b, s.e});
        prev_match = s.match;
      }
      pieces.assign(rev.rbegin(), rev.rend());
      break;
    }
    case Behavior::Contiguous: {
      bool prev_match = false;
      for (auto& s : spans) {
        if (s.match == prev_match && !pieces.empty()) pieces.back().second = s.e;
        else pieces.push_back({s.b, s.e});
        prev_match = s.match;
      }
      break;
    }
  }
  for (auto& p : pieces) if (p.second > p.first) out.emplace_back(t.begin() + (long)p.first, t.begin() + (long)p.second);
}

template <class Pred>
inline std::vector<Span> spans_by_char(const Text& t, Pred is_delim) {
  std::vector<Span> spans;
  size_t last = 0;
  for (size_t i = 0; i < t.size(); ++i) {
    if (is_delim(t[i])) {
      if (i > last) spans.push_back({last, i, false});
      spans.push_back({i, i + 1, true});
      last = i + 1;
    }
  }
  if (last < t.size()) spans.push_back({last, t.size(), false});
  return spans;
}
inline std::vector<Span> spans_by_regex(const Text& t, const MiniRegex& re, bool invert) {
  std::vector<Span> spans;
  size_t last = 0, at = 0;
  while (at <= t.size()) {
    size_t b, e;
    if (!re.search(t.data(), t.size(), at, &b, &e)) break;
    if (b > last) spans.push_back({last, b, invert});
    if (e == b) {                                    // a zero-width match (look-around, \b) cuts the text where it stands
      spans.push_back({b, b, !invert});
      last = b;
      at = b + 1;
      continue;
    }
    spans.push_back({b, e, !invert});
    last = e;
    at = e;
  }
  if (last < t.size()) spans.push_back({last, t.size(), invert});
  return spans;
}
inline std::vector<Span> spans_by_literal(const Text& t, const Text& lit, bool invert) {
  std::vector<Span> spans;
  size_t last = 0;
  if (!lit.empty())
    for (size_t i = 0; i + lit.size() <= t.size();) {
      if (std::equal(lit.begin(), lit.end(), t.begin() + (long)i)) {
        if (i > last) spans.push_back({last, i, invert});
        spans.push_back({i, i + lit.size(), !invert});
        i += lit.size();
        last = i;
      } else {
        ++i;
      }
    }
  if (last < t.size()) spans.push_back({last, t.size(), invert});
  return spans;
}

struct SeqPre : PreTokenizer {
  std::vector<PreP> parts;
  void apply(const Text& t, bool at_start, std::vector<Text>& out) const override {
    std::vector<Text> cur{t};
    std::vector<bool> first{at_start};
    for (auto& p : parts) {
      std::vector<Text> next;
      std::vector<bool> next_first;
      for (size_t i = 0; i < cur.size(); ++i) {
        const size_t before = next.size();
        p->apply(cur[i], first[i], next);
        for (size_t k = before; k < next.size(); ++k) next_first.push_back(first[i] && k == before);
      }
      cur.swap(next);
      first.swap(next_first);
    }
    for (auto& c : cur) out.push_back(std::move(c));
  }
};
struct SplitPre : PreTokenizer {
  std::unique_ptr<MiniRegex> re;
  Text literal;
  Behavior how = Behavior::Isolated;
  bool invert = false;
  void apply(const Text& t, bool, std::vector<Text>& out) const override {
    split_spans(t, re ? spans_by_regex(t, *re, invert) : spans_by_literal(t, literal, invert), how, out);
  }
};
struct CharPre : PreTokenizer {              // WhitespaceSplit, Punctuation, Digits
  std::function<bool(uint32_t)> is_delim;
  Behavior how = Behavior::Removed;
  void apply(const Text& t, bool, std::vector<Text>& out) const override { split_spans(t, spans_by_char(t, is_delim), how, out); }
};
struct FixedLengthPre : PreTokenizer {         // chunks of `length` characters
  size_t length = 5;
  void apply(const Text& t, bool, std::vector<Text>& out) const override {
    for (size_t i = 0; i < t.size(); i += length) out.emplace_back(t.begin() + (long)i, t.begin() + (long)std::min(t.size(), i + length));
  }
};
struct UnicodeScriptsPre : PreTokenizer {      // a new piece wherever the script changes; spaces belong to the piece in front
  int han, hiragana, katakana;
  UnicodeScriptsPre() : han(uni::script_index("Han")), hiragana(uni::script_index("Hiragana")), katakana(uni::script_index("Katakana")) {
    if (han < 0 || hiragana < 0) throw Unsupported("UnicodeScripts pre-tokenizer (built without the script tables)");
  }
  void apply(const Text& t, bool, std::vector<Text>& out) const override {
    constexpr int kAny = -2, kNone = -3;
    int last = kNone;
    std::vector<size_t> cuts;                 // the first one sits at the first character that is not a space: spaces in front are dropped
    for (size_t i = 0; i < t.size(); ++i) {
      const uint32_t c = t[i];
      int sc = uni::script_of(c);
      if (c == 0x30FC || sc == hiragana || sc == katakana) sc = han;       // Japanese text stays together
      if (c == ' ') sc = kAny;
      if (sc != kAny && last != sc) cuts.push_back(i);
      if (sc != kAny) last = sc;
    }
    cuts.push_back(t.size());
    for (size_t k = 0; k + 1 < cuts.size(); ++k) out.emplace_back(t.begin() + (long)cuts[k], t.begin() + (long)cuts[k + 1]);
  }
};
struct BertPre : PreTokenizer {
  void apply(const Text& t, bool, std::vector<Text>& out) const override {
    std::vector<Text> words;
    split_spans(t, spans_by_char(t, [](uint32_t c) { return uni::is_space(c); }), Behavior::Removed, words);
    for (auto& w : words)
      split_spans(w, spans_by_char(w, [](uint32_t c) { return uni::is_ascii_punct(c) || uni::is_punct_category(c); }), Behavior::Isolated, out);
  }
};
struct MetaspacePre : PreTokenizer {
  uint32_t repl = 0x2581;
  enum Scheme { Always, First, Never } scheme = Always;
  bool split = true;
  void apply(const Text& t, bool at_start, std::vector<Text>& out) const override {
    Text cur;
    cur.reserve(t.size() + 1);
    for (uint32_t c : t) cur.push_back(c == ' ' ? repl : c);
    const bool prepend = scheme == Always || (scheme == First && at_start);
    if (prepend && (cur.empty() || cur[0] != repl)) cur.insert(cur.begin(), repl);
    if (!split) { if (!cur.empty()) out.push_back(std::move(cur)); return; }
    const uint32_t r = repl;
    split_spans(cur, spans_by_char(cur, [r](uint32_t c) { return c == r; }), Behavior::MergedWithNext, out);
  }
};

struct ByteLevelPre : PreTokenizer {
  bool add_prefix_space = true, use_regex = true;
  std::unique_ptr<MiniRegex> re;
  ByteLevelPre() {
    re = compile_or_throw("'s|'t|'re|'ve|'m|'ll|'d| ?\\p{L}+| ?\\p{N}+| ?[^\\s\\p{L}\\p{N}]+|\\s+(?!\\S)|\\s+");
  }
  void apply(const Text& t0, bool, std::vector<Text>& out) const override {
    Text t = t0;
    if (add_prefix_space && !t.empty() && t[0] != ' ') t.insert(t.begin(), ' ');
    std::vector<Text> pieces;
    if (use_regex) split_spans(t, spans_by_regex(t, *re, false), Behavior::Isolated, pieces);
    else if (!t.empty()) pieces.push_back(t);
    const uint32_t* map = byte_to_char();
    for (auto& p : pieces) {
      const std::string bytes = uni::to_utf8(p);
      Text mapped;
      mapped.reserve(bytes.size());
      for (unsigned char b : bytes) mapped.push_back(map[b]);
      out.push_back(std::move(mapped));
    }
  }
};

inline PreP make_pretokenizer(const Value& v) {
  if (v.is_null()) return nullptr;
  const std::string& type = v["type"].as_string();
  if (type == "Sequence") {
    auto s = std::make_unique<SeqPre>();
    for (auto& p : v["pretokenizers"].items()) if (auto q = make_pretokenizer(p)) s->parts.push_back(std::move(q));
    return s;
  }
  if (type == "ByteLevel") {
    auto b = std::make_unique<ByteLevelPre>();
    b->add_prefix_space = v["add_prefix_space"].as_bool(true);
    b->use_regex = v["use_regex"].as_bool(true);
    return b;
  }
  if (type == "Split") {
    auto s = std::make_unique<SplitPre>();
    if (v["pattern"]["Regex"].is_string()) s->re = compile_or_throw(v["pattern"]["Regex"].as_string());
    else if (v["pattern"]["String"].is_string()) s->literal = text_of(v["pattern"]["String"].as_string());
    else throw Unsupported("Split pre-tokenizer without a pattern");
    s->how = behavior_of(v["behavior"].as_string());
    s->invert = v["invert"].as_bool(false);
    return s;
  }
  if (type == "Metaspace") {
    auto m = std::make_unique<MetaspacePre>();
    const Text r = text_of(v["replacement"].is_string() ? v["replacement"].as_string() : std::string("\xE2\x96\x81"));
    if (r.size() != 1) throw Unsupported("Metaspace replacement of more than one character");
    m->repl = r[0];
    if (v["prepend_scheme"].is_string()) {
      const std::string& s = v["prepend_scheme"].as_string();
      m->scheme = s == "always" ? MetaspacePre::Always : s == "first" ? MetaspacePre::First : MetaspacePre::Never;
    } else {
      m->scheme = v["add_prefix_space"].as_bool(true) ? MetaspacePre::Always : MetaspacePre::Never;
    }
    m->split = v["split"].as_bool(true);
    return m;
  }
  if (type == "Whitespace") {
    auto s = std::make_unique<SplitPre>();
    s->re = compile_or_throw("\\w+|[^\\w\\s]+");
    s->how = Behavior::Removed;
    s->invert = true;
    return s;
  }
  if (type == "WhitespaceSplit") {
    auto c = std::make_unique<CharPre>();
    c->is_delim = [](uint32_t ch) { return uni::is_space(ch); };
    return c;
  }
  if (type == "CharDelimiterSplit") {
    const Text d = text_of(v["delimiter"].as_string());
    if (d.size() != 1) throw Unsupported("CharDelimiterSplit without a one-character delimiter");
    auto c = std::make_unique<CharPre>();
    const uint32_t delim = d[0];
    c->is_delim = [delim](uint32_t ch) { return ch == delim; };
    return c;
  }
  if (type == "FixedLength") {
    auto f = std::make_unique<FixedLengthPre>();
    f->length = (size_t)std::max<long long>(1, v["length"].as_int(5));
    return f;
  }
  if (type == "UnicodeScripts") return std::make_unique<UnicodeScriptsPre>();
  if (type == "BertPreTokenizer") return std::make_unique<BertPre>();
  if (type == "Punctuation") {
    auto c = std::make_unique<CharPre>();
    c->is_delim = [](uint32_t ch) { return uni::is_ascii_punct(ch) || uni::is_punct_category(ch); };
    c->how = behavior_of(v["behavior"].is_string() ? v["behavior"].as_string() : std::string("Isolated"));
    return c;
  }
  if (type == "Digits") {
    auto c = std::make_unique<CharPre>();
    c->is_delim = [](uint32_t ch) { return uni::is_number(ch); };
    c->how = v["individual_digits"].as_bool(false) ? Behavior::Isolated : Behavior::Contiguous;
    return c;
  }
  throw Unsupported("pre-tokenizer " + type);
}

// ------------------------------------------------------------------------------------------------ models
struct Model {
  virtual ~Model() = default;
  // Appends the ids of one pre-tokenised piece.  Throws std::runtime_error for an input the model cannot encode (a word
  // outside the vocabulary and no unknown token), as the library does.
  virtual void encode(const Text& piece, std::vector<uint32_t>& out) const = 0;
};
using Vocab = std::unordered_map<std::string, uint32_t>;

inline Vocab read_vocab(const Value& v) {
  Vocab vocab;
  vocab.reserve(v.size() * 2);
  for (auto& kv : v.members()) vocab.emplace(kv.first, (uint32_t)kv.second.as_int());
  return vocab;
}
inline std::string byte_token(unsigned char b) {
  static const char* hex = "0123456789ABCDEF";
  std::string s = "<0x";
  s.push_back(hex[b >> 4]); s.push_back(hex[b & 15]); s.push_back('>');
  return s;
}

struct WordLevel : Model {
  Vocab vocab;
  std::optional<uint32_t> unk;
  void encode(const Text& piece, std::vector<uint32_t>& out) const override {
    auto it = vocab.find(uni::to_utf8(piece));
    if (it != vocab.end()) { out.push_back(it->second); return; }
    if (!unk) throw std::runtime_error("WordLevel error: Missing [UNK] token from the vocabulary");
    out.push_back(*unk);
  }
};

struct WordPiece : Model {
  Vocab vocab;
  std::string unk_token = "[UNK]", prefix = "##";
  size_t max_chars = 100;
  void encode(const Text& piece, std::vector<uint32_t>& out) const override {
    auto unk = [&]() {
      auto it = vocab.find(unk_token);
      if (it == vocab.end()) throw std::runtime_error("WordPiece error: Missing [UNK] token from the vocabulary");
      out.push_back(it->second);
    };
    if (piece.size() > max_chars) return unk();
    std::vector<uint32_t> ids;
    size_t start = 0;
    while (start < piece.size()) {
      size_t end = piece.size();
      bool found = false;
      while (end > start) {
        std::string s = start > 0 ? prefix : std::string();
        s += uni::to_utf8(piece.data() + start, end - start);
        auto it = vocab.find(s);
        if (it != vocab.end()) { ids.push_back(it->second); found = true; break; }
        --end;
      }
      if (!found) return unk();
      start = end;
    }
    out.insert(out.end(), ids.begin(), ids.end());
  }
};

struct Bpe : Model {
  Vocab vocab;
  struct PairHash { size_t operator()(uint64_t k) const { return std::hash<uint64_t>()(k * 0x9E3779B97F4A7C15ull); } };
  std::unordered_map<uint64_t, std::pair<uint32_t, uint32_t>, PairHash> merges;     // (a, b) -> (rank, merged id)
  std::optional<uint32_t> unk;
  bool fuse_unk = false, byte_fallback = false, ignore_merges = false;
  std::string subword_prefix, word_suffix;      // continuing_subword_prefix ("##"), end_of_word_suffix ("</w>") of older BPE files
  uint32_t byte_ids[256];
  bool have_bytes = false;

  void encode(const Text& piece, std::vector<uint32_t>& out) const override {
    if (piece.empty()) return;
    if (ignore_merges) {
      auto it = vocab.find(uni::to_utf8(piece));
      if (it != vocab.end()) { out.push_back(it->second); return; }
    }
    // symbols: one per character (or byte, or unknown run)
    struct Sym { uint32_t id; int prev, next; bool alive; };
    std::vector<Sym> syms;
    syms.reserve(piece.size());
    bool pending_unk = false;
    auto push = [&](uint32_t id) { syms.push_back(Sym{id, (int)syms.size() - 1, (int)syms.size() + 1, true}); };
    std::string ch;
    for (size_t ci = 0; ci < piece.size(); ++ci) {
      const uint32_t c = piece[ci];
      ch.clear();
      if (ci > 0) ch = subword_prefix;
      uni::append_utf8(ch, c);
      if (ci + 1 == piece.size()) ch += word_suffix;
      auto it = vocab.find(ch);
      if (it != vocab.end()) { pending_unk = false; push(it->second); continue; }
      if (byte_fallback && have_bytes) {
        pending_unk = false;
        std::string raw;
        uni::append_utf8(raw, c);
        for (unsigned char b : raw) push(byte_ids[b]);
        continue;
      }
      if (unk) {
        if (fuse_unk && pending_unk) continue;           // the run of unknown characters is one symbol
        push(*unk);
        pending_unk = true;
      }
    }
    if (syms.empty()) return;
    syms.back().next = -1;
    // lowest rank first, leftmost among equals; stale queue entries are recognised by the ids they were pushed with
    struct Cand { uint32_t rank; int pos; uint32_t a, b, merged; };
    auto worse = [](const Cand& x, const Cand& y) { return x.rank != y.rank ? x.rank > y.rank : x.pos > y.pos; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(worse)> heap(worse);
    auto consider = [&](int i) {
      if (i < 0) return;
      const int j = syms[(size_t)i].next;
      if (j < 0) return;
      auto it = merges.find((uint64_t)syms[(size_t)i].id << 32 | syms[(size_t)j].id);
      if (it != merges.end()) heap.push(Cand{it->second.first, i, syms[(size_t)i].id, syms[(size_t)j].id, it->second.second});
    };
    for (int i = 0; i + 1 < (int)syms.size(); ++i) consider(i);
    while (!heap.empty()) {
      const Cand c = heap.top();
      heap.pop();
      Sym& l = syms[(size_t)c.pos];
      if (!l.alive || l.id != c.a || l.next < 0) continue;
      Sym& r = syms[(size_t)l.next];
      if (r.id != c.b) continue;
      l.id = c.merged;
      r.alive = false;
      l.next = r.next;
      if (r.next >= 0) syms[(size_t)r.next].prev = c.pos;
      consider(l.prev);
      consider(c.pos);
    }
    for (int i = 0; i >= 0; i = syms[(size_t)i].next) out.push_back(syms[(size_t)i].id);
  }
};

struct Unigram : Model {
  // byte trie over the pieces: one hash map of (node, byte) -> node for the whole vocabulary (a quarter of a million pieces in
  // multilingual models), piece id per node
  std::unordered_map<uint64_t, int> edges;
  std::vector<int> piece_of{-1};
  std::vector<double> scores;
  std::optional<uint32_t> unk;
  double min_score = 0;
  bool byte_fallback = false;
  uint32_t byte_ids[256];
  bool have_bytes = false;

  int step(int node, unsigned char b) const {
    auto it = edges.find((uint64_t)node << 8 | b);
    return it == edges.end() ? -1 : it->second;
  }
  void add(const std::string& piece, int id) {
    int node = 0;
    for (unsigned char b : piece) {
      int next = step(node, b);
      if (next < 0) {
        next = (int)piece_of.size();
        piece_of.push_back(-1);
        edges.emplace((uint64_t)node << 8 | b, next);
      }
      node = next;
    }
    piece_of[(size_t)node] = id;
  }
  // Best segmentation by total score (Viterbi over byte positions); a character no piece covers costs the lowest score minus 10
  // and becomes the unknown token; neighbouring unknowns are one token.
  void encode(const Text& piece, std::vector<uint32_t>& out) const override {
    const std::string s = uni::to_utf8(piece);
    const size_t n = s.size();
    if (n == 0) return;
    struct Best { double score; long from; long id; };
    std::vector<Best> best(n + 1, Best{0, -1, -1});
    const double unk_score = min_score - 10.0;
    for (size_t at = 0; at < n;) {
      const unsigned char lead = (unsigned char)s[at];
      const size_t clen = lead < 0x80 ? 1 : lead >= 0xF0 ? 4 : lead >= 0xE0 ? 3 : 2;
      if (at > 0 && best[at].from < 0) { at += clen; continue; }      // unreachable position (cannot happen: every char has a path)
      const double base = best[at].score;
      bool single = false;
      int node = 0;
      for (size_t k = at; k < n; ++k) {
        node = step(node, (unsigned char)s[k]);
        if (node < 0) break;
        const int id = piece_of[(size_t)node];
        if (id >= 0) {
          const size_t end = k + 1;
          const double cand = base + scores[(size_t)id];
          if (best[end].from < 0 || cand > best[end].score) best[end] = Best{cand, (long)at, id};
          if (end - at == clen) single = true;
        }
      }
      if (!single) {
        const size_t end = std::min(n, at + clen);
        const double cand = base + unk_score;
        if (best[end].from < 0 || cand > best[end].score) best[end] = Best{cand, (long)at, -1};
      }
      at += clen;
    }
    std::vector<std::pair<long, std::pair<size_t, size_t>>> rev;        // (id or -1, byte span)
    for (size_t end = n; end > 0;) {
      const Best& b = best[end];
      rev.push_back({b.id, {(size_t)b.from, end}});
      end = (size_t)b.from;
    }
    bool prev_unk = false;
    for (size_t i = rev.size(); i-- > 0;) {
      if (rev[i].first >= 0) { out.push_back((uint32_t)rev[i].first); prev_unk = false; continue; }
      if (byte_fallback && have_bytes) {
        for (size_t k = rev[i].second.first; k < rev[i].second.second; ++k) out.push_back(byte_ids[(unsigned char)s[k]]);
        prev_unk = false;
        continue;
      }
      if (!unk) throw std::runtime_error("Unigram error: Encountered an unknown token but `unk_id` is missing");
      if (!prev_unk) out.push_back(*unk);
      prev_unk = true;
    }
  }
};

template <class M>
inline void find_byte_tokens(M& m, const std::function<std::optional<uint32_t>(const std::string&)>& lookup) {
  m.have_bytes = true;
  for (int b = 0; b < 256; ++b) {
    auto id = lookup(byte_token((unsigned char)b));
    if (!id) { m.have_bytes = false; return; }
    m.byte_ids[b] = *id;
  }
}

inline std::unique_ptr<Model> make_model(const Value& v) {
  std::string type = v["type"].as_string();
  if (type.empty()) type = v["merges"].is_array() ? "BPE" : "";      // files written before the field existed
  if (type == "WordLevel") {
    auto m = std::make_unique<WordLevel>();
    m->vocab = read_vocab(v["vocab"]);
    auto it = m->vocab.find(v["unk_token"].as_string());
    if (it != m->vocab.end()) m->unk = it->second;
    return m;
  }
  if (type == "WordPiece") {
    auto m = std::make_unique<WordPiece>();
    m->vocab = read_vocab(v["vocab"]);
    if (v["unk_token"].is_string()) m->unk_token = v["unk_token"].as_string();
    if (v["continuing_subword_prefix"].is_string()) m->prefix = v["continuing_subword_prefix"].as_string();
    if (v["max_input_chars_per_word"].is_number()) m->max_chars = (size_t)v["max_input_chars_per_word"].as_int();
    return m;
  }
  if (type == "BPE") {
    auto m = std::make_unique<Bpe>();
    if (v["dropout"].is_number() && v["dropout"].as_double() > 0) throw Unsupported("BPE dropout");
    if (v["continuing_subword_prefix"].is_string()) m->subword_prefix = v["continuing_subword_prefix"].as_string();
    if (v["end_of_word_suffix"].is_string()) m->word_suffix = v["end_of_word_suffix"].as_string();
    m->vocab = read_vocab(v["vocab"]);
    m->fuse_unk = v["fuse_unk"].as_bool(false);
    m->byte_fallback = v["byte_fallback"].as_bool(false);
    m->ignore_merges = v["ignore_merges"].as_bool(false);
    if (v["unk_token"].is_string()) {
      auto it = m->vocab.find(v["unk_token"].as_string());
      if (it != m->vocab.end()) m->unk = it->second;
    }
    uint32_t rank = 0;
    for (auto& e : v["merges"].items()) {
      std::string a, b;
      if (e.is_array() && e.size() == 2) { a = e.items()[0].as_string(); b = e.items()[1].as_string(); }
      else {
        const std::string& s = e.as_string();
        const size_t sp = s.find(' ');
        if (sp == std::string::npos) throw Unsupported("malformed merge `" + s + "`");
        a = s.substr(0, sp); b = s.substr(sp + 1);
      }
      // the merged token drops the continuation prefix of its right half
      const std::string& pre = m->subword_prefix;
      const std::string ab = (!pre.empty() && b.rfind(pre, 0) == 0) ? a + b.substr(pre.size()) : a + b;
      auto ia = m->vocab.find(a), ib = m->vocab.find(b), im = m->vocab.find(ab);
      if (ia == m->vocab.end() || ib == m->vocab.end() || im == m->vocab.end()) throw Unsupported("merge `" + a + " " + b + "` names a token outside the vocabulary");
      m->merges.emplace((uint64_t)ia->second << 32 | ib->second, std::make_pair(rank, im->second));
      ++rank;
    }
    Bpe* raw = m.get();
    find_byte_tokens(*m, [raw](const std::string& s) -> std::optional<uint32_t> {
      auto it = raw->vocab.find(s);
      return it == raw->vocab.end() ? std::nullopt : std::optional<uint32_t>(it->second);
    });
    return m;
  }
  if (type == "Unigram") {
    auto m = std::make_unique<Unigram>();
    Vocab ids;
    double lo = std::numeric_limits<double>::infinity();
    int id = 0;
    for (auto& e : v["vocab"].items()) {
      const std::string& piece = e.items().at(0).as_string();
      const double score = e.items().at(1).as_double();
      m->scores.push_back(score);
      if (!piece.empty()) m->add(piece, id);
      ids.emplace(piece, (uint32_t)id);
      lo = std::min(lo, score);
      ++id;
    }
    m->min_score = lo;
    if (v["unk_id"].is_number()) m->unk = (uint32_t)v["unk_id"].as_int();
    m->byte_fallback = v["byte_fallback"].as_bool(false);
    find_byte_tokens(*m, [&ids](const std::string& s) -> std::optional<uint32_t> {
      auto it = ids.find(s);
      return it == ids.end() ? std::nullopt : std::optional<uint32_t>(it->second);
    });
    return m;
  }
  throw Unsupported("model " + (type.empty() ? std::string("(none)") : type));
}

// ------------------------------------------------------------------------------------------------ post-processing
// What a single sequence becomes when special tokens are asked for: ids in front and behind.
struct PostProcessor {
  std::vector<uint32_t> before, after;
};
inline void read_postprocessor(const Value& v, PostProcessor& pp) {
  if (v.is_null()) return;
  const std::string& type = v["type"].as_string();
  if (type == "Sequence") { for (auto& p : v["processors"].items()) read_postprocessor(p, pp); return; }
  if (type == "ByteLevel") return;                                    // only trims offsets
  if (type == "BertProcessing" || type == "RobertaProcessing") {
    pp.before.push_back((uint32_t)v["cls"].items().at(1).as_int());
    pp.after.push_back((uint32_t)v["sep"].items().at(1).as_int());
    return;
  }
  if (type == "TemplateProcessing") {
    bool seen_seq = false;
    for (auto& piece : v["single"].items()) {
      if (piece["Sequence"].is_object()) {
        if (seen_seq) throw Unsupported("template with the sequence twice");
        seen_seq = true;
      } else if (piece["SpecialToken"].is_object()) {
        const std::string& name = piece["SpecialToken"]["id"].as_string();
        const Value& ids = v["special_tokens"][name]["ids"];
        if (!ids.is_array()) throw Unsupported("template names the unknown special token " + name);
        for (auto& i : ids.items()) (seen_seq ? pp.after : pp.before).push_back((uint32_t)i.as_int());
      }
    }
    return;
  }
  throw Unsupported("post-processor " + type);
}

// ------------------------------------------------------------------------------------------------ added tokens
struct AddedToken {
  Text content;
  uint32_t id = 0;
  bool single_word = false, lstrip = false, rstrip = false, normalized = false, special = false;
};

class Tokenizer {
 public:
  // Reads `path` (a tokenizer.json, or a directory that holds one).  Throws Unsupported / std::runtime_error with the reason.
  static std::unique_ptr<Tokenizer> load(const std::string& path) {
    std::string file = path;
    {
      std::ifstream probe(file + "/tokenizer.json");
      if (probe.good()) file += "/tokenizer.json";
    }
    std::ifstream in(file, std::ios::binary);
    if (!in.good()) throw std::runtime_error("cannot read " + file);
    std::stringstream ss;
    ss << in.rdbuf();
    Value root;
    std::string err;
    if (!json::parse(ss.str(), root, &err)) throw std::runtime_error("tokenizer.json: " + err);
    return from_json(root);
  }
  static std::unique_ptr<Tokenizer> from_json(const Value& root) {
    std::unique_ptr<Tokenizer> t(new Tokenizer());
    if (!root["model"].is_object()) throw std::runtime_error("tokenizer.json has no model");
    t->norm_ = make_normalizer(root["normalizer"]);
    t->pre_ = make_pretokenizer(root["pre_tokenizer"]);
    t->model_ = make_model(root["model"]);
    read_postprocessor(root["post_processor"], t->post_);
    for (auto& a : root["added_tokens"].items()) {
      AddedToken at;
      at.content = text_of(a["content"].as_string());
      if (at.content.empty()) continue;
      at.id = (uint32_t)a["id"].as_int();
      at.single_word = a["single_word"].as_bool(false);
      at.lstrip = a["lstrip"].as_bool(false);
      at.rstrip = a["rstrip"].as_bool(false);
      at.special = a["special"].as_bool(false);
      at.normalized = a["normalized"].is_bool() ? a["normalized"].as_bool() : !at.special;
      if (at.normalized && t->norm_) {
        at.content = t->norm_->apply(at.content);
        if (at.content.empty()) continue;
      }
      (at.normalized ? t->added_norm_ : t->added_raw_).push_back(std::move(at));
    }
    index(t->added_raw_, t->first_raw_);
    index(t->added_norm_, t->first_norm_);
    return t;
  }

  std::vector<uint32_t> encode(const std::string& text, bool add_special_tokens = true) const {
    std::vector<uint32_t> ids;
    if (add_special_tokens) ids = post_.before;
    const Text raw = uni::from_utf8(text);
    std::vector<Section> sections;
    split_added(raw, added_raw_, first_raw_, 0, true, sections);
    for (auto& sec : sections) {
      if (sec.token >= 0) { ids.push_back((uint32_t)sec.token); continue; }
      const Text normal = norm_ ? norm_->apply(sec.text) : sec.text;
      std::vector<Section> inner;
      split_added(normal, added_norm_, first_norm_, 0, sec.at_start, inner);
      for (auto& part : inner) {
        if (part.token >= 0) { ids.push_back((uint32_t)part.token); continue; }
        if (part.text.empty()) continue;
        if (pre_) {
          std::vector<Text> pieces;
          pre_->apply(part.text, part.at_start, pieces);
          for (auto& p : pieces) model_->encode(p, ids);
        } else {
          model_->encode(part.text, ids);
        }
      }
    }
    if (add_special_tokens) ids.insert(ids.end(), post_.after.begin(), post_.after.end());
    return ids;
  }

 private:
  struct Section { Text text; long token; bool at_start; };
  using FirstIndex = std::unordered_map<uint32_t, std::vector<int>>;      // first code point -> tokens, longest first

  static void index(const std::vector<AddedToken>& toks, FirstIndex& idx) {
    for (size_t i = 0; i < toks.size(); ++i) idx[toks[i].content[0]].push_back((int)i);
    for (auto& kv : idx)
      std::stable_sort(kv.second.begin(), kv.second.end(), [&](int a, int b) { return toks[(size_t)a].content.size() > toks[(size_t)b].content.size(); });
  }
  // Cuts `t` at the added tokens: leftmost match, longest among those that start at one place; `single_word` matches need
  // non-word neighbours, `lstrip` / `rstrip` swallow the white space beside the match.
  static void split_added(const Text& t, const std::vector<AddedToken>& toks, const FirstIndex& idx, size_t, bool at_start,
                          std::vector<Section>& out) {
    if (toks.empty()) { out.push_back(Section{t, -1, at_start}); return; }
    size_t last = 0;
    for (size_t i = 0; i < t.size();) {
      auto it = idx.find(t[i]);
      int hit = -1;
      if (it != idx.end())
        for (int k : it->second) {
          const Text& c = toks[(size_t)k].content;
          if (i + c.size() <= t.size() && std::equal(c.begin(), c.end(), t.begin() + (long)i)) { hit = k; break; }
        }
      if (hit < 0) { ++i; continue; }
      const AddedToken& a = toks[(size_t)hit];
      size_t b = i, e = i + a.content.size();
      if (a.single_word) {
        const bool left_ok = b == 0 || !uni::is_word(t[b - 1]);
        const bool right_ok = e == t.size() || !uni::is_word(t[e]);
        if (!left_ok || !right_ok) { i = e; continue; }
      }
      if (a.lstrip) while (b > last && uni::is_space(t[b - 1])) --b;
      if (a.rstrip) while (e < t.size() && uni::is_space(t[e])) ++e;
      if (b > last) out.push_back(Section{Text(t.begin() + (long)last, t.begin() + (long)b), -1, at_start && last == 0});
      out.push_back(Section{Text(), (long)a.id, false});
      last = e;
      i = e;
    }
    if (last < t.size() || out.empty()) out.push_back(Section{Text(t.begin() + (long)last, t.end()), -1, at_start && last == 0});
  }

  NormP norm_;
  PreP pre_;
  std::unique_ptr<Model> model_;
  PostProcessor post_;
  std::vector<AddedToken> added_raw_, added_norm_;
  FirstIndex first_raw_, first_norm_;
};

// ------------------------------------------------------------------------------------------------ worker pool
// `workers` threads share one read-only tokenizer; `encode` blocks the calling request thread until a worker has its ids.
// The bound on concurrent tokenisations is the point: a burst of long prompts occupies at most `workers` cores.
class TokenizerPool {
 public:
  TokenizerPool(std::shared_ptr<const Tokenizer> tok, int workers) : tok_(std::move(tok)) {
    for (int i = 0; i < std::max(1, workers); ++i) threads_.emplace_back([this] { loop(); });
  }
  ~TokenizerPool() {
    { std::lock_guard<std::mutex> g(mu_); stop_ = true; }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  std::vector<uint32_t> encode(const std::string& text, bool add_special_tokens = true) {
    std::promise<std::vector<uint32_t>> done;
    auto fut = done.get_future();
    {
      std::lock_guard<std::mutex> g(mu_);
      jobs_.push_back(Job{&text, add_special_tokens, &done});
    }
    cv_.notify_one();
    return fut.get();
  }
  uint64_t served() const { return served_.load(); }

 private:
  struct Job { const std::string* text; bool special; std::promise<std::vector<uint32_t>>* done; };
  void loop() {
    while (true) {
      Job j;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [&] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        j = jobs_.front();
        jobs_.pop_front();
      }
      try {
        j.done->set_value(tok_->encode(*j.text, j.special));
      } catch (...) {
        j.done->set_exception(std::current_exception());
      }
      ++served_;
    }
  }
  std::shared_ptr<const Tokenizer> tok_;
  std::vector<std::thread> threads_;
  std::deque<Job> jobs_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  std::atomic<uint64_t> served_{0};
};

}  // namespace tok
}  // namespace lx
