// Unicode helpers for the router's tokenizer: UTF-8 <-> code points, character classes by binary search over the generated
// range tables, lower-casing and the four normalisation forms.  No Unicode library is linked; `unicode_tables.hpp` is written
// by gen_unicode_tables.py.
#pragma once
#include <algorithm>
#include <cstdint>
#include <string>
#include <vector>

#include "unicode_tables.hpp"

namespace lx {
namespace uni {

using Text = std::vector<uint32_t>;        // code points

inline void append_utf8(std::string& out, uint32_t cp) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) {
    out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
  } else {
    out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
  }
}
inline std::string to_utf8(const uint32_t* p, size_t n) {
  std::string s;
  s.reserve(n);
  for (size_t i = 0; i < n; ++i) append_utf8(s, p[i]);
  return s;
}
inline std::string to_utf8(const Text& t) { return to_utf8(t.data(), t.size()); }

// Ill-formed sequences decode to U+FFFD, one per offending byte (the text of a request reaches the router as JSON, whose
// strings a Rust server would have rejected or replaced the same way).
inline Text from_utf8(const std::string& s) {
  Text out;
  out.reserve(s.size());
  const unsigned char* p = (const unsigned char*)s.data();
  const size_t n = s.size();
  for (size_t i = 0; i < n;) {
    const unsigned char c = p[i];
    if (c < 0x80) { out.push_back(c); ++i; continue; }
    int len = c >= 0xF0 && c < 0xF8 ? 4 : c >= 0xE0 ? 3 : c >= 0xC2 && c < 0xE0 ? 2 : 0;
    if (len == 0 || i + (size_t)len > n) { out.push_back(0xFFFD); ++i; continue; }
    uint32_t cp = len == 4 ? (c & 0x07) : len == 3 ? (c & 0x0F) : (c & 0x1F);
    bool ok = true;
    for (int k = 1; k < len; ++k) {
      if ((p[i + k] & 0xC0) != 0x80) { ok = false; break; }
      cp = (cp << 6) | (p[i + k] & 0x3F);
    }
    if (!ok || (len == 3 && cp < 0x800) || (len == 4 && (cp < 0x10000 || cp > 0x10FFFF)) || (cp >= 0xD800 && cp < 0xE000)) {
      out.push_back(0xFFFD); ++i; continue;
    }
    out.push_back(cp);
    i += (size_t)len;
  }
  return out;
}

inline bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (cp < r[mid][0]) hi = mid - 1;
    else if (cp > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
inline bool is_letter(uint32_t c) { return c < 0x80 ? ((c | 32) >= 'a' && (c | 32) <= 'z') : in_ranges(kLetter, kLetter_n, c); }
inline bool is_number(uint32_t c) { return c < 0x80 ? (c >= '0' && c <= '9') : in_ranges(kNumber, kNumber_n, c); }
inline bool is_decimal(uint32_t c) { return c < 0x80 ? (c >= '0' && c <= '9') : in_ranges(kDecimal, kDecimal_n, c); }
inline bool is_mark(uint32_t c) { return c >= 0x300 && in_ranges(kMark, kMark_n, c); }
inline bool is_nonspacing_mark(uint32_t c) { return c >= 0x300 && in_ranges(kNonspacingMark, kNonspacingMark_n, c); }
inline bool is_punct_category(uint32_t c) { return in_ranges(kPunct, kPunct_n, c); }
inline bool is_symbol(uint32_t c) { return in_ranges(kSymbol, kSymbol_n, c); }
inline bool is_separator(uint32_t c) { return in_ranges(kSeparator, kSeparator_n, c); }
inline bool is_other(uint32_t c) { return in_ranges(kControl, kControl_n, c); }     // Cc, Cf, Co, Cn
inline bool is_space(uint32_t c) { return c < 0x80 ? (c == ' ' || (c >= 9 && c <= 13)) : in_ranges(kWhiteSpace, kWhiteSpace_n, c); }
inline bool is_word(uint32_t c) {
  return c < 0x80 ? (((c | 32) >= 'a' && (c | 32) <= 'z') || (c >= '0' && c <= '9') || c == '_') : in_ranges(kWord, kWord_n, c);
}
inline bool is_ascii_punct(uint32_t c) { return (c >= 33 && c <= 47) || (c >= 58 && c <= 64) || (c >= 91 && c <= 96) || (c >= 123 && c <= 126); }

// Index of the code point's two-letter general category in kCatNames, -1 for unassigned code points and surrogates.
inline int category_of(uint32_t c) {
  int lo = 0, hi = kCat_n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (c < kCat[mid][0]) hi = mid - 1;
    else if (c > kCat[mid][1]) lo = mid + 1;
    else return (int)kCat[mid][2];
  }
  return -1;
}
inline int category_index(const std::string& name) {
  for (int i = 0; i < kCatNames_n; ++i) if (name == kCatNames[i]) return i;
  return -1;
}

// The code point's script as the id kScriptIds gives its names, -1 for code points without one.
inline int script_of(uint32_t c) {
  int lo = 0, hi = kScript_n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (c < kScript[mid][0]) hi = mid - 1;
    else if (c > kScript[mid][1]) lo = mid + 1;
    else return (int)kScript[mid][2];
  }
  return -1;
}
inline int script_index(const std::string& name) {          // "Han", "han", "Old_Italic": case, '_', '-' and spaces do not count
  std::string key;
  for (char ch : name) if (ch != '_' && ch != '-' && ch != ' ') key.push_back((char)(ch >= 'a' && ch <= 'z' ? ch - 32 : ch));
  for (int i = 0; i < kScriptNames_n; ++i) if (key == kScriptNames[i]) return kScriptIds[i];
  return -1;
}

template <class Idx>
inline const uint32_t* find3(const Idx& idx, int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (cp < idx[mid][0]) hi = mid - 1;
    else if (cp > idx[mid][0]) lo = mid + 1;
    else return idx[mid];
  }
  return nullptr;
}

inline void lower_into(Text& out, uint32_t c) {
  if (c < 0x80) { out.push_back(c >= 'A' && c <= 'Z' ? c + 32 : c); return; }
  if (const uint32_t* e = find3(kLower_idx, kLower_n, c)) {
    for (uint32_t k = 0; k < e[2]; ++k) out.push_back(kLower_data[e[1] + k]);
  } else {
    out.push_back(c);
  }
}
inline uint32_t lower1(uint32_t c) {          // first code point of the lower-case form (regex case folding)
  if (c < 0x80) return c >= 'A' && c <= 'Z' ? c + 32 : c;
  const uint32_t* e = find3(kLower_idx, kLower_n, c);
  return e ? kLower_data[e[1]] : c;
}
inline Text lowercase(const Text& t) {
  Text out;
  out.reserve(t.size());
  for (uint32_t c : t) lower_into(out, c);
  return out;
}

inline uint32_t ccc(uint32_t c) {
  if (c < 0x300) return 0;
  int lo = 0, hi = kCcc_n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (c < kCcc[mid][0]) hi = mid - 1;
    else if (c > kCcc[mid][0]) lo = mid + 1;
    else return kCcc[mid][1];
  }
  return 0;
}

// Decomposition (canonical, or compatibility when `compat`) followed by the canonical ordering of combining marks.
inline Text decompose(const Text& t, bool compat) {
  Text out;
  out.reserve(t.size() + 8);
  for (uint32_t c : t) {
    if (c < 0xA0) { out.push_back(c); continue; }
    if (c >= 0xAC00 && c <= 0xD7A3) {                  // Hangul syllable: L V (T) by arithmetic
      const uint32_t s = c - 0xAC00;
      out.push_back(0x1100 + s / 588);
      out.push_back(0x1161 + (s % 588) / 28);
      if (s % 28) out.push_back(0x11A7 + s % 28);
      continue;
    }
    const uint32_t* e = compat ? find3(kNfkdExtra_idx, kNfkdExtra_n, c) : nullptr;
    if (e) { for (uint32_t k = 0; k < e[2]; ++k) out.push_back(kNfkdExtra_data[e[1] + k]); continue; }
    e = find3(kNfd_idx, kNfd_n, c);
    if (e) { for (uint32_t k = 0; k < e[2]; ++k) out.push_back(kNfd_data[e[1] + k]); continue; }
    out.push_back(c);
  }
  for (size_t i = 0; i < out.size();) {                // stable sort of each run of non-starters by combining class
    if (ccc(out[i]) == 0) { ++i; continue; }
    size_t j = i;
    while (j < out.size() && ccc(out[j]) != 0) ++j;
    std::stable_sort(out.begin() + (long)i, out.begin() + (long)j, [](uint32_t a, uint32_t b) { return ccc(a) < ccc(b); });
    i = j;
  }
  return out;
}

inline uint32_t compose_pair(uint32_t a, uint32_t b) {
  if (a >= 0x1100 && a < 0x1113 && b >= 0x1161 && b < 0x1176) return 0xAC00 + ((a - 0x1100) * 21 + (b - 0x1161)) * 28;
  if (a >= 0xAC00 && a <= 0xD7A3 && (a - 0xAC00) % 28 == 0 && b > 0x11A7 && b < 0x11C3) return a + (b - 0x11A7);
  int lo = 0, hi = kCompose_n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    const uint32_t* e = kCompose[mid];
    if (a < e[0] || (a == e[0] && b < e[1])) hi = mid - 1;
    else if (a > e[0] || b > e[1]) lo = mid + 1;
    else return e[2];
  }
  return 0;
}

// Canonical composition of a decomposed, canonically ordered text.
inline Text compose(const Text& d) {
  Text out;
  out.reserve(d.size());
  long starter = -1;
  uint32_t last_ccc = 0;
  for (uint32_t c : d) {
    const uint32_t cc = ccc(c);
    if (starter >= 0) {
      const bool adjacent = (size_t)starter + 1 == out.size();
      if (adjacent || (last_ccc < cc && cc != 0) ) {
        // blocked only when a mark of the same or a higher class sits between the starter and c
        if (adjacent || last_ccc < cc) {
          const uint32_t m = compose_pair(out[(size_t)starter], c);
          if (m) { out[(size_t)starter] = m; continue; }
        }
      }
    }
    if (cc == 0) { starter = (long)out.size(); last_ccc = 0; }
    else last_ccc = cc;
    out.push_back(c);
  }
  return out;
}

enum class Form { NFC, NFD, NFKC, NFKD };
inline Text normalize(const Text& t, Form f) {
  const bool compat = f == Form::NFKC || f == Form::NFKD;
  const uint32_t quick = compat ? 0xA0 : 0xC0;         // nothing below decomposes or combines
  bool plain = true;
  for (uint32_t c : t) if (c >= quick) { plain = false; break; }
  if (plain) return t;
  Text d = decompose(t, compat);
  return (f == Form::NFC || f == Form::NFKC) ? compose(d) : d;
}

// Extended grapheme clusters (UAX #29, rules GB3-GB13 without the Indic conjunct rule GB9c): the end index of every cluster of `t`.
// Needs the break tables of the generated header (`kHasGcb`).
enum class Gcb { Other, CR, LF, Control, Extend, ZWJ, RI, Prepend, SpacingMark, L, V, T, LV, LVT };
inline Gcb gcb_of(uint32_t c) {
  if (c == '\r') return Gcb::CR;
  if (c == '\n') return Gcb::LF;
  if (c == 0x200D) return Gcb::ZWJ;
  if (c < 0x300) return (c < 0x20 || (c >= 0x7F && c < 0xA0) || c == 0xAD) ? Gcb::Control : Gcb::Other;
  if (c >= 0x1F1E6 && c <= 0x1F1FF) return Gcb::RI;
  if ((c >= 0x1100 && c <= 0x115F) || (c >= 0xA960 && c <= 0xA97C)) return Gcb::L;
  if ((c >= 0x1160 && c <= 0x11A7) || (c >= 0xD7B0 && c <= 0xD7C6)) return Gcb::V;
  if ((c >= 0x11A8 && c <= 0x11FF) || (c >= 0xD7CB && c <= 0xD7FB)) return Gcb::T;
  if (c >= 0xAC00 && c <= 0xD7A3) return (c - 0xAC00) % 28 == 0 ? Gcb::LV : Gcb::LVT;
  if (in_ranges(kGcbExtend, kGcbExtend_n, c)) return Gcb::Extend;
  if (in_ranges(kGcbSpacingMark, kGcbSpacingMark_n, c)) return Gcb::SpacingMark;
  if (in_ranges(kGcbPrepend, kGcbPrepend_n, c)) return Gcb::Prepend;
  if (in_ranges(kGcbControl, kGcbControl_n, c)) return Gcb::Control;
  return Gcb::Other;
}
inline std::vector<size_t> grapheme_ends(const Text& t) {
  std::vector<size_t> ends;
  const size_t n = t.size();
  size_t i = 0;
  while (i < n) {
    Gcb prev = gcb_of(t[i]);
    bool pict_run = in_ranges(kExtPict, kExtPict_n, t[i]);     // ExtPict Extend* seen so far (GB11)
    bool pict_zwj = false;                                      // ... followed by ZWJ
    int ri = prev == Gcb::RI ? 1 : 0;
    size_t j = i + 1;
    for (; j < n; ++j) {
      const Gcb next = gcb_of(t[j]);
      bool join = false;
      if (prev == Gcb::CR && next == Gcb::LF) join = true;                                                    // GB3
      else if (prev == Gcb::CR || prev == Gcb::LF || prev == Gcb::Control) join = false;                      // GB4
      else if (next == Gcb::CR || next == Gcb::LF || next == Gcb::Control) join = false;                      // GB5
      else if (prev == Gcb::L && (next == Gcb::L || next == Gcb::V || next == Gcb::LV || next == Gcb::LVT)) join = true;   // GB6
      else if ((prev == Gcb::LV || prev == Gcb::V) && (next == Gcb::V || next == Gcb::T)) join = true;        // GB7
      else if ((prev == Gcb::LVT || prev == Gcb::T) && next == Gcb::T) join = true;                           // GB8
      else if (next == Gcb::Extend || next == Gcb::ZWJ || next == Gcb::SpacingMark) join = true;              // GB9, GB9a
      else if (prev == Gcb::Prepend) join = true;                                                             // GB9b
      else if (pict_zwj && in_ranges(kExtPict, kExtPict_n, t[j])) join = true;                                // GB11
      else if (prev == Gcb::RI && next == Gcb::RI && (ri & 1)) join = true;                                   // GB12, GB13
      if (!join) break;
      if (next == Gcb::ZWJ) { pict_zwj = pict_run; }
      else if (next == Gcb::Extend) { pict_zwj = false; }                  // pict_run continues through Extend
      else { pict_zwj = false; pict_run = in_ranges(kExtPict, kExtPict_n, t[j]); }
      ri = next == Gcb::RI ? ri + 1 : 0;
      prev = next;
    }
    ends.push_back(j);
    i = j;
  }
  return ends;
}

}  // namespace uni
}  // namespace lx
