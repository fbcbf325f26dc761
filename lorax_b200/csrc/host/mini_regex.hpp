// A small backtracking regular-expression engine over code points, for the patterns that tokenizer files carry (the GPT-2 /
// cl100k / Llama-3 / Qwen2 split patterns, `Replace` normalisers): literals, escapes (\s \S \d \D \w \W \r \n \t \p{..} \P{..}),
// character classes with ranges and negation, `.`, groups (capturing groups are treated as non-capturing), `(?i:..)` and a leading
// `(?i)`, look-ahead `(?=..)` / `(?!..)`, look-behind of fixed length `(?<=..)` / `(?<!..)`, `\b` `\B` `\A` `\z`, alternation, `^` `$`, and the quantifiers ? * + {m} {m,} {m,n} with lazy (`?`) and
// possessive (`+`, run as greedy) suffixes.  Leftmost match, alternatives tried in order: the semantics of the Oniguruma engine
// the `tokenizers` library splits with.  A pattern outside this subset fails to compile and the caller falls back.
//
// The program is a list of instructions run by a backtracking loop with an explicit stack, so long inputs do not recurse.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "unicode.hpp"

namespace lx {

class MiniRegex {
 public:
  // Compiles `pattern` (UTF-8).  Returns null and sets `err` when the pattern uses something outside the subset.
  static std::unique_ptr<MiniRegex> compile(const std::string& pattern, std::string* err = nullptr) {
    std::unique_ptr<MiniRegex> re(new MiniRegex());
    Parser ps{uni::from_utf8(pattern), 0, false, ""};
    if (ps.src.size() >= 4 && ps.src[0] == '(' && ps.src[1] == '?' && ps.src[2] == 'i' && ps.src[3] == ')') { ps.icase = true; ps.pos = 4; }
    NodeP root = ps.alternation();
    if (!root || ps.pos != ps.src.size()) {
      if (err) *err = ps.err.empty() ? "unsupported pattern syntax at offset " + std::to_string(ps.pos) : ps.err;
      return nullptr;
    }
    re->emit(*root, re->prog_);
    re->prog_.push_back(Inst{Inst::Match});
    return re;
  }

  // Length of the match that starts at `pos`, or -1.
  long match_at(const uint32_t* s, size_t n, size_t pos) const { return run(prog_, s, n, pos); }

  // First match at or after `from`: sets [b, e) and returns true.  An empty match is reported like any other.
  bool search(const uint32_t* s, size_t n, size_t from, size_t* b, size_t* e) const {
    for (size_t i = from; i <= n; ++i) {
      const long len = match_at(s, n, i);
      if (len >= 0) { *b = i; *e = i + (size_t)len; return true; }
    }
    return false;
  }

 private:
  struct Class {                              // a set of code points
    std::vector<std::pair<uint32_t, uint32_t>> ranges;
    std::vector<std::pair<int, bool>> props;      // (property, negated): a letter of s d w L N P M S Z C, 256 + a two-letter category, or 512 + a script
    bool negated = false;
    bool icase = false;
    static bool prop(int p, uint32_t c) {
      if (p >= 512) return uni::script_of(c) == p - 512;
      if (p >= 256) return uni::category_of(c) == p - 256;
      switch (p) {
        case 's': return uni::is_space(c);
        case 'd': return uni::is_decimal(c);
        case 'w': return uni::is_word(c);
        case 'L': return uni::is_letter(c);
        case 'N': return uni::is_number(c);
        case 'P': return uni::is_punct_category(c);
        case 'M': return uni::is_mark(c);
        case 'S': return uni::is_symbol(c);
        case 'Z': return uni::is_separator(c);
        case 'C': return uni::is_other(c);
      }
      return false;
    }
    bool has(uint32_t c) const {
      bool in = false;
      for (auto& r : ranges) if (c >= r.first && c <= r.second) { in = true; break; }
      if (!in && icase) {
        const uint32_t lc = uni::lower1(c);
        for (auto& r : ranges) {
          if (lc >= r.first && lc <= r.second) { in = true; break; }
          // an upper-case range matches the lower-case letter too
          for (uint32_t u = r.first; u <= r.second && r.second - r.first < 64; ++u) if (uni::lower1(u) == lc) { in = true; break; }
          if (in) break;
        }
      }
      if (!in) for (auto& p : props) if (prop(p.first, c) != p.second) { in = true; break; }
      return in != negated;
    }
  };
  struct Node;
  using NodeP = std::unique_ptr<Node>;
  struct Node {
    enum Kind { Set, Any, Seq, Alt, Repeat, Look, Bol, Eol, WordB } kind;
    Class cls;                               // Set
    std::vector<NodeP> kids;                 // Seq, Alt; Repeat and Look use kids[0]
    int min = 0, max = -1;                   // Repeat (max < 0: unbounded)
    bool lazy = false, negative = false;     // Repeat / Look / WordB
    int behind = -1;                         // Look: code points in front of the position that must (not) match; -1: look-ahead
  };
  struct Inst {
    enum Op { Set, Any, Split, Jmp, Look, Bol, Eol, WordB, Match } op;
    int x = 0, y = 0;                        // Split: first and second choice; Jmp: x
    int cls = -1;                            // Set
    int sub = -1;                            // Look: index of the sub-program
    bool negative = false;
    int behind = -1;                         // Look: -1 ahead, else the fixed length looked at behind the position
  };
  using Prog = std::vector<Inst>;

  struct Parser {
    uni::Text src;
    size_t pos;
    bool icase;
    std::string err;
    bool more() const { return pos < src.size(); }
    uint32_t peek() const { return src[pos]; }
    NodeP fail(const std::string& why) { if (err.empty()) err = why; return nullptr; }

    NodeP alternation() {
      auto alt = std::make_unique<Node>();
      alt->kind = Node::Alt;
      while (true) {
        NodeP s = sequence();
        if (!s) return nullptr;
        alt->kids.push_back(std::move(s));
        if (more() && peek() == '|') { ++pos; continue; }
        break;
      }
      if (alt->kids.size() == 1) return std::move(alt->kids[0]);
      return alt;
    }
    NodeP sequence() {
      auto seq = std::make_unique<Node>();
      seq->kind = Node::Seq;
      while (more() && peek() != '|' && peek() != ')') {
        NodeP a = atom();
        if (!a) return nullptr;
        a = quantified(std::move(a));
        if (!a) return nullptr;
        seq->kids.push_back(std::move(a));
      }
      return seq;
    }
    NodeP quantified(NodeP a) {
      while (more()) {
        int mn, mx;
        const uint32_t c = peek();
        if (c == '?') { mn = 0; mx = 1; ++pos; }
        else if (c == '*') { mn = 0; mx = -1; ++pos; }
        else if (c == '+') { mn = 1; mx = -1; ++pos; }
        else if (c == '{') {
          size_t p = pos + 1;
          auto num = [&](int* v) { bool any = false; *v = 0; while (p < src.size() && src[p] >= '0' && src[p] <= '9') { *v = *v * 10 + (int)(src[p] - '0'); ++p; any = true; } return any; };
          if (!num(&mn)) return a;                       // a literal brace
          mx = mn;
          if (p < src.size() && src[p] == ',') { ++p; if (!num(&mx)) mx = -1; }
          if (p >= src.size() || src[p] != '}') return a;
          if (mn > 64 || mx > 64) return fail("repetition count too large");
          pos = p + 1;
        } else {
          return a;
        }
        auto r = std::make_unique<Node>();
        r->kind = Node::Repeat;
        r->min = mn; r->max = mx;
        if (more() && peek() == '?') { r->lazy = true; ++pos; }
        else if (more() && peek() == '+') { ++pos; }     // possessive: run as greedy
        r->kids.push_back(std::move(a));
        a = std::move(r);
      }
      return a;
    }
    // Number of code points a node consumes: [lo, hi]; false when unbounded.
    static bool width(const Node& n, int* lo, int* hi) {
      switch (n.kind) {
        case Node::Set: case Node::Any: *lo = *hi = 1; return true;
        case Node::Bol: case Node::Eol: case Node::Look: case Node::WordB: *lo = *hi = 0; return true;
        case Node::Seq: {
          int a = 0, b = 0;
          for (auto& k : n.kids) { int x, y; if (!width(*k, &x, &y)) return false; a += x; b += y; }
          *lo = a; *hi = b; return true;
        }
        case Node::Alt: {
          int a = 1 << 30, b = 0;
          for (auto& k : n.kids) { int x, y; if (!width(*k, &x, &y)) return false; a = x < a ? x : a; b = y > b ? y : b; }
          *lo = a; *hi = b; return true;
        }
        case Node::Repeat: {
          int x, y;
          if (n.max < 0 || !width(*n.kids[0], &x, &y)) return false;
          *lo = x * n.min; *hi = y * n.max; return true;
        }
      }
      return false;
    }
    NodeP literal(uint32_t c) {
      auto n = std::make_unique<Node>();
      n->kind = Node::Set;
      n->cls.icase = icase;
      n->cls.ranges.push_back({c, c});
      return n;
    }
    // \p{Han}, \p{IsHan}, \p{Script=Han}, \p{sc=Han}, \p{scx=Han} (script extensions are read as the script)
    static int script_name(std::string name) {
      for (const char* pre : {"Script=", "Script_Extensions=", "sc=", "scx=", "Is"})
        if (name.rfind(pre, 0) == 0) { name.erase(0, std::string(pre).size()); break; }
      return uni::script_index(name);
    }
    // After a backslash: a class escape adds to `cls` and returns true; a character escape sets `*lit`.
    bool escape(Class& cls, uint32_t* lit, bool* is_lit) {
      if (!more()) { err = "dangling backslash"; return false; }
      const uint32_t c = src[pos++];
      *is_lit = false;
      switch (c) {
        case 's': case 'd': case 'w': cls.props.push_back({(int)c, false}); return true;
        case 'S': case 'D': case 'W': cls.props.push_back({(int)(c + 32), true}); return true;
        case 'p': case 'P': {
          std::string name;
          if (more() && peek() == '{') {
            ++pos;
            while (more() && peek() != '}') name.push_back((char)src[pos++]);
            if (!more()) { err = "unterminated \\p{"; return false; }
            ++pos;
          } else if (more()) {
            name.push_back((char)src[pos++]);
          }
          bool neg = c == 'P';
          if (!name.empty() && name[0] == '^') { neg = !neg; name.erase(0, 1); }
          int p = 0;
          if (name == "L" || name == "Letter") p = 'L';
          else if (name == "N" || name == "Number") p = 'N';
          else if (name == "P" || name == "Punctuation") p = 'P';
          else if (name == "M" || name == "Mark") p = 'M';
          else if (name == "S" || name == "Symbol") p = 'S';
          else if (name == "Z" || name == "Separator") p = 'Z';
          else if (name == "C" || name == "Other") p = 'C';
          else if (uni::category_index(name) >= 0) p = 256 + uni::category_index(name);
          else if (script_name(name) >= 0) p = 512 + script_name(name);
          else { err = "unsupported property \\p{" + name + "}"; return false; }
          cls.props.push_back({p, neg});
          return true;
        }
        case 'n': *lit = '\n'; break;
        case 'r': *lit = '\r'; break;
        case 't': *lit = '\t'; break;
        case 'f': *lit = '\f'; break;
        case 'v': *lit = '\v'; break;
        case '0': *lit = 0; break;
        case 'x': case 'u': {
          uint32_t v = 0;
          int digits = 0;
          if (more() && peek() == '{') {
            ++pos;
            while (more() && peek() != '}') { const uint32_t h = src[pos++]; v = v * 16 + (h <= '9' ? h - '0' : (h | 32) - 'a' + 10); }
            if (!more()) { err = "unterminated \\x{"; return false; }
            ++pos;
          } else {
            const int want = c == 'x' ? 2 : 4;
            while (digits < want && more()) { const uint32_t h = src[pos++]; v = v * 16 + (h <= '9' ? h - '0' : (h | 32) - 'a' + 10); ++digits; }
          }
          *lit = v;
          break;
        }
        default:
          if ((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '1' && c <= '9')) {
            err = std::string("unsupported escape \\") + (char)c;      // \b, \A, \z, back-references ...
            return false;
          }
          *lit = c;
      }
      *is_lit = true;
      return true;
    }
    NodeP char_class() {                     // after '['
      auto n = std::make_unique<Node>();
      n->kind = Node::Set;
      n->cls.icase = icase;
      if (more() && peek() == '^') { n->cls.negated = true; ++pos; }
      bool first = true;
      while (true) {
        if (!more()) return fail("unterminated character class");
        uint32_t c = src[pos];
        if (c == ']' && !first) { ++pos; break; }
        first = false;
        if (c == '[') return fail("nested character class");
        ++pos;
        bool is_lit = true;
        if (c == '\\') {
          if (!escape(n->cls, &c, &is_lit)) return nullptr;
          if (!is_lit) continue;
        }
        uint32_t hi = c;
        if (pos + 1 < src.size() && src[pos] == '-' && src[pos + 1] != ']') {
          pos += 1;
          hi = src[pos++];
          if (hi == '\\') {
            bool hl = true;
            Class tmp;
            if (!escape(tmp, &hi, &hl) || !hl) return fail("class escape as a range end");
          }
          if (hi < c) return fail("reversed range");
        }
        n->cls.ranges.push_back({c, hi});
      }
      return n;
    }
    NodeP atom() {
      const uint32_t c = src[pos++];
      switch (c) {
        case '(': {
          bool saved = icase;
          bool look = false, negative = false, behind = false;
          if (more() && peek() == '?') {
            ++pos;
            if (!more()) return fail("dangling (?");
            const uint32_t k = src[pos++];
            if (k == ':') {
            } else if (k == '=' || k == '!') {
              look = true; negative = k == '!';
            } else if (k == 'i' && more() && peek() == ':') {
              ++pos; icase = true;
            } else if (k == '<' && more() && (peek() == '=' || peek() == '!')) {
              look = true; behind = true; negative = src[pos++] == '!';
            } else if (k == '<' || k == 'P' || k == '\'') {
              return fail("named groups are not supported");
            } else {
              return fail("unsupported group flag");
            }
          }
          NodeP inner = alternation();
          if (!inner) return nullptr;
          if (!more() || peek() != ')') return fail("unbalanced parenthesis");
          ++pos;
          icase = saved;
          if (!look) return inner;
          auto l = std::make_unique<Node>();
          l->kind = Node::Look;
          l->negative = negative;
          if (behind) {
            int lo = 0, hi = 0;
            if (!width(*inner, &lo, &hi) || lo != hi) return fail("look-behind of variable length");
            l->behind = lo;
          }
          l->kids.push_back(std::move(inner));
          return l;
        }
        case '[': return char_class();
        case '.': { auto n = std::make_unique<Node>(); n->kind = Node::Any; return n; }
        case '^': { auto n = std::make_unique<Node>(); n->kind = Node::Bol; return n; }
        case '$': { auto n = std::make_unique<Node>(); n->kind = Node::Eol; return n; }
        case '\\': {
          if (more() && (peek() == 'b' || peek() == 'B')) {
            auto n = std::make_unique<Node>();
            n->kind = Node::WordB;
            n->negative = src[pos++] == 'B';
            return n;
          }
          if (more() && (peek() == 'A' || peek() == 'z')) {
            auto n = std::make_unique<Node>();
            n->kind = src[pos++] == 'A' ? Node::Bol : Node::Eol;
            return n;
          }
          auto n = std::make_unique<Node>();
          n->kind = Node::Set;
          n->cls.icase = icase;
          uint32_t lit = 0;
          bool is_lit = false;
          if (!escape(n->cls, &lit, &is_lit)) return nullptr;
          if (is_lit) n->cls.ranges.push_back({lit, lit});
          return n;
        }
        case '*': case '+': case '?': return fail("quantifier without an operand");
        default: return literal(c);
      }
    }
  };

  void emit(const Node& n, Prog& out) {
    switch (n.kind) {
      case Node::Set: { Inst i{Inst::Set}; i.cls = (int)classes_.size(); classes_.push_back(n.cls); out.push_back(i); break; }
      case Node::Any: out.push_back(Inst{Inst::Any}); break;
      case Node::Bol: out.push_back(Inst{Inst::Bol}); break;
      case Node::Eol: out.push_back(Inst{Inst::Eol}); break;
      case Node::WordB: { Inst i{Inst::WordB}; i.negative = n.negative; out.push_back(i); break; }
      case Node::Seq: for (auto& k : n.kids) emit(*k, out); break;
      case Node::Alt: {
        std::vector<int> jumps;
        for (size_t k = 0; k < n.kids.size(); ++k) {
          if (k + 1 < n.kids.size()) {
            const int split = (int)out.size();
            out.push_back(Inst{Inst::Split});
            out[(size_t)split].x = split + 1;
            emit(*n.kids[k], out);
            jumps.push_back((int)out.size());
            out.push_back(Inst{Inst::Jmp});
            out[(size_t)split].y = (int)out.size();
          } else {
            emit(*n.kids[k], out);
          }
        }
        for (int j : jumps) out[(size_t)j].x = (int)out.size();
        break;
      }
      case Node::Repeat: {
        for (int k = 0; k < n.min; ++k) emit(*n.kids[0], out);
        if (n.max < 0) {                                   // loop: L: split body, out; body; jmp L
          const int loop = (int)out.size();
          out.push_back(Inst{Inst::Split});
          emit(*n.kids[0], out);
          Inst j{Inst::Jmp}; j.x = loop;
          out.push_back(j);
          const int after = (int)out.size();
          out[(size_t)loop].x = n.lazy ? after : loop + 1;
          out[(size_t)loop].y = n.lazy ? loop + 1 : after;
        } else {
          std::vector<int> splits;
          for (int k = n.min; k < n.max; ++k) {
            splits.push_back((int)out.size());
            out.push_back(Inst{Inst::Split});
            emit(*n.kids[0], out);
          }
          const int after = (int)out.size();
          for (int s : splits) {
            out[(size_t)s].x = n.lazy ? after : s + 1;
            out[(size_t)s].y = n.lazy ? s + 1 : after;
          }
        }
        break;
      }
      case Node::Look: {
        Inst i{Inst::Look};
        i.negative = n.negative;
        i.behind = n.behind;
        i.sub = (int)subs_.size();
        subs_.emplace_back();
        Prog sub;
        emit(*n.kids[0], sub);
        sub.push_back(Inst{Inst::Match});
        subs_[(size_t)i.sub] = std::move(sub);
        out.push_back(i);
        break;
      }
    }
  }

  long run(const Prog& prog, const uint32_t* s, size_t n, size_t start) const {
    struct Thread { int pc; size_t pos; };
    std::vector<Thread> stack;
    stack.push_back({0, start});
    size_t steps = 0;
    while (!stack.empty()) {
      Thread t = stack.back();
      stack.pop_back();
      while (true) {
        if (++steps > kStepLimit) return -1;               // a pathological pattern gives up instead of spinning
        const Inst& in = prog[(size_t)t.pc];
        bool dead = false;
        switch (in.op) {
          case Inst::Set:
            if (t.pos < n && classes_[(size_t)in.cls].has(s[t.pos])) { ++t.pos; ++t.pc; } else dead = true;
            break;
          case Inst::Any:
            if (t.pos < n && s[t.pos] != '\n') { ++t.pos; ++t.pc; } else dead = true;
            break;
          case Inst::Bol: if (t.pos == 0) ++t.pc; else dead = true; break;
          case Inst::Eol: if (t.pos == n) ++t.pc; else dead = true; break;
          case Inst::Jmp: t.pc = in.x; break;
          case Inst::Split:
            // an empty loop body must not spin: the second choice is only pushed, never re-entered at the same position
            stack.push_back({in.y, t.pos});
            t.pc = in.x;
            break;
          case Inst::WordB: {
            const bool before = t.pos > 0 && uni::is_word(s[t.pos - 1]), after = t.pos < n && uni::is_word(s[t.pos]);
            if ((before != after) != in.negative) ++t.pc; else dead = true;
            break;
          }
          case Inst::Look: {
            bool hit;
            if (in.behind < 0) hit = run(subs_[(size_t)in.sub], s, n, t.pos) >= 0;
            else hit = t.pos >= (size_t)in.behind && run(subs_[(size_t)in.sub], s, n, t.pos - (size_t)in.behind) == (long)in.behind;
            if (hit != in.negative) ++t.pc; else dead = true;
            break;
          }
          case Inst::Match: return (long)(t.pos - start);
        }
        if (dead) break;
      }
    }
    return -1;
  }

  static constexpr size_t kStepLimit = 50u * 1000 * 1000;
  Prog prog_;
  std::vector<Prog> subs_;
  std::vector<Class> classes_;
};

}  // namespace lx
