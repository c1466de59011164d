// A Jinja subset for chat templates: the statements, expressions, filters and tests that the chat templates shipped
// in tokenizer_config.json files use, with the environment settings of the Hugging Face renderer (trim_blocks and
// lstrip_blocks on, tojson = json.dumps(ensure_ascii=False), raise_exception, namespace, loop controls).  Values are
// b2::Json (insertion-ordered objects, int / float kept apart), so tojson reproduces Python's formatting.
// Reference: crates/agens-server/src/template.rs (minijinja environment with the same additions).
#include <cmath>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../core/json.hpp"
#include "text.hpp"

namespace b2 {
namespace jinja {

struct Error : std::runtime_error { using std::runtime_error::runtime_error; };

struct Val {
  Json j;
  bool undef = false;
  Val() : undef(true) {}
  Val(Json v) : j(std::move(v)) {}
};

// ------------------------------------------------------------------------------------------------ expression AST
struct Expr;
using ExprP = std::shared_ptr<Expr>;
struct Expr {
  enum Kind { Lit, Name, Attr, Index, Slice, Call, Filter, Test, Not, Neg, Bin, Cond, List, Dict } kind;
  Json lit;
  std::string name;                       // Name, Attr (attribute), Filter / Test (name), Bin (operator)
  ExprP a, b, c, d;                       // operands (Slice: a[b:c:d]; Cond: a if b else c)
  std::vector<ExprP> args;                // Call / Filter / Test / List; Dict: key, value, key, value ...
  std::vector<std::pair<std::string, ExprP>> kwargs;
  bool negated = false;                   // Test: "is not"
};

struct Tok { enum T { End, Num, Str, Id, Op } t = End; std::string s; Json num; };

static std::vector<Tok> lex_expr(const std::string& src) {
  std::vector<Tok> out;
  size_t i = 0, n = src.size();
  while (i < n) {
    const char ch = src[i];
    if (std::isspace((unsigned char)ch)) { ++i; continue; }
    Tok t;
    if (std::isdigit((unsigned char)ch)) {
      size_t j = i; bool fl = false;
      while (j < n && (std::isdigit((unsigned char)src[j]) || (src[j] == '.' && j + 1 < n && std::isdigit((unsigned char)src[j + 1])))) { if (src[j] == '.') fl = true; ++j; }
      t.t = Tok::Num; t.s = src.substr(i, j - i);
      t.num = fl ? Json(std::stod(t.s)) : Json((long long)std::stoll(t.s));
      i = j;
    } else if (std::isalpha((unsigned char)ch) || ch == '_') {
      size_t j = i;
      while (j < n && (std::isalnum((unsigned char)src[j]) || src[j] == '_')) ++j;
      t.t = Tok::Id; t.s = src.substr(i, j - i); i = j;
    } else if (ch == '"' || ch == '\'') {
      std::string v; size_t j = i + 1;
      for (; j < n && src[j] != ch; ++j) {
        if (src[j] == '\\' && j + 1 < n) {
          const char e = src[++j];
          v.push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e == 'r' ? '\r' : e);
        } else v.push_back(src[j]);
      }
      if (j >= n) throw Error("unterminated string literal");
      t.t = Tok::Str; t.s = v; i = j + 1;
    } else {
      static const char* two[] = {"==", "!=", "<=", ">=", "//", "**"};
      t.t = Tok::Op;
      bool m = false;
      for (auto op : two) if (src.compare(i, 2, op) == 0) { t.s = op; i += 2; m = true; break; }
      if (!m) { t.s = std::string(1, ch); ++i; }
    }
    out.push_back(t);
  }
  out.push_back(Tok());
  return out;
}

// Recursion limits: a template is configuration, but one that nests without end must be refused, not overflow the stack.
constexpr int kMaxExprDepth = 600;       // three counted frames per level: about 200 nested parentheses, literals or unary operators
constexpr int kMaxExprTokens = 20000;    // bounds the length of an operator chain (its tree is as deep as it is long)
constexpr int kMaxBlockDepth = 200;      // nested if / for / macro / set blocks
constexpr int kMaxEvalDepth = 1000;      // expression evaluation (an operator chain evaluates through its left spine)
constexpr int kMaxMacroDepth = 100;      // macro calls in flight
struct DepthGuard {
  int& d;
  DepthGuard(int& depth, int limit, const char* what) : d(depth) { if (++d > limit) { --d; throw Error(std::string(what) + " nested too deeply"); } }
  ~DepthGuard() { --d; }
};

class ExprParser {
 public:
  explicit ExprParser(std::vector<Tok> t) : t_(std::move(t)) { if (t_.size() > (size_t)kMaxExprTokens) throw Error("expression too long"); }
  ExprP parse_full() { ExprP e = parse_cond(); if (cur().t != Tok::End) throw Error("unexpected '" + cur().s + "' in expression"); return e; }
  ExprP parse_cond() {
    DepthGuard g(depth_, kMaxExprDepth, "expression");
    ExprP e = parse_or();
    while (is_id("if")) {
      ++p_;
      auto n = mk(Expr::Cond); n->a = e; n->b = parse_or();
      if (is_id("else")) { ++p_; n->c = parse_cond(); }
      e = n;
    }
    return e;
  }
  ExprP parse_iterable() { return parse_or(); }           // no conditional expression: "if" is left to the caller
  const Tok& cur() const { return t_[p_]; }
  bool is_id(const char* s) const { return cur().t == Tok::Id && cur().s == s; }
  bool is_op(const char* s) const { return cur().t == Tok::Op && cur().s == s; }
  void expect_op(const char* s) { if (!is_op(s)) throw Error(std::string("expected '") + s + "'"); ++p_; }
  std::string take_id() { if (cur().t != Tok::Id) throw Error("expected a name"); return t_[p_++].s; }
  bool at_end() const { return cur().t == Tok::End; }
  size_t p_ = 0;

 private:
  std::vector<Tok> t_;
  int depth_ = 0;
  static ExprP mk(Expr::Kind k) { auto e = std::make_shared<Expr>(); e->kind = k; return e; }
  static ExprP bin(const std::string& op, ExprP a, ExprP b) { auto e = mk(Expr::Bin); e->name = op; e->a = a; e->b = b; return e; }
  ExprP parse_or() { ExprP e = parse_and(); while (is_id("or")) { ++p_; e = bin("or", e, parse_and()); } return e; }
  ExprP parse_and() { ExprP e = parse_not(); while (is_id("and")) { ++p_; e = bin("and", e, parse_not()); } return e; }
  ExprP parse_not() {
    DepthGuard g(depth_, kMaxExprDepth, "expression");
    if (is_id("not")) { ++p_; auto e = mk(Expr::Not); e->a = parse_not(); return e; }
    return parse_cmp();
  }
  ExprP parse_cmp() {
    ExprP e = parse_add();
    for (;;) {
      if (cur().t == Tok::Op && (cur().s == "==" || cur().s == "!=" || cur().s == "<" || cur().s == ">" || cur().s == "<=" || cur().s == ">=")) {
        const std::string op = t_[p_++].s; e = bin(op, e, parse_add());
      } else if (is_id("in")) { ++p_; e = bin("in", e, parse_add()); }
      else if (is_id("not") && t_[p_ + 1].t == Tok::Id && t_[p_ + 1].s == "in") { p_ += 2; auto n = mk(Expr::Not); n->a = bin("in", e, parse_add()); e = n; }
      else return e;
    }
  }
  ExprP parse_add() {
    ExprP e = parse_concat();
    while (is_op("+") || is_op("-")) { const std::string op = t_[p_++].s; e = bin(op, e, parse_concat()); }
    return e;
  }
  ExprP parse_concat() { ExprP e = parse_mul(); while (is_op("~")) { ++p_; e = bin("~", e, parse_mul()); } return e; }
  ExprP parse_mul() {
    ExprP e = parse_unary();
    while (is_op("*") || is_op("/") || is_op("//") || is_op("%")) { const std::string op = t_[p_++].s; e = bin(op, e, parse_unary()); }
    return e;
  }
  ExprP parse_unary() {
    DepthGuard g(depth_, kMaxExprDepth, "expression");
    if (is_op("-")) { ++p_; auto e = mk(Expr::Neg); e->a = parse_unary(); return e; }
    if (is_op("+")) { ++p_; return parse_unary(); }
    return parse_postfix(parse_primary());
  }
  void parse_call_args(Expr& e) {
    while (!is_op(")")) {
      if (cur().t == Tok::Id && t_[p_ + 1].t == Tok::Op && t_[p_ + 1].s == "=") { std::string k = t_[p_].s; p_ += 2; e.kwargs.emplace_back(k, parse_cond()); }
      else e.args.push_back(parse_cond());
      if (is_op(",")) ++p_; else break;
    }
    expect_op(")");
  }
  ExprP parse_postfix(ExprP e) {
    for (;;) {
      if (is_op(".")) { ++p_; auto n = mk(Expr::Attr); n->a = e; n->name = cur().t == Tok::Num ? t_[p_++].s : take_id(); e = n; }
      else if (is_op("[")) {
        ++p_;
        ExprP first;
        if (!is_op(":")) first = parse_cond();
        if (is_op(":")) {
          auto n = mk(Expr::Slice); n->a = e; n->b = first;
          ++p_;
          if (!is_op(":") && !is_op("]")) n->c = parse_cond();
          if (is_op(":")) { ++p_; if (!is_op("]")) n->d = parse_cond(); }
          e = n;
        } else { auto n = mk(Expr::Index); n->a = e; n->b = first; e = n; }
        expect_op("]");
      } else if (is_op("(")) { ++p_; auto n = mk(Expr::Call); n->a = e; parse_call_args(*n); e = n; }
      else if (is_op("|")) {
        ++p_;
        auto n = mk(Expr::Filter); n->a = e; n->name = take_id();
        if (is_op("(")) { ++p_; parse_call_args(*n); }
        e = n;
      } else if (is_id("is")) {
        ++p_;
        auto n = mk(Expr::Test); n->a = e;
        if (is_id("not")) { ++p_; n->negated = true; }
        n->name = take_id();
        if (is_op("(")) { ++p_; parse_call_args(*n); }
        else if (cur().t == Tok::Str || cur().t == Tok::Num || (cur().t == Tok::Id && !is_id("and") && !is_id("or") && !is_id("else") && !is_id("if") && !is_id("in") && !is_id("is") && !is_id("not")))
          n->args.push_back(parse_postfix(parse_primary()));
        e = n;
      } else return e;
    }
  }
  ExprP parse_primary() {
    const Tok t = cur();
    if (t.t == Tok::Num) { ++p_; auto e = mk(Expr::Lit); e->lit = t.num; return e; }
    if (t.t == Tok::Str) {
      ++p_; auto e = mk(Expr::Lit); std::string s = t.s;
      while (cur().t == Tok::Str) s += t_[p_++].s;                    // adjacent literals concatenate
      e->lit = Json(s); return e;
    }
    if (t.t == Tok::Id) {
      ++p_;
      if (t.s == "true" || t.s == "True") { auto e = mk(Expr::Lit); e->lit = Json(true); return e; }
      if (t.s == "false" || t.s == "False") { auto e = mk(Expr::Lit); e->lit = Json(false); return e; }
      if (t.s == "none" || t.s == "None") { auto e = mk(Expr::Lit); return e; }
      auto e = mk(Expr::Name); e->name = t.s; return e;
    }
    if (is_op("(")) {
      ++p_;
      ExprP e = parse_cond();
      if (is_op(",")) {                                               // tuple literal: treated as a list
        auto l = mk(Expr::List); l->args.push_back(e);
        while (is_op(",")) { ++p_; if (is_op(")")) break; l->args.push_back(parse_cond()); }
        e = l;
      }
      expect_op(")");
      return e;
    }
    if (is_op("[")) {
      ++p_; auto l = mk(Expr::List);
      while (!is_op("]")) { l->args.push_back(parse_cond()); if (is_op(",")) ++p_; else break; }
      expect_op("]");
      return l;
    }
    if (is_op("{")) {
      ++p_; auto d = mk(Expr::Dict);
      while (!is_op("}")) { d->args.push_back(parse_cond()); expect_op(":"); d->args.push_back(parse_cond()); if (is_op(",")) ++p_; else break; }
      expect_op("}");
      return d;
    }
    throw Error("unexpected '" + t.s + "' in expression");
  }
};

// ------------------------------------------------------------------------------------------------ statement AST
struct Node;
using NodeP = std::shared_ptr<Node>;
using Body = std::vector<NodeP>;
struct Node {
  enum Kind { Text, Output, If, For, Set, SetBlock, Macro, Break, Continue } kind;
  std::string text;                                   // Text; Set / SetBlock / Macro: target name
  std::string attr;                                   // Set: "ns.attr" target
  ExprP expr;                                         // Output, Set value, For iterable
  ExprP filter;                                       // For ... if cond
  std::vector<std::pair<ExprP, Body>> branches;       // If / elif (null condition = else)
  std::vector<std::string> targets;                   // For loop variables
  Body body, else_body;
  std::vector<std::pair<std::string, ExprP>> params;  // Macro parameters with optional defaults
};

struct Piece { enum T { Text, Out, Stmt } t; std::string s; };

// Splits the source into text / {{ }} / {% %} pieces with the whitespace rules of the Hugging Face environment:
// "-" on either side of a tag strips all whitespace there; trim_blocks drops one newline after a block tag or comment;
// lstrip_blocks drops the blanks between a line start and a block tag or comment ("+" switches either off).
static std::vector<Piece> split_template(const std::string& src) {
  std::vector<Piece> out;
  size_t i = 0;
  const size_t n = src.size();
  std::string text;
  bool trim_next = false;            // the previous tag ended with "-": strip the whitespace that follows
  bool line_starting = true;         // the current text began at a line start (template start, or a dropped newline)
  auto emit_text = [&]() {
    if (trim_next) { size_t k = 0; while (k < text.size() && std::isspace((unsigned char)text[k])) ++k; text.erase(0, k); }
    if (!text.empty()) out.push_back({Piece::Text, text});
    text.clear();
  };
  while (i < n) {
    if (!(src[i] == '{' && i + 1 < n && (src[i + 1] == '{' || src[i + 1] == '%' || src[i + 1] == '#'))) { text.push_back(src[i++]); continue; }
    const char kind = src[i + 1];
    const char c0 = kind == '{' ? '}' : kind;
    size_t j = i + 2;
    bool lminus = false, lplus = false;
    if (j < n && src[j] == '-') { lminus = true; ++j; }
    else if (j < n && src[j] == '+' && kind != '{') { lplus = true; ++j; }
    size_t k = j;
    char q = 0;
    for (; k + 1 < n; ++k) {                       // the closing delimiter, outside string literals
      if (kind != '#') {
        if (q) { if (src[k] == '\\') ++k; else if (src[k] == q) q = 0; continue; }
        if (src[k] == '"' || src[k] == '\'') { q = src[k]; continue; }
      }
      if (src[k] == c0 && src[k + 1] == '}') break;
    }
    if (k + 1 >= n) throw Error("unclosed template tag");
    size_t e = k;
    bool rminus = false, rplus = false;
    if (e > j && src[e - 1] == '-') { rminus = true; --e; }
    else if (e > j && src[e - 1] == '+' && kind != '{') { rplus = true; --e; }
    if (lminus) { while (!text.empty() && std::isspace((unsigned char)text.back())) text.pop_back(); }
    else if (kind != '{' && !lplus) {
      const size_t nl = text.rfind('\n');
      const size_t l_pos = nl == std::string::npos ? 0 : nl + 1;
      if (nl != std::string::npos || line_starting) {
        bool blanks = true;
        for (size_t b = l_pos; b < text.size(); ++b) if (text[b] != ' ' && text[b] != '\t') { blanks = false; break; }
        if (blanks) text.resize(l_pos);
      }
    }
    emit_text();
    if (kind != '#') out.push_back({kind == '{' ? Piece::Out : Piece::Stmt, src.substr(j, e - j)});
    i = k + 2;
    trim_next = rminus;
    line_starting = false;
    if (kind != '{' && !rminus && !rplus && i < n && src[i] == '\n') { ++i; line_starting = true; }
  }
  emit_text();
  return out;
}

// ------------------------------------------------------------------------------------------------ statements
static std::string first_word(const std::string& s, size_t* rest) {
  size_t a = 0;
  while (a < s.size() && std::isspace((unsigned char)s[a])) ++a;
  size_t b = a;
  while (b < s.size() && (std::isalnum((unsigned char)s[b]) || s[b] == '_')) ++b;
  if (rest) *rest = b;
  return s.substr(a, b - a);
}

class TemplateParser {
 public:
  explicit TemplateParser(std::vector<Piece> p) : p_(std::move(p)) {}
  Body parse() {
    std::string end;
    Body b = parse_body({}, &end);
    return b;
  }

 private:
  std::vector<Piece> p_;
  size_t i_ = 0;
  int depth_ = 0;
  static ExprP expr_of(const std::string& s) { return ExprParser(lex_expr(s)).parse_full(); }

  // Parses until one of the `stops` keywords opens a statement; *stop receives that statement's text.
  Body parse_body(const std::vector<std::string>& stops, std::string* stop) {
    DepthGuard g(depth_, kMaxBlockDepth, "blocks");
    Body body;
    while (i_ < p_.size()) {
      const Piece& pc = p_[i_++];
      if (pc.t == Piece::Text) { auto n = std::make_shared<Node>(); n->kind = Node::Text; n->text = pc.s; body.push_back(n); continue; }
      if (pc.t == Piece::Out) { auto n = std::make_shared<Node>(); n->kind = Node::Output; n->expr = expr_of(pc.s); body.push_back(n); continue; }
      size_t rest = 0;
      const std::string kw = first_word(pc.s, &rest);
      for (auto& s : stops) if (kw == s) { *stop = pc.s; return body; }
      const std::string tail = pc.s.substr(rest);
      auto n = std::make_shared<Node>();
      if (kw == "if") {
        n->kind = Node::If;
        ExprP cond = expr_of(tail);
        for (;;) {
          std::string st;
          Body b = parse_body({"elif", "else", "endif"}, &st);
          n->branches.emplace_back(cond, std::move(b));
          size_t r = 0;
          const std::string k2 = first_word(st, &r);
          if (k2 == "endif") break;
          if (k2 == "elif") { cond = expr_of(st.substr(r)); continue; }
          if (k2 == "else") { cond = nullptr; std::string st2; Body eb = parse_body({"endif"}, &st2); n->branches.emplace_back(nullptr, std::move(eb)); if (first_word(st2, nullptr) != "endif") throw Error("missing endif"); break; }
          throw Error("missing endif");
        }
      } else if (kw == "for") {
        n->kind = Node::For;
        std::vector<Tok> toks = lex_expr(tail);
        ExprParser ep(toks);
        for (;;) {
          if (ep.is_op("(")) { ++ep.p_; continue; }
          n->targets.push_back(ep.take_id());
          if (ep.is_op(")")) ++ep.p_;
          if (ep.is_op(",")) { ++ep.p_; continue; }
          break;
        }
        if (!ep.is_id("in")) throw Error("expected 'in' in for statement");
        ++ep.p_;
        // the iterable is an or-expression, so that "if" starts the loop filter and not a conditional expression
        n->expr = parse_no_cond(ep);
        if (ep.is_id("if")) { ++ep.p_; n->filter = ep.parse_cond(); }
        if (ep.is_id("recursive")) ++ep.p_;
        if (!ep.at_end()) throw Error("unexpected '" + ep.cur().s + "' in for statement");
        std::string st;
        n->body = parse_body({"else", "endfor"}, &st);
        if (first_word(st, nullptr) == "else") { std::string st2; n->else_body = parse_body({"endfor"}, &st2); st = st2; }
        if (first_word(st, nullptr) != "endfor") throw Error("missing endfor");
      } else if (kw == "set") {
        std::vector<Tok> toks = lex_expr(tail);
        ExprParser ep(toks);
        n->text = ep.take_id();
        if (ep.is_op(".")) { ++ep.p_; n->attr = ep.take_id(); }
        if (ep.is_op("=")) { ++ep.p_; n->kind = Node::Set; n->expr = ep.parse_cond(); if (!ep.at_end()) throw Error("unexpected '" + ep.cur().s + "' in set statement"); }
        else {
          n->kind = Node::SetBlock;
          if (ep.is_op("|")) { /* a filtered block: the filter chain applies to the captured text */
            std::string chain = "__block__";
            size_t bar = tail.find('|');
            chain += tail.substr(bar);
            n->expr = expr_of(chain);
          }
          std::string st;
          n->body = parse_body({"endset"}, &st);
          if (first_word(st, nullptr) != "endset") throw Error("missing endset");
        }
      } else if (kw == "macro") {
        n->kind = Node::Macro;
        std::vector<Tok> toks = lex_expr(tail);
        ExprParser ep(toks);
        n->text = ep.take_id();
        ep.expect_op("(");
        while (!ep.is_op(")")) {
          std::string pn = ep.take_id();
          ExprP def;
          if (ep.is_op("=")) { ++ep.p_; def = ep.parse_cond(); }
          n->params.emplace_back(pn, def);
          if (ep.is_op(",")) ++ep.p_; else break;
        }
        ep.expect_op(")");
        std::string st;
        n->body = parse_body({"endmacro"}, &st);
        if (first_word(st, nullptr) != "endmacro") throw Error("missing endmacro");
      } else if (kw == "generation") {            // assistant-mask markers: the content passes through
        std::string st;
        Body b = parse_body({"endgeneration"}, &st);
        for (auto& x : b) body.push_back(x);
        continue;
      } else if (kw == "break") { n->kind = Node::Break; }
      else if (kw == "continue") { n->kind = Node::Continue; }
      else throw Error("unsupported statement: " + kw);
      body.push_back(n);
    }
    if (!stops.empty()) throw Error("missing " + stops.back());
    return body;
  }
  static ExprP parse_no_cond(ExprParser& ep) {
    // parse_cond would swallow "if"; walk one level below it by parsing and stopping at "if"
    return ep.parse_iterable();
  }
};

// ------------------------------------------------------------------------------------------------ values
static bool truthy(const Val& v) {
  if (v.undef) return false;
  switch (v.j.type()) {
    case Json::Null: return false;
    case Json::Bool: return v.j.as_bool();
    case Json::Int: return v.j.as_int() != 0;
    case Json::Double: return v.j.as_double() != 0.0;
    case Json::String: return !v.j.as_string().empty();
    default: return v.j.size() > 0;
  }
}

static std::string py_repr(const Json& j);
static std::string py_str(const Json& j) {
  switch (j.type()) {
    case Json::Null: return "None";
    case Json::Bool: return j.as_bool() ? "True" : "False";
    case Json::String: return j.as_string();
    case Json::Int: return std::to_string(j.as_int());
    case Json::Double: { std::string s = j.dump(); if (s.find_first_of(".eEn") == std::string::npos) s += ".0"; return s; }
    default: return py_repr(j);
  }
}
static std::string py_repr(const Json& j) {
  if (j.is_string()) {
    const std::string& s = j.as_string();
    const char q = s.find('\'') != std::string::npos && s.find('"') == std::string::npos ? '"' : '\'';
    std::string o(1, q);
    for (char ch : s) {
      if (ch == '\\' || ch == q) { o.push_back('\\'); o.push_back(ch); }
      else if (ch == '\n') o += "\\n";
      else if (ch == '\t') o += "\\t";
      else if (ch == '\r') o += "\\r";
      else o.push_back(ch);
    }
    o.push_back(q);
    return o;
  }
  if (j.is_array()) {
    std::string o = "[";
    for (size_t i = 0; i < j.size(); ++i) { if (i) o += ", "; o += py_repr(j[i]); }
    return o + "]";
  }
  if (j.is_object()) {
    std::string o = "{";
    bool first = true;
    for (auto& kv : j.members()) { if (!first) o += ", "; first = false; o += py_repr(Json(kv.first)) + ": " + py_repr(kv.second); }
    return o + "}";
  }
  return py_str(j);
}
static std::string to_str(const Val& v) { return v.undef ? std::string() : py_str(v.j); }

static void dump_indented(const Json& j, int indent, int depth, std::string& out) {
  const Json::Style st{true, false};
  if (j.is_array() && j.size()) {
    out += "[\n";
    for (size_t i = 0; i < j.size(); ++i) {
      out.append((size_t)indent * (depth + 1), ' ');
      dump_indented(j[i], indent, depth + 1, out);
      out += i + 1 < j.size() ? ",\n" : "\n";
    }
    out.append((size_t)indent * depth, ' '); out += "]";
  } else if (j.is_object() && j.size()) {
    out += "{\n";
    size_t i = 0;
    for (auto& kv : j.members()) {
      out.append((size_t)indent * (depth + 1), ' ');
      out += Json(kv.first).dump(st) + ": ";
      dump_indented(kv.second, indent, depth + 1, out);
      out += ++i < j.size() ? ",\n" : "\n";
    }
    out.append((size_t)indent * depth, ' '); out += "}";
  } else out += j.dump(st);
}

static bool json_equal(const Json& a, const Json& b) {
  if (a.is_number() && b.is_number()) return a.is_int() && b.is_int() ? a.as_int() == b.as_int() : a.as_double() == b.as_double();
  if (a.is_bool() && b.is_number()) return (a.as_bool() ? 1.0 : 0.0) == b.as_double();
  if (b.is_bool() && a.is_number()) return (b.as_bool() ? 1.0 : 0.0) == a.as_double();
  if (a.type() != b.type()) return false;
  switch (a.type()) {
    case Json::Null: return true;
    case Json::Bool: return a.as_bool() == b.as_bool();
    case Json::String: return a.as_string() == b.as_string();
    case Json::Array:
      if (a.size() != b.size()) return false;
      for (size_t i = 0; i < a.size(); ++i) if (!json_equal(a[i], b[i])) return false;
      return true;
    case Json::Object:
      if (a.size() != b.size()) return false;
      for (auto& kv : a.members()) { const Json* o = b.find(kv.first); if (!o || !json_equal(kv.second, *o)) return false; }
      return true;
    default: return false;
  }
}
static bool val_equal(const Val& a, const Val& b) { return a.undef || b.undef ? a.undef == b.undef : json_equal(a.j, b.j); }

static int json_compare(const Json& a, const Json& b) {
  if (a.is_number() && b.is_number()) { const double x = a.as_double(), y = b.as_double(); return x < y ? -1 : x > y ? 1 : 0; }
  if (a.is_string() && b.is_string()) return a.as_string().compare(b.as_string()) < 0 ? -1 : a.as_string() == b.as_string() ? 0 : 1;
  throw Error("values of these types cannot be ordered");
}

static std::string strip_chars(const std::string& s, const std::string& chars, bool left, bool right) {
  auto is_strip = [&](char ch) { return chars.empty() ? std::isspace((unsigned char)ch) != 0 : chars.find(ch) != std::string::npos; };
  size_t a = 0, b = s.size();
  if (left) while (a < b && is_strip(s[a])) ++a;
  if (right) while (b > a && is_strip(s[b - 1])) --b;
  return s.substr(a, b - a);
}

static size_t utf8_len(const std::string& s) { size_t n = 0; for (unsigned char ch : s) if ((ch & 0xC0) != 0x80) ++n; return n; }

static std::string case_map(const std::string& s, int mode) {       // 0 lower, 1 upper, 2 title, 3 capitalize (ASCII)
  std::string o = s;
  bool start = true;
  for (size_t i = 0; i < o.size(); ++i) {
    const unsigned char ch = o[i];
    if (mode == 0) o[i] = (char)std::tolower(ch);
    else if (mode == 1) o[i] = (char)std::toupper(ch);
    else if (mode == 2) { o[i] = (char)(start ? std::toupper(ch) : std::tolower(ch)); start = !std::isalpha(ch); }
    else o[i] = (char)(i == 0 ? std::toupper(ch) : std::tolower(ch));
  }
  return o;
}

static Json split_str(const std::string& s, const Val& sep, long long maxsplit) {
  Json out = Json::array();
  if (sep.undef || sep.j.is_null()) {
    size_t i = 0;
    while (i < s.size()) {
      while (i < s.size() && std::isspace((unsigned char)s[i])) ++i;
      if (i >= s.size()) break;
      if (maxsplit >= 0 && (long long)out.size() >= maxsplit) { out.push_back(Json(strip_chars(s.substr(i), "", false, false))); return out; }
      size_t j = i;
      while (j < s.size() && !std::isspace((unsigned char)s[j])) ++j;
      out.push_back(Json(s.substr(i, j - i)));
      i = j;
    }
    return out;
  }
  const std::string& d = sep.j.as_string();
  if (d.empty()) throw Error("empty separator");
  size_t i = 0;
  for (;;) {
    const size_t j = maxsplit >= 0 && (long long)out.size() >= maxsplit ? std::string::npos : s.find(d, i);
    if (j == std::string::npos) { out.push_back(Json(s.substr(i))); break; }
    out.push_back(Json(s.substr(i, j - i)));
    i = j + d.size();
  }
  return out;
}

// ------------------------------------------------------------------------------------------------ interpreter
struct BreakLoop {};
struct ContinueLoop {};

class Interp {
 public:
  explicit Interp(const Json& context) {
    scopes_.emplace_back();
    if (context.is_object()) for (auto& kv : context.members()) scopes_[0][kv.first] = Val(kv.second);
  }
  std::string render(const Body& b) { std::string out; run(b, out); return out; }

 private:
  std::vector<std::map<std::string, Val>> scopes_;
  std::map<std::string, NodeP> macros_;
  int eval_depth_ = 0, macro_depth_ = 0;

  Val lookup(const std::string& name) const {
    for (size_t i = scopes_.size(); i-- > 0;) { auto it = scopes_[i].find(name); if (it != scopes_[i].end()) return it->second; }
    return Val();
  }
  Val* lookup_ref(const std::string& name) {
    for (size_t i = scopes_.size(); i-- > 0;) { auto it = scopes_[i].find(name); if (it != scopes_[i].end()) return &it->second; }
    return nullptr;
  }

  void run(const Body& body, std::string& out) {
    for (auto& n : body) {
      switch (n->kind) {
        case Node::Text: out += n->text; break;
        case Node::Output: out += to_str(eval(n->expr)); break;
        case Node::If:
          for (auto& br : n->branches) if (!br.first || truthy(eval(br.first))) { run(br.second, out); break; }
          break;
        case Node::For: run_for(*n, out); break;
        case Node::Set: {
          Val v = eval(n->expr);
          if (n->attr.empty()) scopes_.back()[n->text] = v;
          else {
            Val* ns = lookup_ref(n->text);
            if (!ns || !ns->j.is_object()) throw Error("cannot set an attribute of " + n->text);
            ns->j.set(n->attr, v.undef ? Json() : v.j);
          }
          break;
        }
        case Node::SetBlock: {
          std::string cap; run(n->body, cap);
          Val v{Json(cap)};
          if (n->expr) { scopes_.emplace_back(); scopes_.back()["__block__"] = v; v = eval(n->expr); scopes_.pop_back(); }
          scopes_.back()[n->text] = v;
          break;
        }
        case Node::Macro: macros_[n->text] = n; break;
        case Node::Break: throw BreakLoop();
        case Node::Continue: throw ContinueLoop();
      }
    }
  }

  static Json iter_items(const Val& v) {
    Json items = Json::array();
    if (v.undef || v.j.is_null()) return items;
    if (v.j.is_array()) return v.j;
    if (v.j.is_object()) { for (auto& kv : v.j.members()) items.push_back(Json(kv.first)); return items; }
    if (v.j.is_string()) {
      const std::string& s = v.j.as_string();
      for (size_t i = 0; i < s.size();) { size_t k = 1; while (i + k < s.size() && ((unsigned char)s[i + k] & 0xC0) == 0x80) ++k; items.push_back(Json(s.substr(i, k))); i += k; }
      return items;
    }
    throw Error("value is not iterable");
  }

  void bind_targets(const std::vector<std::string>& targets, const Json& item) {
    if (targets.size() == 1) { scopes_.back()[targets[0]] = Val(item); return; }
    if (!item.is_array() || item.size() != targets.size()) throw Error("cannot unpack loop item");
    for (size_t i = 0; i < targets.size(); ++i) scopes_.back()[targets[i]] = Val(item[i]);
  }

  void run_for(const Node& n, std::string& out) {
    Json items = iter_items(eval(n.expr));
    if (n.filter) {
      Json kept = Json::array();
      for (auto& it : items.items()) {
        scopes_.emplace_back();
        bind_targets(n.targets, it);
        const bool ok = truthy(eval(n.filter));
        scopes_.pop_back();
        if (ok) kept.push_back(it);
      }
      items = kept;
    }
    const size_t len = items.size();
    if (len == 0) { run(n.else_body, out); return; }
    for (size_t i = 0; i < len; ++i) {
      scopes_.emplace_back();
      bind_targets(n.targets, items[i]);
      Json loop = Json::object();
      loop.set("index", (long long)i + 1); loop.set("index0", (long long)i);
      loop.set("revindex", (long long)(len - i)); loop.set("revindex0", (long long)(len - i - 1));
      loop.set("first", i == 0); loop.set("last", i + 1 == len); loop.set("length", (long long)len);
      if (i > 0) loop.set("previtem", items[i - 1]);
      if (i + 1 < len) loop.set("nextitem", items[i + 1]);
      scopes_.back()["loop"] = Val(loop);
      bool stop = false;
      try { run(n.body, out); } catch (const BreakLoop&) { stop = true; } catch (const ContinueLoop&) {}
      scopes_.pop_back();
      if (stop) break;
    }
  }

  std::vector<Val> eval_args(const Expr& e) { std::vector<Val> v; for (auto& a : e.args) v.push_back(eval(a)); return v; }
  Val kwarg(const Expr& e, const std::string& k) { for (auto& kv : e.kwargs) if (kv.first == k) return eval(kv.second); return Val(); }

  static long long norm_index(long long i, long long n) { return i < 0 ? i + n : i; }

  // A chain of names, attributes and subscripts resolved to the stored value itself, without copying the containers on
  // the way (a template that says messages[i] or message.content inside a loop over the messages would otherwise copy
  // the whole conversation per access: quadratic in its length).  known = false: not such a chain, evaluate normally;
  // known = true and nullptr: the chain resolves to undefined.
  const Json* ref_of(const Expr& e, bool& known) {
    known = true;
    switch (e.kind) {
      case Expr::Name: { Val* v = lookup_ref(e.name); return v && !v->undef ? &v->j : nullptr; }
      case Expr::Attr: {
        const Json* o = ref_of(*e.a, known);
        if (!known || !o) return nullptr;
        return o->is_object() ? o->find(e.name) : nullptr;
      }
      case Expr::Index: {
        Val k = eval(e.b);                                 // first: evaluating the key may run arbitrary expressions
        const Json* o = ref_of(*e.a, known);
        if (!known || !o || k.undef) return nullptr;
        if (o->is_object()) return k.j.is_string() ? o->find(k.j.as_string()) : nullptr;
        if (o->is_array() && k.j.is_int()) { const long long n = (long long)o->size(), i = norm_index(k.j.as_int(), n); return i >= 0 && i < n ? &(*o)[(size_t)i] : nullptr; }
        if (o->is_string()) known = false;                 // characters of a string: the general path
        return nullptr;
      }
      default: known = false; return nullptr;
    }
  }

  Val eval(const ExprP& ep) {
    DepthGuard g(eval_depth_, kMaxEvalDepth, "expression evaluation");
    const Expr& e = *ep;
    switch (e.kind) {
      case Expr::Lit: return Val(e.lit);
      case Expr::Name: return lookup(e.name);
      case Expr::List: { Json a = Json::array(); for (auto& x : e.args) { Val v = eval(x); a.push_back(v.undef ? Json() : v.j); } return Val(a); }
      case Expr::Dict: {
        Json o = Json::object();
        for (size_t i = 0; i + 1 < e.args.size(); i += 2) { Val v = eval(e.args[i + 1]); o.set(to_str(eval(e.args[i])), v.undef ? Json() : v.j); }
        return Val(o);
      }
      case Expr::Not: return Val(Json(!truthy(eval(e.a))));
      case Expr::Neg: { Val v = eval(e.a); if (v.undef || !v.j.is_number()) throw Error("cannot negate this value"); return v.j.is_int() ? Val(Json(-v.j.as_int())) : Val(Json(-v.j.as_double())); }
      case Expr::Cond: if (truthy(eval(e.b))) return eval(e.a); return e.c ? eval(e.c) : Val();
      case Expr::Attr: {
        { bool known; const Json* p = ref_of(e, known); if (known) return p ? Val(*p) : Val(); }
        Val o = eval(e.a);
        if (o.undef) return Val();
        if (o.j.is_object()) { const Json* p = o.j.find(e.name); return p ? Val(*p) : Val(); }
        return Val();
      }
      case Expr::Index: {
        { bool known; const Json* p = ref_of(e, known); if (known) return p ? Val(*p) : Val(); }
        Val o = eval(e.a), k = eval(e.b);
        if (o.undef || k.undef) return Val();
        if (o.j.is_object()) { if (!k.j.is_string()) return Val(); const Json* p = o.j.find(k.j.as_string()); return p ? Val(*p) : Val(); }
        if (o.j.is_array() && k.j.is_int()) { const long long n = (long long)o.j.size(), i = norm_index(k.j.as_int(), n); return i >= 0 && i < n ? Val(o.j[(size_t)i]) : Val(); }
        if (o.j.is_string() && k.j.is_int()) {
          Json chars = iter_items(o);
          const long long n = (long long)chars.size(), i = norm_index(k.j.as_int(), n);
          return i >= 0 && i < n ? Val(chars[(size_t)i]) : Val();
        }
        return Val();
      }
      case Expr::Slice: return eval_slice(e);
      case Expr::Bin: return eval_bin(e);
      case Expr::Filter: {
        if ((e.name == "length" || e.name == "count") && e.args.empty() && e.kwargs.empty()) {     // the size of a stored container
          bool known; const Json* p = ref_of(*e.a, known);
          if (known && p && (p->is_array() || p->is_object())) return Val(Json((long long)p->size()));
        }
        return apply_filter(e.name, eval(e.a), e);
      }
      case Expr::Test: { const bool r = apply_test(e.name, eval(e.a), e); return Val(Json(e.negated ? !r : r)); }
      case Expr::Call: return eval_call(e);
    }
    return Val();
  }

  Val eval_slice(const Expr& e) {
    Val o = eval(e.a);
    if (o.undef) return Val();
    const bool is_str = o.j.is_string();
    Json seq = is_str ? iter_items(o) : o.j;
    if (!seq.is_array()) throw Error("value cannot be sliced");
    const long long n = (long long)seq.size();
    auto opt = [&](const ExprP& x, bool& has) -> long long { has = false; if (!x) return 0; Val v = eval(x); if (v.undef || v.j.is_null()) return 0; has = true; return v.j.as_int(); };
    bool hs, he, hst;
    long long start = opt(e.b, hs), stop = opt(e.c, he), step = opt(e.d, hst);
    if (!hst) step = 1;
    if (step == 0) throw Error("slice step cannot be zero");
    auto clamp = [&](long long v, long long lo, long long hi) { return v < lo ? lo : v > hi ? hi : v; };
    if (step > 0) { start = hs ? clamp(norm_index(start, n), 0, n) : 0; stop = he ? clamp(norm_index(stop, n), 0, n) : n; }
    else { start = hs ? clamp(norm_index(start, n), -1, n - 1) : n - 1; stop = he ? clamp(norm_index(stop, n), -1, n - 1) : -1; }
    Json out = Json::array();
    for (long long i = start; step > 0 ? i < stop : i > stop; i += step) out.push_back(seq[(size_t)i]);
    if (!is_str) return Val(out);
    std::string s; for (auto& ch : out.items()) s += ch.as_string();
    return Val(Json(s));
  }

  Val eval_bin(const Expr& e) {
    const std::string& op = e.name;
    if (op == "and") { Val a = eval(e.a); return truthy(a) ? eval(e.b) : a; }
    if (op == "or") { Val a = eval(e.a); return truthy(a) ? a : eval(e.b); }
    Val a = eval(e.a), b = eval(e.b);
    if (op == "~") return Val(Json(to_str(a) + to_str(b)));
    if (op == "==") return Val(Json(val_equal(a, b)));
    if (op == "!=") return Val(Json(!val_equal(a, b)));
    if (op == "in") {
      if (b.undef || a.undef) return Val(Json(false));
      if (b.j.is_string()) return Val(Json(a.j.is_string() && b.j.as_string().find(a.j.as_string()) != std::string::npos));
      if (b.j.is_array()) { for (auto& x : b.j.items()) if (json_equal(x, a.j)) return Val(Json(true)); return Val(Json(false)); }
      if (b.j.is_object()) return Val(Json(a.j.is_string() && b.j.contains(a.j.as_string())));
      return Val(Json(false));
    }
    if (a.undef || b.undef) throw Error("operation on an undefined value");
    if (op == "<" || op == ">" || op == "<=" || op == ">=") {
      const int c = json_compare(a.j, b.j);
      return Val(Json(op == "<" ? c < 0 : op == ">" ? c > 0 : op == "<=" ? c <= 0 : c >= 0));
    }
    if (op == "+") {
      if (a.j.is_string() && b.j.is_string()) return Val(Json(a.j.as_string() + b.j.as_string()));
      if (a.j.is_array() && b.j.is_array()) { Json o = a.j; for (auto& x : b.j.items()) o.push_back(x); return Val(o); }
    }
    if (op == "*" && a.j.is_string() && b.j.is_int()) { std::string s; for (long long i = 0; i < b.j.as_int(); ++i) s += a.j.as_string(); return Val(Json(s)); }
    if (op == "%" && a.j.is_string()) throw Error("string formatting with % is not supported");
    auto num = [](const Json& j) { return j.is_bool() ? Json((long long)j.as_bool()) : j; };
    const Json x = num(a.j), y = num(b.j);
    if (!x.is_number() || !y.is_number()) throw Error("unsupported operand types for " + op);
    const bool ints = x.is_int() && y.is_int();
    if (op == "+") return ints ? Val(Json(x.as_int() + y.as_int())) : Val(Json(x.as_double() + y.as_double()));
    if (op == "-") return ints ? Val(Json(x.as_int() - y.as_int())) : Val(Json(x.as_double() - y.as_double()));
    if (op == "*") return ints ? Val(Json(x.as_int() * y.as_int())) : Val(Json(x.as_double() * y.as_double()));
    if (op == "/") { if (y.as_double() == 0) throw Error("division by zero"); return Val(Json(x.as_double() / y.as_double())); }
    if (op == "//") {
      if (y.as_double() == 0) throw Error("division by zero");
      if (ints) { long long q = x.as_int() / y.as_int(); if ((x.as_int() % y.as_int() != 0) && ((x.as_int() < 0) != (y.as_int() < 0))) --q; return Val(Json(q)); }
      return Val(Json(std::floor(x.as_double() / y.as_double())));
    }
    if (op == "%") {
      if (y.as_double() == 0) throw Error("division by zero");
      if (ints) { long long r = x.as_int() % y.as_int(); if (r != 0 && ((r < 0) != (y.as_int() < 0))) r += y.as_int(); return Val(Json(r)); }
      const double r = std::fmod(x.as_double(), y.as_double());
      return Val(Json(r != 0 && ((r < 0) != (y.as_double() < 0)) ? r + y.as_double() : r));
    }
    throw Error("unsupported operator " + op);
  }

  bool apply_test(const std::string& name, const Val& v, const Expr& e) {
    if (name == "defined") return !v.undef;
    if (name == "undefined") return v.undef;
    if (name == "none") return !v.undef && v.j.is_null();
    if (name == "string") return !v.undef && v.j.is_string();
    if (name == "mapping") return !v.undef && v.j.is_object();
    if (name == "number") return !v.undef && v.j.is_number();
    if (name == "integer") return !v.undef && v.j.is_int();
    if (name == "float") return !v.undef && v.j.type() == Json::Double;
    if (name == "boolean") return !v.undef && v.j.is_bool();
    if (name == "true") return !v.undef && v.j.is_bool() && v.j.as_bool();
    if (name == "false") return !v.undef && v.j.is_bool() && !v.j.as_bool();
    if (name == "iterable") return !v.undef && (v.j.is_array() || v.j.is_object() || v.j.is_string());
    if (name == "sequence") return !v.undef && (v.j.is_array() || v.j.is_object() || v.j.is_string());
    if (name == "odd") return !v.undef && v.j.is_int() && (v.j.as_int() % 2 != 0);
    if (name == "even") return !v.undef && v.j.is_int() && (v.j.as_int() % 2 == 0);
    std::vector<Val> a = eval_args(e);
    if (name == "equalto" || name == "eq" || name == "sameas") return !a.empty() && val_equal(v, a[0]);
    if (name == "ne") return !a.empty() && !val_equal(v, a[0]);
    if (name == "in") return !a.empty() && !v.undef && a[0].j.is_array() && [&] { for (auto& x : a[0].j.items()) if (json_equal(x, v.j)) return true; return false; }();
    if (name == "gt" || name == "ge" || name == "lt" || name == "le") {
      if (a.empty() || v.undef || a[0].undef) return false;
      const int c = json_compare(v.j, a[0].j);
      return name == "gt" ? c > 0 : name == "ge" ? c >= 0 : name == "lt" ? c < 0 : c <= 0;
    }
    throw Error("unknown test: " + name);
  }

  // selectattr / rejectattr / select / reject share the "test by name" machinery
  bool test_by_name(const Val& v, const std::vector<Val>& a, size_t first) {
    if (a.size() <= first) return truthy(v);
    Expr fake; fake.kind = Expr::Test;
    for (size_t i = first + 1; i < a.size(); ++i) { auto l = std::make_shared<Expr>(); l->kind = Expr::Lit; l->lit = a[i].undef ? Json() : a[i].j; fake.args.push_back(l); }
    return apply_test(a[first].j.as_string(), v, fake);
  }
  static Val attr_path(const Val& v, const std::string& path) {
    Val cur = v;
    size_t i = 0;
    while (i <= path.size()) {
      size_t j = path.find('.', i);
      if (j == std::string::npos) j = path.size();
      const std::string part = path.substr(i, j - i);
      if (cur.undef || !cur.j.is_object()) return Val();
      const Json* p = cur.j.find(part);
      cur = p ? Val(*p) : Val();
      i = j + 1;
    }
    return cur;
  }

  Val apply_filter(const std::string& name, const Val& v, const Expr& e) {
    std::vector<Val> a = eval_args(e);
    auto str = [&]() { return to_str(v); };
    Json seq_;                                              // keeps the iterated sequence alive for the loops below
    auto seq = [&]() -> const Json::Arr& { seq_ = iter_items(v); return seq_.items(); };
    if (name == "default" || name == "d") {
      const bool boolean = (a.size() > 1 && truthy(a[1])) || truthy(kwarg(e, "boolean"));
      if (v.undef || (boolean && !truthy(v))) return a.empty() ? Val(Json("")) : a[0];
      return v;
    }
    if (name == "tojson") {
      Val ind = a.empty() ? kwarg(e, "indent") : a[0];
      const Json j = v.undef ? Json() : v.j;
      if (!ind.undef && ind.j.is_int()) { std::string out; dump_indented(j, (int)ind.j.as_int(), 0, out); return Val(Json(out)); }
      return Val(Json(j.dump(Json::Style{true, false})));
    }
    if (name == "trim") return Val(Json(strip_chars(str(), a.empty() ? "" : to_str(a[0]), true, true)));
    if (name == "length" || name == "count") { if (v.undef) throw Error("length of an undefined value"); return Val(Json((long long)(v.j.is_string() ? utf8_len(v.j.as_string()) : v.j.size()))); }
    if (name == "string") return Val(Json(str()));
    if (name == "safe" || name == "e" || name == "escape") return v;
    if (name == "upper") return Val(Json(case_map(str(), 1)));
    if (name == "lower") return Val(Json(case_map(str(), 0)));
    if (name == "title") return Val(Json(case_map(str(), 2)));
    if (name == "capitalize") return Val(Json(case_map(str(), 3)));
    if (name == "int") {
      if (!v.undef && v.j.is_number()) return Val(Json(v.j.as_int()));
      if (!v.undef && v.j.is_bool()) return Val(Json((long long)v.j.as_bool()));
      try { size_t p = 0; const std::string s = strip_chars(str(), "", true, true); long long r = std::stoll(s, &p); if (p == s.size()) return Val(Json(r)); } catch (...) {}
      return a.empty() ? Val(Json(0)) : a[0];
    }
    if (name == "float") { try { return Val(Json(v.j.is_number() ? v.j.as_double() : std::stod(str()))); } catch (...) { return Val(Json(0.0)); } }
    if (name == "abs") { if (v.j.is_int()) return Val(Json(std::llabs(v.j.as_int()))); return Val(Json(std::fabs(v.j.as_double()))); }
    if (name == "list") return Val(iter_items(v));
    if (name == "items") {
      Json out = Json::array();
      if (!v.undef && v.j.is_object()) for (auto& kv : v.j.members()) { Json p = Json::array(); p.push_back(Json(kv.first)); p.push_back(kv.second); out.push_back(p); }
      return Val(out);
    }
    if (name == "first") { Json it = iter_items(v); return it.size() ? Val(it[0]) : Val(); }
    if (name == "last") { Json it = iter_items(v); return it.size() ? Val(it[it.size() - 1]) : Val(); }
    if (name == "reverse") {
      if (v.j.is_string()) { Json it = iter_items(v); std::string s; for (size_t i = it.size(); i-- > 0;) s += it[i].as_string(); return Val(Json(s)); }
      Json it = iter_items(v), out = Json::array();
      for (size_t i = it.size(); i-- > 0;) out.push_back(it[i]);
      return Val(out);
    }
    if (name == "join") {
      const std::string sep = a.empty() ? to_str(kwarg(e, "d")) : to_str(a[0]);
      Val attr = kwarg(e, "attribute");
      Json it = iter_items(v);
      std::string out;
      for (size_t i = 0; i < it.size(); ++i) { if (i) out += sep; out += attr.undef ? py_str(it[i]) : to_str(attr_path(Val(it[i]), to_str(attr))); }
      return Val(Json(out));
    }
    if (name == "replace") { if (a.size() < 2) throw Error("replace needs two arguments"); return Val(Json(replace_all(str(), to_str(a[0]), to_str(a[1])))); }
    if (name == "selectattr" || name == "rejectattr") {
      if (a.empty()) throw Error(name + " needs an attribute name");
      Json out = Json::array();
      for (auto& it : seq()) if (test_by_name(attr_path(Val(it), to_str(a[0])), a, 1) == (name == "selectattr")) out.push_back(it);
      return Val(out);
    }
    if (name == "select" || name == "reject") {
      Json out = Json::array();
      for (auto& it : seq()) if (test_by_name(Val(it), a, 0) == (name == "select")) out.push_back(it);
      return Val(out);
    }
    if (name == "map") {
      Val attr = kwarg(e, "attribute");
      Json out = Json::array();
      for (auto& it : seq()) {
        if (!attr.undef) { Val r = attr_path(Val(it), to_str(attr)); out.push_back(r.undef ? (kwarg(e, "default").undef ? Json() : kwarg(e, "default").j) : r.j); }
        else if (!a.empty()) { Expr fake; fake.kind = Expr::Filter; Val r = apply_filter(to_str(a[0]), Val(it), fake); out.push_back(r.undef ? Json() : r.j); }
        else out.push_back(it);
      }
      return Val(out);
    }
    if (name == "unique") { Json out = Json::array(); for (auto& it : seq()) { bool seen = false; for (auto& o : out.items()) if (json_equal(o, it)) seen = true; if (!seen) out.push_back(it); } return Val(out); }
    if (name == "sum") { double s = 0; bool ints = true; for (auto& it : seq()) { s += it.as_double(); ints = ints && it.is_int(); } return ints ? Val(Json((long long)s)) : Val(Json(s)); }
    if (name == "indent") {
      const long long w = a.empty() ? 4 : a[0].j.as_int();
      const bool first = (a.size() > 1 && truthy(a[1])) || truthy(kwarg(e, "first"));
      const std::string pad((size_t)w, ' '), s = str();
      std::string out = first ? pad : "";
      for (size_t i = 0; i < s.size(); ++i) { out.push_back(s[i]); if (s[i] == '\n' && i + 1 < s.size() && s[i + 1] != '\n') out += pad; }
      return Val(Json(out));
    }
    throw Error("unknown filter: " + name);
  }

  static std::string replace_all(std::string s, const std::string& from, const std::string& to) {
    if (from.empty()) return s;
    for (size_t p = 0; (p = s.find(from, p)) != std::string::npos; p += to.size()) s.replace(p, from.size(), to);
    return s;
  }

  Val eval_call(const Expr& e) {
    const Expr& callee = *e.a;
    if (callee.kind == Expr::Attr) {                         // method call
      Val o = eval(callee.a);
      const std::string& m = callee.name;
      std::vector<Val> a = eval_args(e);
      if (!o.undef && o.j.is_string()) {
        const std::string& s = o.j.as_string();
        auto arg = [&](size_t i) { return i < a.size() ? to_str(a[i]) : std::string(); };
        auto any_prefix = [&](bool suffix) {
          std::vector<std::string> opts;
          if (!a.empty() && a[0].j.is_array()) for (auto& x : a[0].j.items()) opts.push_back(x.as_string()); else opts.push_back(arg(0));
          for (auto& p : opts) if (p.size() <= s.size() && s.compare(suffix ? s.size() - p.size() : 0, p.size(), p) == 0) return true;
          return false;
        };
        if (m == "startswith") return Val(Json(any_prefix(false)));
        if (m == "endswith") return Val(Json(any_prefix(true)));
        if (m == "strip") return Val(Json(strip_chars(s, arg(0), true, true)));
        if (m == "lstrip") return Val(Json(strip_chars(s, arg(0), true, false)));
        if (m == "rstrip") return Val(Json(strip_chars(s, arg(0), false, true)));
        if (m == "upper") return Val(Json(case_map(s, 1)));
        if (m == "lower") return Val(Json(case_map(s, 0)));
        if (m == "title") return Val(Json(case_map(s, 2)));
        if (m == "capitalize") return Val(Json(case_map(s, 3)));
        if (m == "replace") return Val(Json(replace_all(s, arg(0), arg(1))));
        if (m == "split") return Val(split_str(s, a.empty() ? Val() : a[0], a.size() > 1 ? a[1].j.as_int() : -1));
        if (m == "find") { const size_t p = s.find(arg(0)); return Val(Json(p == std::string::npos ? -1LL : (long long)utf8_len(s.substr(0, p)))); }
        if (m == "count") { long long c = 0; const std::string n = arg(0); if (!n.empty()) for (size_t p = 0; (p = s.find(n, p)) != std::string::npos; p += n.size()) ++c; return Val(Json(c)); }
        if (m == "join") { Json it = a.empty() ? Json::array() : iter_items(a[0]); std::string out; for (size_t i = 0; i < it.size(); ++i) { if (i) out += s; out += py_str(it[i]); } return Val(Json(out)); }
        throw Error("unknown string method: " + m);
      }
      if (!o.undef && o.j.is_object()) {
        if (const Json* member = o.j.find(m); member == nullptr || a.empty()) {
          if (m == "items") { Expr fake; fake.kind = Expr::Filter; return apply_filter("items", o, fake); }
          if (m == "keys") { Json out = Json::array(); for (auto& kv : o.j.members()) out.push_back(Json(kv.first)); return Val(out); }
          if (m == "values") { Json out = Json::array(); for (auto& kv : o.j.members()) out.push_back(kv.second); return Val(out); }
        }
        if (m == "get") { if (a.empty()) throw Error("get needs a key"); const Json* p = a[0].j.is_string() ? o.j.find(a[0].j.as_string()) : nullptr; return p ? Val(*p) : (a.size() > 1 ? a[1] : Val(Json())); }
      }
      if (!o.undef && o.j.is_array()) {
        if (m == "index" && !a.empty()) { for (size_t i = 0; i < o.j.size(); ++i) if (json_equal(o.j[i], a[0].j)) return Val(Json((long long)i)); throw Error("value is not in the list"); }
        if (m == "count" && !a.empty()) { long long c = 0; for (auto& x : o.j.items()) if (json_equal(x, a[0].j)) ++c; return Val(Json(c)); }
      }
      throw Error("cannot call ." + m + "() on this value");
    }
    if (callee.kind != Expr::Name) throw Error("this expression cannot be called");
    const std::string& fn = callee.name;
    if (auto it = macros_.find(fn); it != macros_.end()) {
      const Node& mc = *it->second;
      DepthGuard g(macro_depth_, kMaxMacroDepth, "macro calls");
      std::vector<Val> a = eval_args(e);
      std::map<std::string, Val> frame;
      for (size_t i = 0; i < mc.params.size(); ++i) {
        Val v = i < a.size() ? a[i] : kwarg(e, mc.params[i].first);
        if (v.undef && i >= a.size() && mc.params[i].second) v = eval(mc.params[i].second);
        frame[mc.params[i].first] = v;
      }
      scopes_.push_back(std::move(frame));
      std::string out;
      try { run(mc.body, out); } catch (...) { scopes_.pop_back(); throw; }
      scopes_.pop_back();
      return Val(Json(out));
    }
    if (fn == "raise_exception") { std::vector<Val> a = eval_args(e); throw Error(a.empty() ? "template error" : to_str(a[0])); }
    if (fn == "namespace" || fn == "dict") {
      Json o = Json::object();
      for (auto& kv : e.kwargs) { Val v = eval(kv.second); o.set(kv.first, v.undef ? Json() : v.j); }
      return Val(o);
    }
    if (fn == "range") {
      std::vector<Val> a = eval_args(e);
      long long lo = 0, hi = 0, st = 1;
      if (a.size() == 1) hi = a[0].j.as_int();
      else if (a.size() >= 2) { lo = a[0].j.as_int(); hi = a[1].j.as_int(); if (a.size() > 2) st = a[2].j.as_int(); }
      if (st == 0) throw Error("range step cannot be zero");
      Json out = Json::array();
      for (long long i = lo; st > 0 ? i < hi : i > hi; i += st) { out.push_back(Json(i)); if (out.size() > 1000000) throw Error("range is too long"); }
      return Val(out);
    }
    if (fn == "strftime_now") { std::vector<Val> a = eval_args(e); char buf[128]; time_t t = time(nullptr); struct tm tmv; localtime_r(&t, &tmv); strftime(buf, sizeof buf, a.empty() ? "%Y-%m-%d" : to_str(a[0]).c_str(), &tmv); return Val(Json(std::string(buf))); }
    throw Error("unknown function: " + fn);
  }
};

}  // namespace jinja

// Renders `source` with the variables of `context` (a JSON object).  Throws std::runtime_error with the template's
// own message for raise_exception, or a description of what the subset does not cover.
std::string render_jinja(const std::string& source, const Json& context) {
  // as in the Python renderer, one trailing newline of the source does not belong to the template
  const std::string src = !source.empty() && source.back() == '\n' ? source.substr(0, source.size() - 1) : source;
  jinja::Body body = jinja::TemplateParser(jinja::split_template(src)).parse();
  return jinja::Interp(context).render(body);
}

}  // namespace b2
