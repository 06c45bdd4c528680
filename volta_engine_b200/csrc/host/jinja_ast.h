// Jinja2 subset interpreter for chat templates: expressions, filters, tests, if / for / set / macro,
// namespace(), whitespace control, loop variables. Covers what the Qwen, GLM, DeepSeek, Gemma and Llama
// chat templates use. Counterpart of the reference's own interpreter (src/loader/jinja.cpp,
// src/loader/chat_template.cpp); values are JSON values with insertion-ordered objects.
#include <cctype>
#include <cmath>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "json.h"

namespace vh {
namespace jinja {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// Undefined is a Null with b == true.
static Json undefined() { Json j; j.b = true; return j; }
static bool is_undefined(const Json& j) { return j.type == Json::Null && j.b; }

static bool truthy(const Json& v) {
  switch (v.type) {
    case Json::Null: return false;
    case Json::Bool: return v.b;
    case Json::Int: return v.i != 0;
    case Json::Float: return v.f != 0.0;
    case Json::String: return !v.s.empty();
    case Json::Array: return !v.arr.empty();
    case Json::Object: return !v.obj.empty();
  }
  return false;
}

static std::string to_str(const Json& v) {
  switch (v.type) {
    case Json::Null: return is_undefined(v) ? "" : "None";
    case Json::Bool: return v.b ? "True" : "False";
    case Json::Int: return std::to_string(v.i);
    case Json::Float: { std::string o; json_dump(v, o); return o; }
    case Json::String: return v.s;
    default: {
      // python-like repr of containers
      std::string o;
      if (v.type == Json::Array) {
        o = "[";
        for (size_t n = 0; n < v.arr.size(); ++n) {
          if (n) o += ", ";
          o += v.arr[n].type == Json::String ? "'" + v.arr[n].s + "'" : to_str(v.arr[n]);
        }
        return o + "]";
      }
      o = "{";
      for (size_t n = 0; n < v.obj.size(); ++n) {
        if (n) o += ", ";
        o += "'" + v.obj[n].first + "': ";
        o += v.obj[n].second.type == Json::String ? "'" + v.obj[n].second.s + "'" : to_str(v.obj[n].second);
      }
      return o + "}";
    }
  }
}

static bool equals(const Json& a, const Json& b) {
  if (a.is_number() && b.is_number()) return a.as_double() == b.as_double();
  if (a.type != b.type) return false;
  switch (a.type) {
    case Json::Null: return true;
    case Json::Bool: return a.b == b.b;
    case Json::String: return a.s == b.s;
    case Json::Array:
      if (a.arr.size() != b.arr.size()) return false;
      for (size_t n = 0; n < a.arr.size(); ++n) if (!equals(a.arr[n], b.arr[n])) return false;
      return true;
    case Json::Object:
      if (a.obj.size() != b.obj.size()) return false;
      for (auto& kv : a.obj) {
        const Json* o = b.find(kv.first);
        if (!o || !equals(kv.second, *o)) return false;
      }
      return true;
    default: return false;
  }
}

// ------------------------------------------------------------------------------------------------ lexer
enum TokType { T_END, T_NAME, T_STR, T_INT, T_FLOAT, T_OP };
struct Tok {
  TokType t;
  std::string s;
};

static std::vector<Tok> lex_expr(const std::string& src) {
  std::vector<Tok> out;
  size_t i = 0, n = src.size();
  while (i < n) {
    char c = src[i];
    if (isspace((unsigned char)c)) { ++i; continue; }
    if (isalpha((unsigned char)c) || c == '_') {
      size_t j = i;
      while (j < n && (isalnum((unsigned char)src[j]) || src[j] == '_')) ++j;
      out.push_back({T_NAME, src.substr(i, j - i)});
      i = j;
      continue;
    }
    if (isdigit((unsigned char)c)) {
      size_t j = i;
      bool f = false;
      while (j < n && (isdigit((unsigned char)src[j]) || (src[j] == '.' && j + 1 < n && isdigit((unsigned char)src[j + 1])))) {
        if (src[j] == '.') f = true;
        ++j;
      }
      out.push_back({f ? T_FLOAT : T_INT, src.substr(i, j - i)});
      i = j;
      continue;
    }
    if (c == '"' || c == '\'') {
      std::string s;
      size_t j = i + 1;
      while (j < n && src[j] != c) {
        if (src[j] == '\\' && j + 1 < n) {
          char e = src[j + 1];
          s.push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e == 'r' ? '\r' : e);
          j += 2;
        } else {
          s.push_back(src[j++]);
        }
      }
      if (j >= n) throw Error("unterminated string literal");
      out.push_back({T_STR, s});
      i = j + 1;
      continue;
    }
    static const char* ops2[] = {"==", "!=", "<=", ">=", "//", "**"};
    bool hit = false;
    for (auto o : ops2)
      if (i + 1 < n && src[i] == o[0] && src[i + 1] == o[1]) { out.push_back({T_OP, o}); i += 2; hit = true; break; }
    if (hit) continue;
    out.push_back({T_OP, std::string(1, c)});
    ++i;
  }
  out.push_back({T_END, ""});
  return out;
}

// ------------------------------------------------------------------------------------------------ AST
struct Expr;
using ExprP = std::shared_ptr<Expr>;
struct Expr {
  enum Kind { Lit, Var, Attr, Index, Slice, Call, Filter, Test, Unary, Binary, Cond, List, Dict } kind;
  Json lit;
  std::string name;                       // Var, Attr, Filter/Test name, operator
  ExprP a, b, c;                          // operands
  std::vector<ExprP> args;
  std::vector<std::pair<std::string, ExprP>> kwargs;
  std::vector<std::pair<ExprP, ExprP>> items;  // Dict
  bool negate = false;                    // "is not"
};

class ExprParser {
 public:
  explicit ExprParser(std::vector<Tok> toks) : t_(std::move(toks)) {}
  ExprP parse_full() {
    ExprP e = ternary();
    if (cur().t != T_END) throw Error("unexpected token '" + cur().s + "' in expression");
    return e;
  }
  ExprP ternary() {
    ExprP v = or_();
    if (is_name("if")) {
      ++p_;
      ExprP cnd = or_();
      ExprP els;
      if (is_name("else")) { ++p_; els = ternary(); }
      auto e = mk(Expr::Cond);
      e->a = cnd; e->b = v; e->c = els;
      return e;
    }
    return v;
  }
  bool at_end() const { return t_[p_].t == T_END; }
  const Tok& cur() const { return t_[p_]; }
  bool is_op(const char* s) const { return t_[p_].t == T_OP && t_[p_].s == s; }
  bool is_name(const char* s) const { return t_[p_].t == T_NAME && t_[p_].s == s; }
  void expect_op(const char* s) {
    if (!is_op(s)) throw Error(std::string("expected '") + s + "' but found '" + cur().s + "'");
    ++p_;
  }
  std::string expect_name() {
    if (cur().t != T_NAME) throw Error("expected a name, found '" + cur().s + "'");
    return t_[p_++].s;
  }
  size_t p_ = 0;

 private:
  std::vector<Tok> t_;
  static ExprP mk(Expr::Kind k) { auto e = std::make_shared<Expr>(); e->kind = k; return e; }
  ExprP bin(const std::string& op, ExprP l, ExprP r) { auto e = mk(Expr::Binary); e->name = op; e->a = l; e->b = r; return e; }
  ExprP or_() {
    ExprP l = and_();
    while (is_name("or")) { ++p_; l = bin("or", l, and_()); }
    return l;
  }
  ExprP and_() {
    ExprP l = not_();
    while (is_name("and")) { ++p_; l = bin("and", l, not_()); }
    return l;
  }
  ExprP not_() {
    if (is_name("not")) { ++p_; auto e = mk(Expr::Unary); e->name = "not"; e->a = not_(); return e; }
    return cmp();
  }
  ExprP cmp() {
    ExprP l = add();
    for (;;) {
      if (cur().t == T_OP && (cur().s == "==" || cur().s == "!=" || cur().s == "<" || cur().s == ">" || cur().s == "<=" || cur().s == ">=")) {
        std::string op = t_[p_++].s;
        l = bin(op, l, add());
      } else if (is_name("in")) {
        ++p_;
        l = bin("in", l, add());
      } else if (is_name("not") && t_[p_ + 1].t == T_NAME && t_[p_ + 1].s == "in") {
        p_ += 2;
        auto e = mk(Expr::Unary); e->name = "not"; e->a = bin("in", l, add());
        l = e;
      } else if (is_name("is")) {
        ++p_;
        auto e = mk(Expr::Test);
        if (is_name("not")) { ++p_; e->negate = true; }
        e->name = expect_name();
        e->a = l;
        if (is_op("(")) { ++p_; while (!is_op(")")) { e->args.push_back(ternary()); if (is_op(",")) ++p_; } ++p_; }
        else if (cur().t == T_STR || cur().t == T_INT || (cur().t == T_NAME && !is_name("and") && !is_name("or") && !is_name("else") && !is_name("if")))
          e->args.push_back(unary());
        l = e;
      } else {
        return l;
      }
    }
  }
  ExprP add() {
    ExprP l = mul();
    while (is_op("+") || is_op("-") || is_op("~")) { std::string op = t_[p_++].s; l = bin(op, l, mul()); }
    return l;
  }
  ExprP mul() {
    ExprP l = unary();
    while (is_op("*") || is_op("/") || is_op("//") || is_op("%")) { std::string op = t_[p_++].s; l = bin(op, l, unary()); }
    return l;
  }
  ExprP unary() {
    if (is_op("-")) { ++p_; auto e = mk(Expr::Unary); e->name = "-"; e->a = unary(); return e; }
    if (is_op("+")) { ++p_; return unary(); }
    return postfix(primary());
  }
  void call_args(Expr& e) {
    // after '('
    while (!is_op(")")) {
      if (cur().t == T_NAME && t_[p_ + 1].t == T_OP && t_[p_ + 1].s == "=") {
        std::string k = t_[p_].s;
        p_ += 2;
        e.kwargs.emplace_back(k, ternary());
      } else {
        e.args.push_back(ternary());
      }
      if (is_op(",")) ++p_;
      else if (!is_op(")")) throw Error("expected ',' or ')' in call");
    }
    ++p_;
  }
  ExprP postfix(ExprP e) {
    for (;;) {
      if (is_op(".")) {
        ++p_;
        auto n = mk(Expr::Attr);
        n->a = e;
        n->name = cur().t == T_INT ? t_[p_++].s : expect_name();
        e = n;
      } else if (is_op("[")) {
        ++p_;
        ExprP lo, hi, st;
        bool slice = false;
        if (!is_op(":")) lo = ternary();
        if (is_op(":")) {
          slice = true;
          ++p_;
          if (!is_op("]") && !is_op(":")) hi = ternary();
          if (is_op(":")) { ++p_; if (!is_op("]")) st = ternary(); }
        }
        expect_op("]");
        auto n = mk(slice ? Expr::Slice : Expr::Index);
        n->a = e;
        if (slice) { n->args = {lo, hi, st}; } else { n->b = lo; }
        e = n;
      } else if (is_op("(")) {
        ++p_;
        auto n = mk(Expr::Call);
        n->a = e;
        call_args(*n);
        e = n;
      } else if (is_op("|")) {
        ++p_;
        auto n = mk(Expr::Filter);
        n->a = e;
        n->name = expect_name();
        if (is_op("(")) { ++p_; call_args(*n); }
        e = n;
      } else {
        return e;
      }
    }
  }
  ExprP primary() {
    const Tok& t = cur();
    if (t.t == T_STR) { ++p_; auto e = mk(Expr::Lit); e->lit = Json::string(t.s);
      while (cur().t == T_STR) { e->lit.s += cur().s; ++p_; }
      return e; }
    if (t.t == T_INT) { ++p_; auto e = mk(Expr::Lit); e->lit = Json::integer(strtoll(t.s.c_str(), nullptr, 10)); return e; }
    if (t.t == T_FLOAT) { ++p_; auto e = mk(Expr::Lit); e->lit = Json::number(strtod(t.s.c_str(), nullptr)); return e; }
    if (t.t == T_NAME) {
      ++p_;
      auto lit = [&](Json v) { auto e = mk(Expr::Lit); e->lit = std::move(v); return e; };
      if (t.s == "true" || t.s == "True") return lit(Json::boolean(true));
      if (t.s == "false" || t.s == "False") return lit(Json::boolean(false));
      if (t.s == "none" || t.s == "None") return lit(Json::null());
      auto e = mk(Expr::Var);
      e->name = t.s;
      return e;
    }
    if (is_op("(")) {
      ++p_;
      ExprP e = ternary();
      if (is_op(",")) {  // tuple -> list
        auto l = mk(Expr::List);
        l->args.push_back(e);
        while (is_op(",")) { ++p_; if (is_op(")")) break; l->args.push_back(ternary()); }
        e = l;
      }
      expect_op(")");
      return e;
    }
    if (is_op("[")) {
      ++p_;
      auto l = mk(Expr::List);
      while (!is_op("]")) { l->args.push_back(ternary()); if (is_op(",")) ++p_; else if (!is_op("]")) throw Error("bad list literal"); }
      ++p_;
      return l;
    }
    if (is_op("{")) {
      ++p_;
      auto d = mk(Expr::Dict);
      while (!is_op("}")) {
        ExprP k = ternary();
        expect_op(":");
        d->items.emplace_back(k, ternary());
        if (is_op(",")) ++p_; else if (!is_op("}")) throw Error("bad dict literal");
      }
      ++p_;
      return d;
    }
    throw Error("unexpected token '" + t.s + "'");
  }
};

// ------------------------------------------------------------------------------------------------ template tree
struct Node;
using NodeP = std::shared_ptr<Node>;
struct Node {
  enum Kind { Text, Output, If, For, Set, SetBlock, Macro, Block } kind = Text;
  std::string text;                                   // Text; Set target; Macro name
  std::string attr;                                   // Set: ns.attr target
  ExprP expr;                                         // Output, Set value, For iterable
  ExprP cond;                                         // For filter
  std::vector<std::pair<ExprP, std::vector<NodeP>>> branches;   // If (null expr = else)
  std::vector<std::string> vars;                      // For loop variables; Macro parameters
  std::vector<ExprP> defaults;                        // Macro defaults (aligned to the tail of vars)
  std::vector<NodeP> body, else_body;
};

struct Piece {
  int kind;  // 0 text, 1 {{ }}, 2 {% %}
  std::string s;
};

static std::vector<Piece> split_template(const std::string& src, bool trim_blocks, bool lstrip_blocks) {
  std::vector<Piece> out;
  size_t i = 0, n = src.size();
  bool strip_next = false;
  auto add_text = [&](std::string t, bool rstrip, bool lstrip_tag) {
    if (strip_next) {
      size_t k = 0;
      while (k < t.size() && isspace((unsigned char)t[k])) ++k;
      t.erase(0, k);
    }
    if (rstrip) {
      while (!t.empty() && isspace((unsigned char)t.back())) t.pop_back();
    } else if (lstrip_tag) {
      size_t k = t.size();
      while (k > 0 && (t[k - 1] == ' ' || t[k - 1] == '\t')) --k;
      if (k == 0 || t[k - 1] == '\n') t.erase(k);
    }
    if (!t.empty()) out.push_back({0, t});
  };
  while (i < n) {
    size_t a = src.find('{', i);
    while (a != std::string::npos && !(a + 1 < n && (src[a + 1] == '{' || src[a + 1] == '%' || src[a + 1] == '#'))) a = src.find('{', a + 1);
    if (a == std::string::npos) { add_text(src.substr(i), false, false); strip_next = false; break; }
    char kind = src[a + 1];
    const char* close = kind == '{' ? "}}" : kind == '%' ? "%}" : "#}";
    size_t b = src.find(close, a + 2);
    if (b == std::string::npos) throw Error("unclosed template tag");
    bool lminus = a + 2 < n && src[a + 2] == '-';
    bool rminus = b > 0 && src[b - 1] == '-';
    add_text(src.substr(i, a - i), lminus, lstrip_blocks && kind != '{' && !lminus);
    strip_next = false;
    size_t s0 = a + 2 + (lminus ? 1 : 0), s1 = b - (rminus ? 1 : 0);
    std::string inner = s1 > s0 ? src.substr(s0, s1 - s0) : "";
    if (kind == '{') out.push_back({1, inner});
    else if (kind == '%') out.push_back({2, inner});
    i = b + 2;
    if (rminus) strip_next = true;
    else if (trim_blocks && kind != '{' && i < n && src[i] == '\n') ++i;
  }
  return out;
}

static std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && isspace((unsigned char)s[a])) ++a;
  while (b > a && isspace((unsigned char)s[b - 1])) --b;
  return s.substr(a, b - a);
}

class TemplateParser {
 public:
  explicit TemplateParser(std::vector<Piece> p) : p_(std::move(p)) {}
  std::vector<NodeP> parse() {
    std::string end;
    auto body = block({}, end);
    return body;
  }

 private:
  std::vector<Piece> p_;
  size_t i_ = 0;
  static std::string first_word(const std::string& s) {
    size_t a = 0;
    while (a < s.size() && isspace((unsigned char)s[a])) ++a;
    size_t b = a;
    while (b < s.size() && (isalnum((unsigned char)s[b]) || s[b] == '_')) ++b;
    return s.substr(a, b - a);
  }
  // Parses until one of `stops`; returns which stop tag ended the block in `hit` (with its full text).
  std::vector<NodeP> block(const std::vector<std::string>& stops, std::string& hit) {
    std::vector<NodeP> out;
    while (i_ < p_.size()) {
      Piece& pc = p_[i_];
      if (pc.kind == 0) { auto n = std::make_shared<Node>(); n->kind = Node::Text; n->text = pc.s; out.push_back(n); ++i_; continue; }
      if (pc.kind == 1) {
        auto n = std::make_shared<Node>();
        n->kind = Node::Output;
        n->expr = ExprParser(lex_expr(pc.s)).parse_full();
        out.push_back(n);
        ++i_;
        continue;
      }
      std::string w = first_word(pc.s);
      for (auto& s : stops) if (w == s) { hit = pc.s; ++i_; return out; }
      ++i_;
      std::string rest = trim(trim(pc.s).substr(w.size()));
      if (w == "if") out.push_back(parse_if(rest));
      else if (w == "for") out.push_back(parse_for(rest));
      else if (w == "set") out.push_back(parse_set(rest));
      else if (w == "macro") out.push_back(parse_macro(rest));
      else if (w == "generation" || w == "endgeneration") continue;   // training-mask markers: transparent
      else if (w == "raw" || w == "filter" || w == "call" || w == "include" || w == "import" || w == "extends")
        throw Error("unsupported tag '" + w + "'");
      else throw Error("unknown tag '" + w + "'");
    }
    if (!stops.empty()) throw Error("missing end tag for block (expected " + stops.back() + ")");
    hit.clear();
    return out;
  }
  NodeP parse_if(const std::string& cond) {
    auto n = std::make_shared<Node>();
    n->kind = Node::If;
    ExprP c = ExprParser(lex_expr(cond)).parse_full();
    for (;;) {
      std::string hit;
      auto body = block({"elif", "else", "endif"}, hit);
      n->branches.emplace_back(c, body);
      std::string w = first_word(hit);
      if (w == "endif") break;
      if (w == "elif") c = ExprParser(lex_expr(trim(trim(hit).substr(4)))).parse_full();
      else c = nullptr;   // else
      if (w == "else") {
        std::string h2;
        auto eb = block({"endif"}, h2);
        n->branches.emplace_back(nullptr, eb);
        break;
      }
    }
    return n;
  }
  NodeP parse_for(const std::string& spec) {
    auto n = std::make_shared<Node>();
    n->kind = Node::For;
    ExprParser ep(lex_expr(spec));
    n->vars.push_back(ep.expect_name());
    while (ep.is_op(",")) { ++ep.p_; n->vars.push_back(ep.expect_name()); }
    if (!ep.is_name("in")) throw Error("expected 'in' in for tag");
    ++ep.p_;
    // iterable: parse an expression that stops at a top-level "if" / "recursive"
    // (ternary() would swallow "if"): re-lex the remainder by hand
    size_t in_pos = spec.find(" in ");
    std::string rest = spec.substr(in_pos + 4);
    std::string iter_src = rest, cond_src;
    int depth = 0;
    for (size_t k = 0; k + 3 < rest.size(); ++k) {
      char ch = rest[k];
      if (ch == '(' || ch == '[' || ch == '{') ++depth;
      if (ch == ')' || ch == ']' || ch == '}') --depth;
      if (depth == 0 && rest.compare(k, 4, " if ") == 0) { iter_src = rest.substr(0, k); cond_src = rest.substr(k + 4); break; }
    }
    n->expr = ExprParser(lex_expr(iter_src)).parse_full();
    if (!cond_src.empty()) n->cond = ExprParser(lex_expr(cond_src)).parse_full();
    std::string hit;
    n->body = block({"else", "endfor"}, hit);
    if (first_word(hit) == "else") { std::string h2; n->else_body = block({"endfor"}, h2); }
    return n;
  }
  NodeP parse_set(const std::string& spec) {
    auto n = std::make_shared<Node>();
    size_t eq = std::string::npos;
    int depth = 0;
    for (size_t k = 0; k < spec.size(); ++k) {
      char ch = spec[k];
      if (ch == '(' || ch == '[') ++depth;
      if (ch == ')' || ch == ']') --depth;
      if (ch == '=' && depth == 0 && (k + 1 >= spec.size() || spec[k + 1] != '=') && (k == 0 || (spec[k - 1] != '=' && spec[k - 1] != '!' && spec[k - 1] != '<' && spec[k - 1] != '>'))) { eq = k; break; }
    }
    std::string target = trim(eq == std::string::npos ? spec : spec.substr(0, eq));
    size_t dot = target.find('.');
    if (dot != std::string::npos) { n->text = trim(target.substr(0, dot)); n->attr = trim(target.substr(dot + 1)); }
    else n->text = target;
    if (eq == std::string::npos) {
      n->kind = Node::SetBlock;
      std::string hit;
      n->body = block({"endset"}, hit);
    } else {
      n->kind = Node::Set;
      n->expr = ExprParser(lex_expr(spec.substr(eq + 1))).parse_full();
    }
    return n;
  }
  NodeP parse_macro(const std::string& spec) {
    auto n = std::make_shared<Node>();
    n->kind = Node::Macro;
    ExprParser ep(lex_expr(spec));
    n->text = ep.expect_name();
    ep.expect_op("(");
    while (!ep.is_op(")")) {
      n->vars.push_back(ep.expect_name());
      if (ep.is_op("=")) { ++ep.p_; n->defaults.push_back(ep.ternary()); }
      else if (!n->defaults.empty()) throw Error("macro parameter without default after one with default");
      if (ep.is_op(",")) ++ep.p_;
    }
    std::string hit;
    n->body = block({"endmacro"}, hit);
    return n;
  }
};
