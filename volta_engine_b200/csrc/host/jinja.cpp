// Evaluator of the Jinja2 subset (AST and parsers are in jinja_ast.h) and the C entry points used by the
// chat-template layer. jinja_ast.h opens namespaces vh::jinja; this file closes them.
#include <algorithm>
#include <cstdlib>
#include <ctime>

#include "jinja_ast.h"   // leaves namespace vh::jinja open

struct Macro {
  const Node* node;
};

class Interp {
 public:
  explicit Interp(const Json& ctx) { scopes_.push_back(ctx.type == Json::Object ? ctx : Json::object()); }
  std::string render(const std::vector<NodeP>& nodes) {
    std::string out;
    exec(nodes, out);
    return out;
  }

 private:
  std::vector<Json> scopes_;
  std::map<std::string, Macro> macros_;
  std::vector<std::shared_ptr<Json>> namespaces_;   // namespace() objects are shared by reference

  // namespace objects: stored as {"__ns__": index}; attribute reads/writes go to namespaces_[index]
  Json* ns_of(const Json& v) {
    if (v.type != Json::Object) return nullptr;
    const Json* k = v.find("__ns__");
    if (!k) return nullptr;
    return namespaces_[(size_t)k->i].get();
  }
  Json lookup(const std::string& name) {
    for (size_t n = scopes_.size(); n-- > 0;) {
      const Json* v = scopes_[n].find(name);
      if (v) return *v;
    }
    return undefined();
  }
  void assign(const std::string& name, Json v) { scopes_.back().set(name, std::move(v)); }

  void exec(const std::vector<NodeP>& nodes, std::string& out) {
    for (auto& np : nodes) {
      const Node& n = *np;
      switch (n.kind) {
        case Node::Text: out += n.text; break;
        case Node::Output: out += to_str(eval(*n.expr)); break;
        case Node::If:
          for (auto& br : n.branches)
            if (!br.first || truthy(eval(*br.first))) { exec(br.second, out); break; }
          break;
        case Node::For: exec_for(n, out); break;
        case Node::Set: {
          Json v = eval(*n.expr);
          if (!n.attr.empty()) {
            Json target = lookup(n.text);
            Json* ns = ns_of(target);
            if (!ns) throw Error("cannot set attribute on non-namespace '" + n.text + "'");
            ns->set(n.attr, std::move(v));
          } else {
            assign(n.text, std::move(v));
          }
          break;
        }
        case Node::SetBlock: {
          std::string s;
          exec(n.body, s);
          assign(n.text, Json::string(s));
          break;
        }
        case Node::Macro: macros_[n.text] = Macro{&n}; break;
        case Node::Block: exec(n.body, out); break;
      }
    }
  }

  void exec_for(const Node& n, std::string& out) {
    Json it = eval(*n.expr);
    std::vector<Json> items;
    if (it.type == Json::Array) items = it.arr;
    else if (it.type == Json::Object) for (auto& kv : it.obj) items.push_back(Json::string(kv.first));
    else if (it.type == Json::String) {
      for (size_t i = 0; i < it.s.size();) {
        size_t j = i + 1;
        while (j < it.s.size() && ((unsigned char)it.s[j] & 0xC0) == 0x80) ++j;
        items.push_back(Json::string(it.s.substr(i, j - i)));
        i = j;
      }
    } else if (it.type != Json::Null) throw Error("object is not iterable");
    auto bind = [&](const Json& item) {
      if (n.vars.size() == 1) { assign(n.vars[0], item); return; }
      if (item.type != Json::Array || item.arr.size() != n.vars.size()) throw Error("cannot unpack loop item");
      for (size_t k = 0; k < n.vars.size(); ++k) assign(n.vars[k], item.arr[k]);
    };
    if (n.cond) {
      std::vector<Json> kept;
      scopes_.push_back(Json::object());
      for (auto& item : items) { bind(item); if (truthy(eval(*n.cond))) kept.push_back(item); }
      scopes_.pop_back();
      items.swap(kept);
    }
    if (items.empty()) { exec(n.else_body, out); return; }
    scopes_.push_back(Json::object());
    const int64_t len = (int64_t)items.size();
    for (int64_t i = 0; i < len; ++i) {
      bind(items[(size_t)i]);
      Json loop = Json::object();
      loop.set("index", Json::integer(i + 1));
      loop.set("index0", Json::integer(i));
      loop.set("first", Json::boolean(i == 0));
      loop.set("last", Json::boolean(i == len - 1));
      loop.set("length", Json::integer(len));
      loop.set("revindex", Json::integer(len - i));
      loop.set("revindex0", Json::integer(len - i - 1));
      loop.set("previtem", i > 0 ? items[(size_t)i - 1] : undefined());
      loop.set("nextitem", i + 1 < len ? items[(size_t)i + 1] : undefined());
      assign("loop", loop);
      exec(n.body, out);
    }
    scopes_.pop_back();
  }

  Json call_macro(const Macro& m, const std::vector<Json>& args, const std::vector<std::pair<std::string, Json>>& kw) {
    const Node& n = *m.node;
    scopes_.push_back(Json::object());
    const size_t nreq = n.vars.size() - n.defaults.size();
    for (size_t k = 0; k < n.vars.size(); ++k) {
      Json v = undefined();
      if (k < args.size()) v = args[k];
      else if (k >= nreq) v = eval(*n.defaults[k - nreq]);
      for (auto& p : kw) if (p.first == n.vars[k]) v = p.second;
      assign(n.vars[k], v);
    }
    std::string out;
    exec(n.body, out);
    scopes_.pop_back();
    return Json::string(out);
  }

  static int64_t norm_index(int64_t i, int64_t n) { return i < 0 ? i + n : i; }

  Json get_attr(const Json& base, const std::string& name) {
    if (Json* ns = ns_of(base)) {
      const Json* v = ns->find(name);
      return v ? *v : undefined();
    }
    if (base.type == Json::Object) {
      const Json* v = base.find(name);
      return v ? *v : undefined();
    }
    return undefined();
  }

  Json eval(const Expr& e) {
    switch (e.kind) {
      case Expr::Lit: return e.lit;
      case Expr::Var: return lookup(e.name);
      case Expr::List: {
        Json a = Json::array();
        for (auto& x : e.args) a.arr.push_back(eval(*x));
        return a;
      }
      case Expr::Dict: {
        Json o = Json::object();
        for (auto& kv : e.items) o.set(to_str(eval(*kv.first)), eval(*kv.second));
        return o;
      }
      case Expr::Attr: return get_attr(eval(*e.a), e.name);
      case Expr::Index: {
        Json base = eval(*e.a), idx = eval(*e.b);
        if (base.type == Json::Array && idx.is_number()) {
          int64_t i = norm_index(idx.as_int(), (int64_t)base.arr.size());
          if (i < 0 || i >= (int64_t)base.arr.size()) return undefined();
          return base.arr[(size_t)i];
        }
        if (base.type == Json::String && idx.is_number()) {
          int64_t i = norm_index(idx.as_int(), (int64_t)base.s.size());
          if (i < 0 || i >= (int64_t)base.s.size()) return undefined();
          return Json::string(base.s.substr((size_t)i, 1));
        }
        if (idx.type == Json::String) return get_attr(base, idx.s);
        return undefined();
      }
      case Expr::Slice: {
        Json base = eval(*e.a);
        const int64_t n = base.type == Json::Array ? (int64_t)base.arr.size() : (int64_t)base.s.size();
        int64_t step = e.args[2] ? eval(*e.args[2]).as_int() : 1;
        if (step == 0) throw Error("slice step cannot be zero");
        int64_t lo = e.args[0] ? norm_index(eval(*e.args[0]).as_int(), n) : (step > 0 ? 0 : n - 1);
        int64_t hi = e.args[1] ? norm_index(eval(*e.args[1]).as_int(), n) : (step > 0 ? n : -1);
        if (step > 0) { lo = std::max<int64_t>(0, std::min(lo, n)); hi = std::max<int64_t>(0, std::min(hi, n)); }
        else { lo = std::max<int64_t>(-1, std::min(lo, n - 1)); hi = std::max<int64_t>(-1, std::min(hi, n - 1)); }
        Json out = base.type == Json::Array ? Json::array() : Json::string("");
        for (int64_t i = lo; step > 0 ? i < hi : i > hi; i += step) {
          if (base.type == Json::Array) out.arr.push_back(base.arr[(size_t)i]);
          else out.s.push_back(base.s[(size_t)i]);
        }
        return out;
      }
      case Expr::Unary: {
        Json v = eval(*e.a);
        if (e.name == "not") return Json::boolean(!truthy(v));
        if (v.type == Json::Int) return Json::integer(-v.i);
        return Json::number(-v.as_double());
      }
      case Expr::Cond:
        if (truthy(eval(*e.a))) return eval(*e.b);
        return e.c ? eval(*e.c) : undefined();
      case Expr::Binary: return eval_binary(e);
      case Expr::Test: {
        bool r = eval_test(e);
        return Json::boolean(e.negate ? !r : r);
      }
      case Expr::Filter: {
        std::vector<Json> args;
        for (auto& a : e.args) args.push_back(eval(*a));
        std::vector<std::pair<std::string, Json>> kw;
        for (auto& k : e.kwargs) kw.emplace_back(k.first, eval(*k.second));
        return apply_filter(e.name, eval(*e.a), args, kw);
      }
      case Expr::Call: return eval_call(e);
    }
    return undefined();
  }

  Json eval_binary(const Expr& e) {
    const std::string& op = e.name;
    if (op == "and") { Json l = eval(*e.a); return truthy(l) ? eval(*e.b) : l; }
    if (op == "or") { Json l = eval(*e.a); return truthy(l) ? l : eval(*e.b); }
    Json l = eval(*e.a), r = eval(*e.b);
    if (op == "==") return Json::boolean(equals(l, r));
    if (op == "!=") return Json::boolean(!equals(l, r));
    if (op == "in") {
      if (r.type == Json::String) return Json::boolean(l.type == Json::String && r.s.find(l.s) != std::string::npos);
      if (r.type == Json::Array) { for (auto& x : r.arr) if (equals(x, l)) return Json::boolean(true); return Json::boolean(false); }
      if (r.type == Json::Object) return Json::boolean(l.type == Json::String && (ns_of(r) ? ns_of(r)->find(l.s) : r.find(l.s)) != nullptr);
      return Json::boolean(false);
    }
    if (op == "~") return Json::string(to_str(l) + to_str(r));
    if (op == "<" || op == ">" || op == "<=" || op == ">=") {
      int c;
      if (l.type == Json::String && r.type == Json::String) c = l.s.compare(r.s);
      else { double a = l.as_double(), b = r.as_double(); c = a < b ? -1 : a > b ? 1 : 0; }
      return Json::boolean(op == "<" ? c < 0 : op == ">" ? c > 0 : op == "<=" ? c <= 0 : c >= 0);
    }
    if (op == "+") {
      if (l.type == Json::String && r.type == Json::String) return Json::string(l.s + r.s);
      if (l.type == Json::Array && r.type == Json::Array) { Json o = l; o.arr.insert(o.arr.end(), r.arr.begin(), r.arr.end()); return o; }
      if (l.type == Json::Int && r.type == Json::Int) return Json::integer(l.i + r.i);
      if (l.is_number() && r.is_number()) return Json::number(l.as_double() + r.as_double());
      throw Error("unsupported operands for +");
    }
    if (op == "*" && l.type == Json::String && r.type == Json::Int) {
      std::string s;
      for (int64_t k = 0; k < r.i; ++k) s += l.s;
      return Json::string(s);
    }
    if (!l.is_number() || !r.is_number()) {
      if (op == "%" && l.type == Json::String) return l;  // printf-style formatting is not supported
      throw Error("unsupported operands for " + op);
    }
    const bool ints = l.type == Json::Int && r.type == Json::Int;
    if (op == "-") return ints ? Json::integer(l.i - r.i) : Json::number(l.as_double() - r.as_double());
    if (op == "*") return ints ? Json::integer(l.i * r.i) : Json::number(l.as_double() * r.as_double());
    if (op == "/") { if (r.as_double() == 0) throw Error("division by zero"); return Json::number(l.as_double() / r.as_double()); }
    if (op == "//") { if (r.as_double() == 0) throw Error("division by zero"); return Json::integer((int64_t)std::floor(l.as_double() / r.as_double())); }
    if (op == "%") {
      if (r.as_double() == 0) throw Error("modulo by zero");
      if (ints) { int64_t m = l.i % r.i; if (m != 0 && ((m < 0) != (r.i < 0))) m += r.i; return Json::integer(m); }
      return Json::number(std::fmod(l.as_double(), r.as_double()));
    }
    throw Error("unknown operator " + op);
  }

  bool eval_test(const Expr& e) {
    Json v = eval(*e.a);
    const std::string& t = e.name;
    if (t == "defined") return !is_undefined(v);
    if (t == "undefined") return is_undefined(v);
    if (t == "none") return v.type == Json::Null && !is_undefined(v);
    if (t == "string") return v.type == Json::String;
    if (t == "number") return v.is_number();
    if (t == "integer") return v.type == Json::Int;
    if (t == "float") return v.type == Json::Float;
    if (t == "boolean") return v.type == Json::Bool;
    if (t == "mapping") return v.type == Json::Object;
    if (t == "sequence") return v.type == Json::Array || v.type == Json::String || v.type == Json::Object;
    if (t == "iterable") return v.type == Json::Array || v.type == Json::String || v.type == Json::Object;
    if (t == "true") return v.type == Json::Bool && v.b;
    if (t == "false") return v.type == Json::Bool && !v.b;
    if (t == "odd") return v.as_int() % 2 != 0;
    if (t == "even") return v.as_int() % 2 == 0;
    if (t == "equalto" || t == "eq" || t == "sameas") return !e.args.empty() && equals(v, eval(*e.args[0]));
    if (t == "ne") return !e.args.empty() && !equals(v, eval(*e.args[0]));
    if (t == "in") { if (e.args.empty()) return false; Json c = eval(*e.args[0]); if (c.type == Json::Array) { for (auto& x : c.arr) if (equals(x, v)) return true; } return false; }
    if (t == "callable") return false;
    throw Error("unknown test '" + t + "'");
  }

  static Json kwarg(const std::vector<std::pair<std::string, Json>>& kw, const std::string& k, Json d = undefined()) {
    for (auto& p : kw) if (p.first == k) return p.second;
    return d;
  }
  static std::string strip(const std::string& s, const std::string& chars, bool left, bool right) {
    auto in = [&](char c) { return chars.empty() ? isspace((unsigned char)c) != 0 : chars.find(c) != std::string::npos; };
    size_t a = 0, b = s.size();
    if (left) while (a < b && in(s[a])) ++a;
    if (right) while (b > a && in(s[b - 1])) --b;
    return s.substr(a, b - a);
  }

  Json apply_filter(const std::string& f, Json v, const std::vector<Json>& args,
                    const std::vector<std::pair<std::string, Json>>& kw);
  Json eval_call(const Expr& e);
  Json call_method(const Json& self, const Expr& target, const std::string& m, const std::vector<Json>& args,
                   const std::vector<std::pair<std::string, Json>>& kw);
  friend std::string render_template(const std::string&, const Json&);
};

}  // namespace jinja
}  // namespace vh

#include "jinja_builtins.inc"
