// ir.cc — parser for the S-expression form of Sarek kernel IR and the
// structural recogniser that maps a kernel onto this backend's operators.
// The shapes matched are the ones the reference's PPX lowers the benchmark
// kernels to (sarek/ppx/Sarek_lower_ir.ml:274-526,577-702).
#include "ir.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <map>
#include <set>
#include <sstream>

#include "../../include/sb200.h"

namespace sb200 {

// ------------------------------------------------------------------ parser
namespace {
struct Parser {
  const std::string& t;
  size_t i = 0;
  std::string err;
  explicit Parser(const std::string& text) : t(text) {}
  void skip() {
    while (i < t.size()) {
      if (isspace(static_cast<unsigned char>(t[i]))) {
        ++i;
      } else if (t[i] == ';') {
        while (i < t.size() && t[i] != '\n') ++i;
      } else {
        break;
      }
    }
  }
  bool parse(Sx* out, int depth) {
    skip();
    if (i >= t.size()) {
      err = "unexpected end of IR text";
      return false;
    }
    if (depth > 512) {
      err = "IR nesting deeper than 512";
      return false;
    }
    if (t[i] == '(') {
      ++i;
      out->atom = false;
      for (;;) {
        skip();
        if (i >= t.size()) {
          err = "unbalanced '(' in IR text";
          return false;
        }
        if (t[i] == ')') {
          ++i;
          return true;
        }
        Sx kid;
        if (!parse(&kid, depth + 1)) return false;
        out->kids.push_back(std::move(kid));
      }
    }
    if (t[i] == ')') {
      err = "unexpected ')' in IR text";
      return false;
    }
    out->atom = true;
    if (t[i] == '"') {
      size_t j = i + 1;
      std::string s;
      while (j < t.size() && t[j] != '"') {
        if (t[j] == '\\' && j + 1 < t.size()) ++j;
        s.push_back(t[j++]);
      }
      if (j >= t.size()) {
        err = "unterminated string in IR text";
        return false;
      }
      out->s = s;
      i = j + 1;
      return true;
    }
    size_t j = i;
    while (j < t.size() && !isspace(static_cast<unsigned char>(t[j])) && t[j] != '(' && t[j] != ')') ++j;
    out->s = t.substr(i, j - i);
    i = j;
    return true;
  }
};
}  // namespace

bool sx_parse(const std::string& text, Sx* out, std::string* err) {
  Parser p(text);
  Sx x;
  if (!p.parse(&x, 0)) {
    if (err) *err = p.err;
    return false;
  }
  p.skip();
  if (p.i != text.size()) {
    if (err) *err = "trailing characters after the kernel form";
    return false;
  }
  *out = std::move(x);
  return true;
}

std::string sx_print(const Sx& x) {
  if (x.atom) {
    bool plain = !x.s.empty();
    for (char c : x.s)
      if (isspace(static_cast<unsigned char>(c)) || c == '(' || c == ')' || c == '"' || c == ';') plain = false;
    if (plain) return x.s;
    std::string o = "\"";
    for (char c : x.s) {
      if (c == '"' || c == '\\') o.push_back('\\');
      o.push_back(c);
    }
    return o + "\"";
  }
  std::string o = "(";
  for (size_t i = 0; i < x.kids.size(); ++i) {
    if (i) o.push_back(' ');
    o += sx_print(x.kids[i]);
  }
  return o + ")";
}

bool sx_equal(const Sx& a, const Sx& b) {
  if (a.atom != b.atom) return false;
  if (a.atom) return a.s == b.s;
  if (a.kids.size() != b.kids.size()) return false;
  for (size_t i = 0; i < a.kids.size(); ++i)
    if (!sx_equal(a.kids[i], b.kids[i])) return false;
  return true;
}

// --------------------------------------------------------------- recogniser
namespace {

using Env = std::map<std::string, Sx>;  // var id -> inlined defining expression

// Replace every (evar NAME ID) whose ID is let-bound by its definition.
Sx inline_expr(const Sx& e, const Env& env) {
  if (e.atom) return e;
  if (e.is("evar") && e.size() >= 3) {
    auto it = env.find(e[2].s);
    if (it != env.end()) return it->second;
    return e;
  }
  Sx o;
  o.kids.reserve(e.kids.size());
  for (const Sx& k : e.kids) o.kids.push_back(inline_expr(k, env));
  return o;
}

bool is_binop(const Sx& e, const char* op, const Sx** l, const Sx** r) {
  if (!e.is("binop") || e.size() != 4 || !e[1].atom || e[1].s != op) return false;
  *l = &e[2];
  *r = &e[3];
  return true;
}

// Commutative binop: calls f(l, r) and f(r, l) until one succeeds.
bool is_comm(const Sx& e, const char* op, const std::function<bool(const Sx&, const Sx&)>& f) {
  const Sx *l, *r;
  if (!is_binop(e, op, &l, &r)) return false;
  return f(*l, *r) || f(*r, *l);
}

bool is_intrinsic(const Sx& e, const char* name) {
  return e.is("intrinsic") && e.size() >= 3 && e[2].atom && e[2].s == name;
}

bool contains_intrinsic(const Sx& e, const char* name) {
  if (e.atom) return false;
  if (is_intrinsic(e, name)) return true;
  for (const Sx& k : e.kids)
    if (contains_intrinsic(k, name)) return true;
  return false;
}

// global x index: global_thread_id / global_idx_x, or thread_idx_x + block_dim_x*block_idx_x
bool is_global_x(const Sx& e) {
  if (is_intrinsic(e, "global_thread_id") || is_intrinsic(e, "global_idx_x")) return true;
  return is_comm(e, "add", [](const Sx& a, const Sx& b) {
    return is_intrinsic(a, "thread_idx_x") && is_comm(b, "mul", [](const Sx& c, const Sx& d) {
             return is_intrinsic(c, "block_dim_x") && is_intrinsic(d, "block_idx_x");
           });
  });
}
bool is_global_y(const Sx& e) {
  if (is_intrinsic(e, "global_idx_y")) return true;
  return is_comm(e, "add", [](const Sx& a, const Sx& b) {
    return is_intrinsic(a, "thread_idx_y") && is_comm(b, "mul", [](const Sx& c, const Sx& d) {
             return is_intrinsic(c, "block_dim_y") && is_intrinsic(d, "block_idx_y");
           });
  });
}

struct Ctx {
  KernelPlan* plan;
  std::string why;  // first reason a match failed, for the error message
  int param_index(const std::string& name) const {
    for (size_t i = 0; i < plan->params.size(); ++i)
      if (plan->params[i].name == name) return static_cast<int>(i);
    return -1;
  }
  // (evar NAME ID) naming a scalar parameter of element type elt (or any when elt == nullptr)
  int scalar_param(const Sx& e, const char* elt) const {
    if (!e.is("evar") || e.size() < 3) return -1;
    for (size_t i = 0; i < plan->params.size(); ++i) {
      const ParamInfo& p = plan->params[i];
      if (!p.is_vec && p.name == e[1].s && std::to_string(p.id) == e[2].s && (!elt || p.elt == elt))
        return static_cast<int>(i);
    }
    return -1;
  }
  int vec_param(const std::string& name, const char* elt) const {
    int i = param_index(name);
    if (i < 0 || !plan->params[i].is_vec) return -1;
    if (elt && plan->params[i].elt != elt) return -1;
    return i;
  }
  // (read ARR IDX) of a float32 vector parameter
  bool is_read(const Sx& e, int* param, const Sx** idx) const {
    if (!e.is("read") || e.size() != 3 || !e[1].atom) return false;
    int p = vec_param(e[1].s, "f32");
    if (p < 0) return false;
    *param = p;
    *idx = &e[2];
    return true;
  }
  bool is_coef(const Sx& e, Coef* c) const {
    if (e.is("const") && e.size() == 3 && (e[1].s == "f32" || e[1].s == "f64")) {
      c->param = -1;
      c->value = strtod(e[2].s.c_str(), nullptr);
      return true;
    }
    int p = scalar_param(e, "f32");
    if (p >= 0) {
      c->param = p;
      return true;
    }
    return false;
  }
};

bool is_const_i32(const Sx& e, long long v) {
  return e.is("const") && e.size() == 3 && (e[1].s == "i32" || e[1].s == "i64") && atoll(e[2].s.c_str()) == v;
}
bool is_const_f_zero(const Sx& e) {
  return e.is("const") && e.size() == 3 && (e[1].s == "f32" || e[1].s == "f64") && strtod(e[2].s.c_str(), nullptr) == 0.0;
}

// Peel lets / blocks / single-statement seqs / pragmas / else-less ifs off the
// front of a body.  Shared-array lets are recorded, not inlined.
struct Peeled {
  Env env;
  std::set<std::string> shared;
  std::vector<Sx> guards;
  const Sx* core = nullptr;
};

bool is_shared_let(const Sx& s) {
  return s.is("let") && s.size() == 6 && s[4].is("arraycreate");
}

void peel(const Sx& stmt, Peeled* p, bool through_guards) {
  const Sx* s = &stmt;
  for (;;) {
    if (s->is("let") && s->size() == 6) {
      if (is_shared_let(*s)) {
        p->shared.insert((*s)[1].s);
      } else {
        p->env[(*s)[2].s] = inline_expr((*s)[4], p->env);
      }
      s = &(*s)[5];
    } else if (s->is("block") && s->size() == 2) {
      s = &(*s)[1];
    } else if (s->is("pragma") && s->size() == 3) {
      s = &(*s)[2];
    } else if (s->is("seq")) {
      const Sx* only = nullptr;
      int count = 0;
      for (size_t i = 1; i < s->size(); ++i)
        if (!(*s)[i].is("empty")) {
          only = &(*s)[i];
          ++count;
        }
      if (count != 1) break;
      s = only;
    } else if (through_guards && s->is("sif") && s->size() == 3) {
      p->guards.push_back(inline_expr((*s)[1], p->env));
      s = &(*s)[2];
    } else {
      break;
    }
  }
  p->core = s;
}

std::vector<const Sx*> seq_items(const Sx& s) {
  std::vector<const Sx*> v;
  if (s.is("seq")) {
    for (size_t i = 1; i < s.size(); ++i) {
      if (s[i].is("empty")) continue;
      if (s[i].is("seq")) {
        for (const Sx* k : seq_items(s[i])) v.push_back(k);
      } else {
        v.push_back(&s[i]);
      }
    }
  } else if (!s.is("empty")) {
    v.push_back(&s);
  }
  return v;
}

// ------------------------------------------------------------------- maps

Sx strip_stored_marks(const Sx& e) {
  if (e.atom) return e;
  if (e.is("intrinsic") && e.size() == 4 && e[2].atom && e[2].s == "stored_f32") return strip_stored_marks(e[3]);
  Sx o;
  o.kids.reserve(e.kids.size());
  for (const Sx& k : e.kids) o.kids.push_back(strip_stored_marks(k));
  return o;
}

// Substitute reads of arrays written earlier in the same straight-line body.
Sx subst_reads(const Sx& e, const std::map<std::string, Sx>& written, const Sx& idx) {
  if (e.atom) return e;
  if (e.is("read") && e.size() == 3 && e[1].atom) {
    auto it = written.find(e[1].s);
    if (it != written.end() && sx_equal(e[2], idx)) return it->second;
  }
  Sx o;
  for (const Sx& k : e.kids) o.kids.push_back(subst_reads(k, written, idx));
  return o;
}

struct Triad {
  int b, c;
  Coef s;
};

bool match_triad(const Ctx& cx, const Sx& e, const Sx& idx, Triad* t) {
  return is_comm(e, "add", [&](const Sx& l, const Sx& r) {
    const Sx* i0;
    int b;
    if (!cx.is_read(l, &b, &i0) || !sx_equal(*i0, idx)) return false;
    return is_comm(r, "mul", [&](const Sx& m0, const Sx& m1) {
      const Sx* i1;
      int c;
      Coef s;
      if (!cx.is_read(m0, &c, &i1) || !sx_equal(*i1, idx) || !cx.is_coef(m1, &s)) return false;
      t->b = b;
      t->c = c;
      t->s = s;
      return true;
    });
  });
}

bool match_map(Ctx& cx, const Sx& body) {
  KernelPlan& plan = *cx.plan;
  Peeled pl;
  peel(body, &pl, true);
  if (!pl.shared.empty()) {
    cx.why = "uses shared arrays";
    return false;
  }
  std::vector<const Sx*> items = seq_items(*pl.core);
  if (items.empty() || items.size() > 2) {
    cx.why = "body is not one or two element stores";
    return false;
  }
  MapPlan mp;
  Sx idx;
  bool have_idx = false;
  std::map<std::string, Sx> written;
  std::vector<std::pair<int, Sx>> stores;  // (out param, inlined+substituted rhs)
  for (const Sx* it : items) {
    if (!it->is("assign") || it->size() != 3 || !(*it)[1].is("elem") || (*it)[1].size() != 3) {
      cx.why = "statement is not an array element store";
      return false;
    }
    const Sx& lv = (*it)[1];
    Sx this_idx = inline_expr(lv[2], pl.env);
    if (!have_idx) {
      idx = this_idx;
      have_idx = true;
    } else if (!sx_equal(idx, this_idx)) {
      cx.why = "stores use different indices";
      return false;
    }
    int out = cx.vec_param(lv[1].s, "f32");
    if (out < 0) {
      cx.why = "store target is not a float32 vector parameter";
      return false;
    }
    Sx rhs = subst_reads(inline_expr((*it)[2], pl.env), written, idx);
    written[lv[1].s] = rhs;
    stores.emplace_back(out, rhs);
  }
  if (is_global_x(idx)) {
    mp.index_kind = IDX_GLOBAL;
  } else if (is_intrinsic(idx, "thread_idx_x")) {
    mp.index_kind = IDX_THREAD_X;
  } else {
    cx.why = "element index is not the global or block-local x thread index";
    return false;
  }
  if (pl.guards.size() > 1) {
    cx.why = "more than one guard";
    return false;
  }
  if (pl.guards.size() == 1) {
    const Sx *l, *r;
    if (!is_binop(pl.guards[0], "lt", &l, &r) || !sx_equal(*l, idx) || (mp.n_param = cx.scalar_param(*r, "i32")) < 0) {
      cx.why = "guard is not `index < n` with n an int32 parameter";
      return false;
    }
  }
  // classify the final store (and the optional kept intermediate).  The ahead-of-time operators round an
  // eliminated intermediate to float32 themselves (one fused multiply-add per former kernel), so the
  // stored_f32 marks of the backend's guarded fusion are dropped for the classification.
  const Sx rhs_unmarked = strip_stored_marks(stores.back().second);
  const Sx& rhs = rhs_unmarked;
  mp.out0 = stores.back().first;
  Triad t;
  bool ok = false;
  // vector_add
  ok = is_comm(rhs, "add", [&](const Sx& l, const Sx& r) {
    const Sx *i0, *i1;
    int a, b;
    if (!cx.is_read(l, &a, &i0) || !cx.is_read(r, &b, &i1)) return false;
    if (!sx_equal(*i0, idx) || !sx_equal(*i1, idx)) return false;
    mp.op = OP_VECADD;
    mp.in0 = a;
    mp.in1 = b;
    return true;
  });
  if (ok && stores.size() == 2) ok = false;
  if (!ok && stores.size() == 1 && match_triad(cx, rhs, idx, &t)) {
    mp.op = OP_TRIAD;
    mp.in0 = t.b;
    mp.in1 = t.c;
    mp.scalar = t.s;
    ok = true;
  }
  if (!ok) {
    // d = T*T + b with T = b + c*s
    ok = is_comm(rhs, "add", [&](const Sx& l, const Sx& r) {
      const Sx *m0, *m1, *i0;
      int b;
      if (!is_binop(l, "mul", &m0, &m1) || !sx_equal(*m0, *m1)) return false;
      if (!match_triad(cx, *m0, idx, &t)) return false;
      if (!cx.is_read(r, &b, &i0) || !sx_equal(*i0, idx) || b != t.b) return false;
      mp.op = OP_CHAIN;
      mp.in0 = t.b;
      mp.in1 = t.c;
      mp.scalar = t.s;
      return true;
    });
    if (ok && stores.size() == 2) {
      Triad t2;
      if (match_triad(cx, stores[0].second, idx, &t2) && t2.b == t.b && t2.c == t.c && t2.s.param == t.s.param &&
          t2.s.value == t.s.value) {
        mp.op = OP_CHAIN_KEEP;
        mp.out1 = stores[0].first;
      } else {
        ok = false;
      }
    }
  }
  if (!ok) {
    cx.why = "element expression is not one of: a+b, b+c*s, (b+c*s)^2+b";
    return false;
  }
  if (mp.out0 == mp.out1) {
    cx.why = "both stores target the same vector";
    return false;
  }
  plan.kind = KIND_MAP;
  plan.map = mp;
  static const char* names[] = {"vector_add", "stream_triad", "triad_square_chain", "triad_square_chain(keep)"};
  plan.description = std::string("map:") + names[mp.op] + (mp.n_param >= 0 ? " guarded" : " unguarded") +
                     (mp.index_kind == IDX_GLOBAL ? " idx=global_x" : " idx=thread_idx_x");
  return true;
}

// ------------------------------------------------------- generic map codegen
// Emits the element function of an arbitrary straight-line element-wise map.
// Arithmetic follows the Native backend exactly: loads widen to double, every
// operation is a separately rounded double operation (no contraction), literals
// are doubles, one rounding to float32 at each store, and a later read of a
// vector stored earlier in the same body sees the rounded value.
struct GenCtx {
  const Ctx* cx;
  const Sx* idx;
  GenericMap* gm;
  std::map<std::string, std::string> stored;  // array name -> temp holding its rounded value
  std::string why;
  int input_slot(int param) {
    for (size_t i = 0; i < gm->inputs.size(); ++i)
      if (gm->inputs[i] == param) return static_cast<int>(i);
    gm->inputs.push_back(param);
    return static_cast<int>(gm->inputs.size()) - 1;
  }
  int scalar_slot(int param) {
    for (size_t i = 0; i < gm->scalars.size(); ++i)
      if (gm->scalars[i] == param) return static_cast<int>(i);
    gm->scalars.push_back(param);
    return static_cast<int>(gm->scalars.size()) - 1;
  }
};

bool gen_int(GenCtx& g, const Sx& e, std::string* out);

bool gen_float(GenCtx& g, const Sx& e, std::string* out) {
  const Ctx& cx = *g.cx;
  if (e.is("const") && e.size() == 3 && (e[1].s == "f32" || e[1].s == "f64")) {
    char buf[64];
    snprintf(buf, sizeof buf, "%.17g", strtod(e[2].s.c_str(), nullptr));
    std::string t = buf;
    if (t.find_first_of(".eEn") == std::string::npos) t += ".0";
    *out = "(" + t + ")";
    return true;
  }
  if (e.is("evar")) {
    int p = cx.scalar_param(e, nullptr);
    if (p < 0) {
      g.why = "variable " + (e.size() > 1 ? e[1].s : std::string("?")) + " is not a scalar parameter";
      return false;
    }
    const std::string& elt = cx.plan->params[p].elt;
    if (elt != "f32" && elt != "f64") {
      g.why = "integer parameter used as a float value";
      return false;
    }
    *out = "s" + std::to_string(g.scalar_slot(p));
    return true;
  }
  if (e.is("read") && e.size() == 3 && e[1].atom) {
    if (!sx_equal(e[2], *g.idx)) {
      g.why = "vector " + e[1].s + " is read at an index other than the element index";
      return false;
    }
    auto it = g.stored.find(e[1].s);
    if (it != g.stored.end()) {
      *out = "((double)" + it->second + ")";
      return true;
    }
    int p = cx.vec_param(e[1].s, "f32");
    if (p < 0) {
      g.why = "read of " + e[1].s + ", which is not a float32 vector parameter";
      return false;
    }
    *out = "X" + std::to_string(g.input_slot(p));
    return true;
  }
  if (e.is("binop") && e.size() == 4) {
    static const std::map<std::string, const char*> ar = {{"add", "__dadd_rn"}, {"sub", "__dsub_rn"}, {"mul", "__dmul_rn"}, {"div", "__ddiv_rn"}};
    auto it = ar.find(e[1].s);
    if (it == ar.end()) {
      g.why = "operator " + e[1].s + " in a float expression";
      return false;
    }
    std::string a, b;
    if (!gen_float(g, e[2], &a) || !gen_float(g, e[3], &b)) return false;
    *out = std::string(it->second) + "(" + a + ", " + b + ")";
    return true;
  }
  if (e.is("unop") && e.size() == 3 && e[1].s == "neg") {
    std::string a;
    if (!gen_float(g, e[2], &a)) return false;
    *out = "(-" + a + ")";
    return true;
  }
  if (e.is("if") && e.size() == 4) {
    std::string c, a, b;
    std::function<bool(const Sx&, std::string*)> cond = [&](const Sx& x, std::string* o) -> bool {
      if (x.is("const") && x.size() == 3 && x[1].s == "bool") {
        *o = x[2].s == "true" ? "true" : "false";
        return true;
      }
      if (x.is("unop") && x.size() == 3 && x[1].s == "not") {
        std::string i;
        if (!cond(x[2], &i)) return false;
        *o = "(!" + i + ")";
        return true;
      }
      if (x.is("binop") && x.size() == 4) {
        static const std::map<std::string, const char*> cmp = {{"lt", "<"}, {"le", "<="}, {"gt", ">"}, {"ge", ">="}, {"eq", "=="}, {"ne", "!="}};
        auto it = cmp.find(x[1].s);
        std::string l, r;
        if (it != cmp.end()) {
          if (gen_float(g, x[2], &l) && gen_float(g, x[3], &r)) {
            *o = "(" + l + " " + it->second + " " + r + ")";
            return true;
          }
          return false;
        }
        if (x[1].s == "and" || x[1].s == "or") {
          if (!cond(x[2], &l) || !cond(x[3], &r)) return false;
          *o = "(" + l + (x[1].s == "and" ? " && " : " || ") + r + ")";
          return true;
        }
      }
      g.why = "unsupported condition";
      return false;
    };
    if (!cond(e[1], &c) || !gen_float(g, e[2], &a) || !gen_float(g, e[3], &b)) return false;
    *out = "(" + c + " ? " + a + " : " + b + ")";
    return true;
  }
  if (e.is("intrinsic") && e.size() >= 3) {
    static const std::map<std::string, const char*> un = {
        {"sin", "sin"}, {"cos", "cos"}, {"tan", "tan"}, {"asin", "asin"}, {"acos", "acos"}, {"atan", "atan"},
        {"sinh", "sinh"}, {"cosh", "cosh"}, {"tanh", "tanh"}, {"exp", "exp"}, {"log", "log"}, {"log10", "log10"},
        {"sqrt", "sqrt"}, {"ceil", "ceil"}, {"floor", "floor"}, {"expm1", "expm1"}, {"log1p", "log1p"}, {"abs_float", "fabs"}};
    static const std::map<std::string, const char*> bin = {{"pow", "pow"}, {"atan2", "atan2"}, {"hypot", "hypot"}, {"copysign", "copysign"},
                                                            {"add", "__dadd_rn"}, {"minus", "__dsub_rn"}, {"mul", "__dmul_rn"}, {"div", "__ddiv_rn"},
                                                            {"add_float32", "__dadd_rn"}, {"sub_float32", "__dsub_rn"},
                                                            {"mul_float32", "__dmul_rn"}, {"div_float32", "__ddiv_rn"}};
    const std::string& name = e[2].s;
    if (un.count(name) && e.size() == 4) {
      std::string a;
      if (!gen_float(g, e[3], &a)) return false;
      *out = std::string(un.at(name)) + "(" + a + ")";
      return true;
    }
    if (name == "stored_f32" && e.size() == 4) {
      // the value as a float32 vector would have held it: the backend's guarded fusion marks the store it
      // eliminated this way, so that the fused kernel rounds where the unfused kernels did
      std::string a;
      if (!gen_float(g, e[3], &a)) return false;
      *out = "((double)(float)(" + a + "))";
      return true;
    }
    if (name == "rsqrt" && e.size() == 4) {
      std::string a;
      if (!gen_float(g, e[3], &a)) return false;
      *out = "__ddiv_rn(1.0, sqrt(" + a + "))";
      return true;
    }
    if (bin.count(name) && e.size() == 5) {
      std::string a, b;
      if (!gen_float(g, e[3], &a) || !gen_float(g, e[4], &b)) return false;
      *out = std::string(bin.at(name)) + "(" + a + ", " + b + ")";
      return true;
    }
    if ((name == "of_int" || name == "float" || name == "float_of_int") && e.size() == 4) {
      std::string a;
      if (!gen_int(g, e[3], &a)) return false;
      *out = "((double)" + a + ")";
      return true;
    }
    g.why = "intrinsic " + name + " is not supported in element-wise maps";
    return false;
  }
  if (e.is("cast") && e.size() == 3 && (e[1].s == "f32" || e[1].s == "f64")) return gen_float(g, e[2], out);
  g.why = "unsupported expression form " + (e.atom ? e.s : (e.kids.empty() ? std::string("()") : e[0].s));
  return false;
}

bool gen_int(GenCtx& g, const Sx& e, std::string* out) {
  if (e.is("const") && e.size() == 3 && (e[1].s == "i32" || e[1].s == "i64")) {
    *out = "((long long)" + std::to_string(atoll(e[2].s.c_str())) + "ll)";
    return true;
  }
  if (e.is("evar")) {
    int p = g.cx->scalar_param(e, nullptr);
    if (p >= 0 && (g.cx->plan->params[p].elt == "i32" || g.cx->plan->params[p].elt == "i64")) {
      *out = "s" + std::to_string(g.scalar_slot(p));
      return true;
    }
  }
  if (e.is("binop") && e.size() == 4 && (e[1].s == "add" || e[1].s == "sub" || e[1].s == "mul")) {
    std::string a, b;
    if (!gen_int(g, e[2], &a) || !gen_int(g, e[3], &b)) return false;
    // int32 arithmetic wraps, as in the Native backend
    *out = "((long long)(int)(" + a + (e[1].s == "add" ? " + " : e[1].s == "sub" ? " - " : " * ") + b + "))";
    return true;
  }
  g.why = "unsupported integer expression";
  return false;
}

std::string generic_map_source(const KernelPlan& plan, const GenericMap& gm, const std::vector<std::string>& store_exprs) {
  const size_t ni = gm.inputs.size(), no = gm.outputs.size(), ns = gm.scalars.size();
  auto scalar_type = [&](size_t i) {
    const std::string& elt = plan.params[gm.scalars[i]].elt;
    return (elt == "f32" || elt == "f64") ? "double" : "long long";
  };
  std::ostringstream o;
  o << "// generated for kernel '" << plan.name << "'\n";
  o << "__device__ __forceinline__ void sb200_elem(";
  for (size_t i = 0; i < ni; ++i) o << "float x" << i << ", ";
  for (size_t i = 0; i < ns; ++i) o << scalar_type(i) << " s" << i << ", ";
  for (size_t i = 0; i < no; ++i) o << "float& y" << i << (i + 1 < no ? ", " : "");
  o << ") {\n";
  for (size_t i = 0; i < ni; ++i) o << "  const double X" << i << " = (double)x" << i << ";\n";
  for (size_t i = 0; i < no; ++i) o << "  const float t" << i << " = (float)(" << store_exprs[i] << ");\n  y" << i << " = t" << i << ";\n";
  o << "}\n";
  // vector kernel, one launch for any n: after `head` (0..3) single elements every operand is 16-byte aligned and
  // nvec whole vectors follow; the ragged ends (head, and up to 3 elements after the vectors) are taken by the
  // first threads of block 0
  o << "extern \"C\" __global__ void __launch_bounds__(256) sb200_map_vec(";
  for (size_t i = 0; i < ni; ++i) o << "const float* __restrict__ sin" << i << ", ";
  for (size_t i = 0; i < no; ++i) o << "float* __restrict__ sout" << i << ", ";
  for (size_t i = 0; i < ns; ++i) o << scalar_type(i) << " s" << i << ", ";
  o << "int head, long long nvec, long long n) {\n";
  o << "  if (blockIdx.x == 0) {\n";
  o << "    const long long body_end = head + nvec * 4;\n";
  o << "    const int ragged = head + (int)(n - body_end);\n";
  o << "    if ((int)threadIdx.x < ragged) {\n";
  o << "      const long long e = (int)threadIdx.x < head ? (long long)threadIdx.x : body_end + ((int)threadIdx.x - head);\n";
  for (size_t i = 0; i < no; ++i) o << "      float r" << i << ";\n";
  o << "      sb200_elem(";
  for (size_t i = 0; i < ni; ++i) o << "sin" << i << "[e], ";
  for (size_t i = 0; i < ns; ++i) o << "s" << i << ", ";
  for (size_t i = 0; i < no; ++i) o << "r" << i << (i + 1 < no ? ", " : "");
  o << ");\n";
  for (size_t i = 0; i < no; ++i) o << "      sout" << i << "[e] = r" << i << ";\n";
  o << "    }\n  }\n";
  for (size_t i = 0; i < ni; ++i) o << "  const float4* __restrict__ in" << i << " = reinterpret_cast<const float4*>(sin" << i << " + head);\n";
  for (size_t i = 0; i < no; ++i) o << "  float4* __restrict__ out" << i << " = reinterpret_cast<float4*>(sout" << i << " + head);\n";
  o << "  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {\n";
  for (size_t i = 0; i < ni; ++i) o << "    const float4 a" << i << " = in" << i << "[v];\n";
  for (size_t i = 0; i < no; ++i) o << "    float4 r" << i << ";\n";
  for (const char* c : {"x", "y", "z", "w"}) {
    o << "    sb200_elem(";
    for (size_t i = 0; i < ni; ++i) o << "a" << i << "." << c << ", ";
    for (size_t i = 0; i < ns; ++i) o << "s" << i << ", ";
    for (size_t i = 0; i < no; ++i) o << "r" << i << "." << c << (i + 1 < no ? ", " : "");
    o << ");\n";
  }
  for (size_t i = 0; i < no; ++i) o << "    out" << i << "[v] = r" << i << ";\n";
  o << "  }\n}\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) sb200_map_scalar(";
  for (size_t i = 0; i < ni; ++i) o << "const float* __restrict__ in" << i << ", ";
  for (size_t i = 0; i < no; ++i) o << "float* __restrict__ out" << i << ", ";
  for (size_t i = 0; i < ns; ++i) o << scalar_type(i) << " s" << i << ", ";
  o << "long long first, long long n) {\n";
  o << "  for (long long e = first + blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {\n";
  for (size_t i = 0; i < no; ++i) o << "    float r" << i << ";\n";
  o << "    sb200_elem(";
  for (size_t i = 0; i < ni; ++i) o << "in" << i << "[e], ";
  for (size_t i = 0; i < ns; ++i) o << "s" << i << ", ";
  for (size_t i = 0; i < no; ++i) o << "r" << i << (i + 1 < no ? ", " : "");
  o << ");\n";
  for (size_t i = 0; i < no; ++i) o << "    out" << i << "[e] = r" << i << ";\n";
  o << "  }\n}\n";
  return o.str();
}

bool match_map_generic(Ctx& cx, const Sx& body) {
  KernelPlan& plan = *cx.plan;
  Peeled pl;
  peel(body, &pl, true);
  if (!pl.shared.empty()) {
    cx.why = "uses shared arrays";
    return false;
  }
  std::vector<const Sx*> items = seq_items(*pl.core);
  if (items.empty() || items.size() > 8) {
    cx.why = "body is not one to eight element stores";
    return false;
  }
  MapPlan mp;
  GenericMap gm;
  Sx idx;
  bool have_idx = false;
  for (const Sx* it : items) {
    if (!it->is("assign") || it->size() != 3 || !(*it)[1].is("elem") || (*it)[1].size() != 3) {
      cx.why = "statement is not an array element store";
      return false;
    }
    Sx this_idx = inline_expr((*it)[1][2], pl.env);
    if (!have_idx) {
      idx = this_idx;
      have_idx = true;
    } else if (!sx_equal(idx, this_idx)) {
      cx.why = "stores use different indices";
      return false;
    }
  }
  if (is_global_x(idx)) {
    mp.index_kind = IDX_GLOBAL;
  } else if (is_intrinsic(idx, "thread_idx_x")) {
    mp.index_kind = IDX_THREAD_X;
  } else {
    cx.why = "element index is not the global or block-local x thread index";
    return false;
  }
  if (pl.guards.size() > 1) {
    cx.why = "more than one guard";
    return false;
  }
  if (pl.guards.size() == 1) {
    const Sx *l, *r;
    if (!is_binop(pl.guards[0], "lt", &l, &r) || !sx_equal(*l, idx) || (mp.n_param = cx.scalar_param(*r, "i32")) < 0) {
      cx.why = "guard is not `index < n` with n an int32 parameter";
      return false;
    }
  }
  GenCtx g{&cx, &idx, &gm, {}, ""};
  std::vector<std::string> exprs;
  for (const Sx* it : items) {
    const std::string& arr = (*it)[1][1].s;
    int out = cx.vec_param(arr, "f32");
    if (out < 0) {
      cx.why = "store target " + arr + " is not a float32 vector parameter";
      return false;
    }
    for (int prev : gm.outputs)
      if (prev == out) {
        cx.why = "vector " + arr + " is stored twice";
        return false;
      }
    std::string code;
    if (!gen_float(g, inline_expr((*it)[2], pl.env), &code)) {
      cx.why = g.why;
      return false;
    }
    exprs.push_back(code);
    g.stored[arr] = "t" + std::to_string(gm.outputs.size());
    gm.outputs.push_back(out);
  }
  // an input that is also an output is read before it is written by the same thread: allowed
  gm.source = generic_map_source(plan, gm, exprs);
  mp.op = OP_GENERIC;
  mp.out0 = gm.outputs[0];
  plan.kind = KIND_MAP;
  plan.map = mp;
  plan.generic = gm;
  plan.description = "map:generic(jit) inputs=" + std::to_string(gm.inputs.size()) + " outputs=" + std::to_string(gm.outputs.size()) +
                     " scalars=" + std::to_string(gm.scalars.size()) + (mp.n_param >= 0 ? " guarded" : " unguarded") +
                     (mp.index_kind == IDX_GLOBAL ? " idx=global_x" : " idx=thread_idx_x");
  return true;
}

void walk(const Sx& s, Env env, const std::function<void(const Sx&, const Env&)>& f);

// ------------------------------------------------------- block tree reduction
// The shape of benchmarks/bench_reduction.ml:62-105 and bench_dot_product.ml:17-57:
//   sdata[tid] <- (gid < n ? f(a[gid], ...) : 0);  barrier
//   for c = B/2 ... 1:  if tid < c then sdata[tid] <- sdata[tid] + sdata[tid + c];  barrier
//   if tid = 0 then out[block_idx_x] <- sdata[0]
std::string block_reduce_source(const KernelPlan& plan, const GenericMap& gm, const std::string& expr, int block) {
  const size_t ni = gm.inputs.size(), ns = gm.scalars.size();
  auto scalar_type = [&](size_t i) {
    const std::string& elt = plan.params[gm.scalars[i]].elt;
    return (elt == "f32" || elt == "f64") ? "double" : "long long";
  };
  std::ostringstream o;
  o << "// generated for kernel '" << plan.name << "' (block tree reduction, block = " << block << ")\n";
  o << "__device__ __forceinline__ double sb200_elem(";
  for (size_t i = 0; i < ni; ++i) o << "float x" << i << (i + 1 < ni || ns ? ", " : "");
  for (size_t i = 0; i < ns; ++i) o << scalar_type(i) << " s" << i << (i + 1 < ns ? ", " : "");
  o << ") {\n";
  for (size_t i = 0; i < ni; ++i) o << "  const double X" << i << " = (double)x" << i << ";\n";
  o << "  return " << expr << ";\n}\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) sb200_reduce(";
  for (size_t i = 0; i < ni; ++i) o << "const float* __restrict__ in" << i << ", ";
  o << "float* __restrict__ out, ";
  for (size_t i = 0; i < ns; ++i) o << scalar_type(i) << " s" << i << ", ";
  o << "long long n, long long nseg) {\n";
  o << "  constexpr int B = " << block << ", PER = B / 32;\n";
  o << "  const int lane = threadIdx.x & 31;\n";
  o << "  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;\n";
  o << "  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;\n";
  o << "  for (long long seg = warp; seg < nseg; seg += nwarps) {\n";
  o << "    double v[PER];\n";
  o << "#pragma unroll\n    for (int j = 0; j < PER; ++j) {\n";
  o << "      const long long g = seg * B + lane + 32 * j;\n";
  o << "      v[j] = g < n ? sb200_elem(";
  for (size_t i = 0; i < ni; ++i) o << "in" << i << "[g]" << (i + 1 < ni || ns ? ", " : "");
  for (size_t i = 0; i < ns; ++i) o << "s" << i << (i + 1 < ns ? ", " : "");
  o << ") : 0.0;\n    }\n";
  // strides B/2 ... 32 pair registers of one lane; strides 16 ... 1 pair lanes: the reference's tree order
  o << "#pragma unroll\n    for (int h = PER / 2; h >= 1; h >>= 1)\n";
  o << "#pragma unroll\n      for (int j = 0; j < h; ++j) v[j] = __dadd_rn(v[j], v[j + h]);\n";
  o << "    double r = v[0];\n";
  o << "#pragma unroll\n    for (int c = 16; c >= 1; c >>= 1) r = __dadd_rn(r, __shfl_down_sync(0xffffffffu, r, c));\n";
  o << "    if (lane == 0) out[seg] = (float)r;\n";
  o << "  }\n}\n";
  return o.str();
}

bool match_block_reduce(Ctx& cx, const Sx& body) {
  KernelPlan& plan = *cx.plan;
  Peeled pl;
  peel(body, &pl, false);
  if (pl.shared.size() != 1) return false;
  const std::string S = *pl.shared.begin();
  auto strip = [](const Sx* s) {
    while ((s->is("block") && s->size() == 2) || (s->is("seq") && s->size() == 2)) s = &(*s)[1];
    return s;
  };
  auto is_tid = [](const Sx& e) { return is_intrinsic(e, "thread_idx_x"); };
  std::set<const Sx*> handled;
  std::vector<long long> steps;
  int barriers = 0, out = -1, n_param = -1;
  bool bad = false, have_load = false, have_final = false;
  Sx load_expr, gid;
  std::string why;
  walk(*pl.core, pl.env, [&](const Sx& s, const Env& env) {
    if (bad) return;
    if (s.is("barrier")) ++barriers;
    if (s.is("for") || s.is("while") || s.is("letmut")) {
      bad = true;
      why = "loops are not part of the block-reduction shape";
      return;
    }
    if (s.is("sif") && s.size() >= 3) {
      const Sx cond = inline_expr(s[1], env);
      const Sx* th = strip(&s[2]);
      const Sx* el = s.size() == 4 ? strip(&s[3]) : nullptr;
      const Sx *l, *r;
      if (!th->is("assign") || th->size() != 3 || !(*th)[1].is("elem")) return;
      const Sx& lv = (*th)[1];
      const Sx lidx = inline_expr(lv[2], env);
      const Sx rhs = inline_expr((*th)[2], env);
      if (lv[1].s == S && is_tid(lidx)) {
        if (el) {  // load step
          if (have_load || !is_binop(cond, "lt", &l, &r) || !is_global_x(*l) || cx.scalar_param(*r, "i32") < 0 ||
              !el->is("assign") || !(*el)[1].is("elem") || (*el)[1][1].s != S || !is_tid(inline_expr((*el)[1][2], env)) ||
              !is_const_f_zero(inline_expr((*el)[2], env))) {
            bad = true;
            why = "load step is not `if gid < n then s[tid] <- f(...) else s[tid] <- 0.0`";
            return;
          }
          have_load = true;
          n_param = cx.scalar_param(*r, "i32");
          gid = *l;
          load_expr = rhs;
          handled.insert(th);
          handled.insert(el);
        } else {  // tree step: if tid < c then s[tid] <- s[tid] + s[tid + c]
          long long c = -1;
          if (is_binop(cond, "lt", &l, &r) && is_tid(*l) && r->is("const")) c = atoll((*r)[2].s.c_str());
          bool ok = c > 0 && is_comm(rhs, "add", [&](const Sx& a, const Sx& b) {
                      if (!a.is("read") || a[1].s != S || !is_tid(a[2])) return false;
                      if (!b.is("read") || b[1].s != S) return false;
                      return is_comm(b[2], "add", [&](const Sx& p, const Sx& q) { return is_tid(p) && is_const_i32(q, c); });
                    });
          if (!ok) {
            bad = true;
            why = "reduction step is not `if tid < c then s[tid] <- s[tid] + s[tid + c]`";
            return;
          }
          steps.push_back(c);
          handled.insert(th);
        }
      } else if (lv[1].s != S) {  // final store
        if (have_final || el || !is_binop(cond, "eq", &l, &r) || !is_tid(*l) || !is_const_i32(*r, 0) ||
            !is_intrinsic(lidx, "block_idx_x") || !rhs.is("read") || rhs[1].s != S || !is_const_i32(rhs[2], 0) ||
            (out = cx.vec_param(lv[1].s, "f32")) < 0) {
          bad = true;
          why = "final store is not `if tid = 0 then out[block_idx_x] <- s[0]`";
          return;
        }
        have_final = true;
        handled.insert(th);
      }
    }
    if (s.is("assign") && s.size() == 3 && s[1].is("elem") && !handled.count(&s)) {
      bad = true;
      why = "store outside the load / tree / final steps";
    }
  });
  if (bad || !have_load || !have_final || steps.empty()) {
    if (!why.empty()) cx.why = why;
    return false;
  }
  const long long B = steps[0] * 2;
  {
    // the shared array must hold the block's B partial sums
    const Sx* q = &body;
    long long size = -1;
    while ((q->is("let") || q->is("letmut")) && q->size() == 6) {
      if (is_shared_let(*q) && (*q)[1].s == S && (*q)[4].size() == 4 && (*q)[4][2].is("const") && (*q)[4][2].size() == 3)
        size = atoll((*q)[4][2][2].s.c_str());
      q = &(*q)[5];
    }
    if (size < B) {
      cx.why = "shared array is shorter than the block the tree steps imply";
      return false;
    }
  }
  bool pow2 = B >= 32 && B <= 1024 && (B & (B - 1)) == 0;
  for (size_t i = 0; i < steps.size() && pow2; ++i)
    if (steps[i] != (B >> (i + 1))) pow2 = false;
  if (!pow2 || steps.back() != 1 || barriers < static_cast<int>(steps.size())) {
    cx.why = "tree steps are not B/2, B/4, ..., 1 for a power-of-two block size of 32 to 1024";
    return false;
  }
  GenericMap gm;
  GenCtx g{&cx, &gid, &gm, {}, ""};
  std::string code;
  if (!gen_float(g, load_expr, &code)) {
    cx.why = g.why;
    return false;
  }
  gm.outputs.push_back(out);
  gm.source = block_reduce_source(plan, gm, code, static_cast<int>(B));
  plan.kind = KIND_BLOCK_REDUCE;
  plan.generic = gm;
  plan.reduce.n_param = n_param;
  plan.reduce.block = static_cast<int>(B);
  plan.description = "reduce:block_tree(jit) block=" + std::to_string(B) + " inputs=" + std::to_string(gm.inputs.size()) +
                     " out=" + plan.params[out].name;
  return true;
}

// ------------------------------------------------------------------- GEMM

// relu wrapper: (if (binop gt X (const f32 0)) X (const f32 0))
const Sx* strip_relu(const Sx& e, int* act) {
  *act = 0;
  if (e.is("if") && e.size() == 4) {
    const Sx *l, *r;
    if (is_binop(e[1], "gt", &l, &r) && is_const_f_zero(*r) && sx_equal(*l, e[2]) && is_const_f_zero(e[3])) {
      *act = 1;
      return &e[2];
    }
  }
  return &e;
}

void flatten_add(const Sx& e, std::vector<const Sx*>* terms) {
  const Sx *l, *r;
  if (is_binop(e, "add", &l, &r)) {
    flatten_add(*l, terms);
    flatten_add(*r, terms);
  } else {
    terms->push_back(&e);
  }
}

// EPI(acc) = act(alpha*acc + beta*C[row*n+col] + bias[col]); every read index
// is compared after let-inlining.
bool match_epilogue(Ctx& cx, const Sx& e_in, const std::string& acc_id, const Sx& out_idx, const Sx& col, GemmPlan* g) {
  int act;
  const Sx* e = strip_relu(e_in, &act);
  g->act = act;
  g->alpha.param = -1;
  g->alpha.value = 1.0;
  g->beta.param = -1;
  g->beta.value = 0.0;
  std::vector<const Sx*> terms;
  flatten_add(*e, &terms);
  bool have_acc = false;
  auto is_acc = [&](const Sx& x) { return x.is("evar") && x.size() >= 3 && x[2].s == acc_id; };
  for (const Sx* t : terms) {
    const Sx* idx;
    int prm;
    Coef cf;
    if (is_acc(*t)) {
      if (have_acc) return false;
      have_acc = true;
    } else if (is_comm(*t, "mul", [&](const Sx& a, const Sx& b) { return cx.is_coef(a, &cf) && is_acc(b); })) {
      if (have_acc) return false;
      have_acc = true;
      g->alpha = cf;
    } else if (cx.is_read(*t, &prm, &idx)) {
      if (sx_equal(*idx, out_idx) && g->c < 0) {
        g->c = prm;
        g->beta.param = -1;
        g->beta.value = 1.0;
      } else if (sx_equal(*idx, col) && g->bias < 0) {
        g->bias = prm;
      } else {
        return false;
      }
    } else if (is_comm(*t, "mul", [&](const Sx& a, const Sx& b) {
                 return cx.is_coef(a, &cf) && cx.is_read(b, &prm, &idx) && sx_equal(*idx, out_idx);
               })) {
      if (g->c >= 0) return false;
      g->c = prm;
      g->beta = cf;
    } else {
      return false;
    }
  }
  return have_acc;
}

bool match_guard_mn(Ctx& cx, const Sx& guard, const Sx& row, const Sx& col, GemmPlan* g) {
  return is_comm(guard, "and", [&](const Sx& a, const Sx& b) {
    const Sx *l, *r;
    if (!is_binop(a, "lt", &l, &r) || !sx_equal(*l, row)) return false;
    int m = cx.scalar_param(*r, "i32");
    if (!is_binop(b, "lt", &l, &r) || !sx_equal(*l, col)) return false;
    int n = cx.scalar_param(*r, "i32");
    if (m < 0 || n < 0) return false;
    g->m = m;
    g->n = n;
    return true;
  });
}

// acc := acc + X*Y ; returns X and Y (not inlined)
bool match_accumulate(const Sx& s, std::string* acc_id, const Sx** x, const Sx** y) {
  if (!s.is("assign") || s.size() != 3 || !s[1].is("lvar") || s[1].size() < 3) return false;
  const std::string id = s[1][2].s;
  const Sx& rhs = s[2];
  bool ok = is_comm(rhs, "add", [&](const Sx& a, const Sx& b) {
    const Sx *m0, *m1;
    if (!a.is("evar") || a.size() < 3 || a[2].s != id) return false;
    if (!is_binop(b, "mul", &m0, &m1)) return false;
    *x = m0;
    *y = m1;
    return true;
  });
  if (ok) *acc_id = id;
  return ok;
}

// upper bound `k - 1` of an inclusive upto loop starting at 0
bool loop_0_to_km1(const Sx& f, const Env& env, Sx* k_expr) {
  if (!f.is("for") || f.size() != 7 || f[5].s != "upto") return false;
  if (!is_const_i32(inline_expr(f[3], env), 0)) return false;
  Sx hi = inline_expr(f[4], env);
  const Sx *l, *r;
  if (!is_binop(hi, "sub", &l, &r) || !is_const_i32(*r, 1)) return false;
  *k_expr = *l;
  return true;
}

bool match_gemm_naive(Ctx& cx, const Sx& body) {
  KernelPlan& plan = *cx.plan;
  Peeled pl;
  peel(body, &pl, true);
  if (!pl.shared.empty() || pl.guards.size() != 1) return false;
  const Sx& core = *pl.core;
  if (!core.is("letmut") || core.size() != 6 || !is_const_f_zero(inline_expr(core[4], pl.env))) return false;
  const std::string acc_id = core[2].s;
  std::vector<const Sx*> items = seq_items(core[5]);
  if (items.size() != 2) return false;
  const Sx& loop = *items[0];
  Sx k_expr;
  if (!loop_0_to_km1(loop, pl.env, &k_expr)) return false;
  GemmPlan g;
  g.k = cx.scalar_param(k_expr, "i32");
  if (g.k < 0) return false;
  const std::string loop_id = loop[2].s;
  Peeled lp;
  lp.env = pl.env;
  peel(loop[6], &lp, false);
  std::string aid;
  const Sx *x, *y;
  if (!match_accumulate(*lp.core, &aid, &x, &y) || aid != acc_id) return false;
  Sx xa = inline_expr(*x, lp.env), yb = inline_expr(*y, lp.env);
  const Sx *ia, *ib;
  if (!cx.is_read(xa, &g.a, &ia) || !cx.is_read(yb, &g.b, &ib)) return false;
  auto is_loop_var = [&](const Sx& e) { return e.is("evar") && e.size() >= 3 && e[2].s == loop_id; };
  // A index: row*k + i ; B index: i*n + col
  Sx row, col;
  int kk = -1, nn = -1;
  bool ok_a = is_comm(*ia, "add", [&](const Sx& p, const Sx& q) {
    return is_loop_var(q) && is_comm(p, "mul", [&](const Sx& r, const Sx& s) {
             int kp = cx.scalar_param(s, "i32");
             if (kp < 0) return false;
             kk = kp;
             row = r;
             return true;
           });
  });
  bool ok_b = is_comm(*ib, "add", [&](const Sx& p, const Sx& q) {
    return is_comm(p, "mul", [&](const Sx& r, const Sx& s) {
             int np = cx.scalar_param(s, "i32");
             if (!is_loop_var(r) || np < 0) return false;
             nn = np;
             col = q;
             return true;
           });
  });
  if (!ok_a || !ok_b || kk != g.k) {
    cx.why = "operand indices are not a[row*k+i] and b[i*n+col]";
    return false;
  }
  // row = tid / n, col = tid mod n
  const Sx *l, *r;
  if (!is_binop(row, "div", &l, &r) || !is_global_x(*l) || cx.scalar_param(*r, "i32") != nn) return false;
  if (!is_binop(col, "mod", &l, &r) || !is_global_x(*l) || cx.scalar_param(*r, "i32") != nn) return false;
  if (!match_guard_mn(cx, pl.guards[0], row, col, &g) || g.n != nn) {
    cx.why = "guard is not row < m && col < n";
    return false;
  }
  // final store d[row*n+col] <- EPI(acc)
  const Sx& st = *items[1];
  if (!st.is("assign") || st.size() != 3 || !st[1].is("elem")) return false;
  g.d = cx.vec_param(st[1][1].s, "f32");
  Sx out_idx = inline_expr(st[1][2], pl.env);
  bool ok_o = is_comm(out_idx, "add", [&](const Sx& p, const Sx& q) {
    return sx_equal(q, col) && is_comm(p, "mul", [&](const Sx& rr, const Sx& ss) {
             return sx_equal(rr, row) && cx.scalar_param(ss, "i32") == nn;
           });
  });
  if (g.d < 0 || !ok_o) {
    cx.why = "result is not stored at d[row*n+col]";
    return false;
  }
  if (!match_epilogue(cx, inline_expr(st[2], pl.env), acc_id, out_idx, col, &g)) {
    cx.why = "stored expression is not act(alpha*sum + beta*c[row*n+col] + bias[col])";
    return false;
  }
  plan.kind = KIND_GEMM_NAIVE;
  plan.gemm = g;
  return true;
}

// Walk every statement under `s`, carrying the let environment.
void walk(const Sx& s, Env env, const std::function<void(const Sx&, const Env&)>& f) {
  if (s.atom) return;
  f(s, env);
  if (s.is("let") && s.size() == 6) {
    if (!is_shared_let(s)) env[s[2].s] = inline_expr(s[4], env);
    walk(s[5], env, f);
  } else if (s.is("letmut") && s.size() == 6) {
    walk(s[5], env, f);
  } else if (s.is("seq")) {
    for (size_t i = 1; i < s.size(); ++i) walk(s[i], env, f);
  } else if (s.is("sif")) {
    for (size_t i = 2; i < s.size(); ++i) walk(s[i], env, f);
  } else if (s.is("for") && s.size() == 7) {
    walk(s[6], env, f);
  } else if (s.is("block") && s.size() == 2) {
    walk(s[1], env, f);
  } else if (s.is("pragma") && s.size() == 3) {
    walk(s[2], env, f);
  } else if (s.is("while") && s.size() == 3) {
    walk(s[2], env, f);
  }
}

// ---- integer index expressions as polynomials ----------------------------------------------
// Index arithmetic can be written in many equivalent ways (operands commuted, products distributed, the
// global index spelt out or taken from an intrinsic).  The tiled-kernel recogniser therefore compares
// index expressions as polynomials with integer coefficients over opaque atoms: scalar parameters,
// thread/block intrinsics, loop variables, and whole div/mod sub-expressions.
using Mono = std::vector<std::string>;  // sorted atom names; empty = the constant term
using Poly = std::map<Mono, long long>;

Poly poly_const(long long c) {
  Poly p;
  if (c) p[Mono{}] = c;
  return p;
}
Poly poly_atom(const std::string& a) {
  Poly p;
  p[Mono{a}] = 1;
  return p;
}
Poly poly_add(const Poly& a, const Poly& b, long long sign = 1) {
  Poly r = a;
  for (const auto& kv : b) {
    long long& c = r[kv.first];
    c += sign * kv.second;
    if (c == 0) r.erase(kv.first);
  }
  return r;
}
Poly poly_mul(const Poly& a, const Poly& b) {
  Poly r;
  for (const auto& x : a)
    for (const auto& y : b) {
      Mono m = x.first;
      m.insert(m.end(), y.first.begin(), y.first.end());
      std::sort(m.begin(), m.end());
      long long& c = r[m];
      c += x.second * y.second;
      if (c == 0) r.erase(m);
    }
  return r;
}
std::string poly_print(const Poly& p) {
  std::string o;
  for (const auto& kv : p) {
    o += (kv.second >= 0 ? "+" : "") + std::to_string(kv.second);
    for (const std::string& a : kv.first) o += "*" + a;
  }
  return o.empty() ? "0" : o;
}

// e must already have its lets inlined.  False for anything that is not integer index arithmetic.
bool poly_of(const Ctx& cx, const Sx& e, Poly* out) {
  if (e.is("const") && e.size() == 3 && (e[1].s == "i32" || e[1].s == "i64")) {
    *out = poly_const(atoll(e[2].s.c_str()));
    return true;
  }
  if (e.is("evar") && e.size() == 3) {
    const int prm = cx.scalar_param(e, nullptr);
    *out = poly_atom(prm >= 0 ? "p" + std::to_string(prm) : "v" + e[2].s);
    return true;
  }
  if (e.is("intrinsic") && e.size() == 3) {
    const std::string& n = e[2].s;
    auto global = [](const char* t, const char* bd, const char* bi) {
      return poly_add(poly_atom(t), poly_mul(poly_atom(bd), poly_atom(bi)));
    };
    if (n == "global_idx_x" || n == "global_thread_id") {
      *out = global("i:thread_idx_x", "i:block_dim_x", "i:block_idx_x");
    } else if (n == "global_idx_y") {
      *out = global("i:thread_idx_y", "i:block_dim_y", "i:block_idx_y");
    } else {
      *out = poly_atom("i:" + n);
    }
    return true;
  }
  if (e.is("binop") && e.size() == 4) {
    Poly l, r;
    if (!poly_of(cx, e[2], &l) || !poly_of(cx, e[3], &r)) return false;
    const std::string& op = e[1].s;
    if (op == "add") *out = poly_add(l, r);
    else if (op == "sub") *out = poly_add(l, r, -1);
    else if (op == "mul") *out = poly_mul(l, r);
    else if (op == "div" || op == "mod") *out = poly_atom(op + "(" + poly_print(l) + "|" + poly_print(r) + ")");
    else return false;
    return true;
  }
  return false;
}

bool poly_is(const Ctx& cx, const Sx& e, const Poly& want) {
  Poly got;
  return poly_of(cx, e, &got) && got == want;
}

// cond is (l1 < r1) && (l2 < r2), either order, with the given polynomials
bool guard_is(const Ctx& cx, const Sx& cond, const Poly& l1, const Poly& r1, const Poly& l2, const Poly& r2) {
  return is_comm(cond, "and", [&](const Sx& a, const Sx& b) {
    const Sx *al, *ar, *bl, *br;
    return is_binop(a, "lt", &al, &ar) && is_binop(b, "lt", &bl, &br) && poly_is(cx, *al, l1) && poly_is(cx, *ar, r1) &&
           poly_is(cx, *bl, l2) && poly_is(cx, *br, r2);
  });
}

// The tiled kernel of benchmarks/bench_matrix_mul_tiled.ml:55-94, checked statement by statement:
//   shared tile_a[T*T], tile_b[T*T];  sum := 0
//   for t = 0 .. (k+T-1)/T - 1:
//     tile_a[ty*T+tx] <- (row < m && t*T+tx < k) ? a[row*k + t*T+tx] : 0        barrier
//     tile_b[ty*T+tx] <- (t*T+ty < k && col < n) ? b[(t*T+ty)*n + col] : 0      barrier
//     for i = 0 .. T-1: sum := sum + tile_a[ty*T+i] * tile_b[i*T+tx]            barrier
//   if row < m && col < n then out[row*n+col] <- epilogue(sum)
// with row / col the global y / x indices and tx / ty the thread indices.  Index expressions are compared as
// polynomials, so any equivalent spelling is accepted and nothing else is.
bool match_gemm_tiled(Ctx& cx, const Sx& body) {
  KernelPlan& plan = *cx.plan;
  Peeled pl;
  peel(body, &pl, false);
  if (pl.shared.size() != 2) return false;
  const Sx& core = *pl.core;
  if (!core.is("letmut") || core.size() != 6 || !is_const_f_zero(inline_expr(core[4], pl.env))) return false;
  const std::string acc_id = core[2].s;
  std::vector<const Sx*> items = seq_items(core[5]);
  if (items.size() != 2 || !items[0]->is("for") || items[0]->size() != 7 || (*items[0])[5].s != "upto") return false;
  const Sx& outer = *items[0];
  GemmPlan g;

  // final guarded store: gives row, col, m, n and the output
  Peeled fin;
  fin.env = pl.env;
  peel(*items[1], &fin, true);
  if (fin.guards.size() != 1 || !fin.core->is("assign") || !(*fin.core)[1].is("elem")) return false;
  const Sx& st = *fin.core;
  g.d = cx.vec_param(st[1][1].s, "f32");
  Sx out_idx = inline_expr(st[1][2], fin.env);
  Sx row, col;
  int nn = -1;
  bool ok_o = is_comm(out_idx, "add", [&](const Sx& p, const Sx& q) {
    return is_comm(p, "mul", [&](const Sx& rr, const Sx& ss) {
      int np = cx.scalar_param(ss, "i32");
      if (np < 0) return false;
      nn = np;
      row = rr;
      col = q;
      return true;
    });
  });
  if (g.d < 0 || !ok_o || !is_global_y(row) || !is_global_x(col)) {
    cx.why = "result is not stored at c[row*n+col] with row/col the global y/x indices";
    return false;
  }
  if (!match_guard_mn(cx, fin.guards[0], row, col, &g) || g.n != nn) return false;

  // the statements of one k-tile iteration, in order
  std::vector<const Sx*> steps;
  std::function<void(const Sx&)> flat = [&](const Sx& s) {
    if (s.is("seq")) {
      for (size_t i = 1; i < s.size(); ++i) flat(s[i]);
    } else if (s.is("block") && s.size() == 2) {
      flat(s[1]);
    } else if (!s.is("empty")) {
      steps.push_back(&s);
    }
  };
  flat(outer[6]);
  // a load may be wrapped in lets (a_col, b_row): peel them into an environment of its own
  struct Step {
    char kind;  // 'L' load, 'B' barrier, 'C' compute
    const Sx* core;
    Env env;
  };
  std::vector<Step> seq;
  for (const Sx* sp : steps) {
    if (sp->is("barrier")) {
      seq.push_back({'B', sp, pl.env});
      continue;
    }
    Peeled one;
    one.env = pl.env;
    peel(*sp, &one, false);
    if (!one.shared.empty()) return false;
    if (one.core->is("sif") && one.core->size() == 4) seq.push_back({'L', one.core, one.env});
    else if (one.core->is("for") && one.core->size() == 7) seq.push_back({'C', one.core, one.env});
    else {
      cx.why = "k-tile loop holds a statement that is neither a tile load, a barrier nor the inner product loop";
      return false;
    }
  }
  std::string shape;
  for (const Step& x : seq) shape += x.kind;
  if (shape != "LBLBCB" && shape != "LLBCB") {
    cx.why = "k-tile loop is not load, barrier, load, barrier, accumulate, barrier";
    return false;
  }
  std::vector<const Step*> loads;
  const Step* comp = nullptr;
  for (const Step& x : seq) {
    if (x.kind == 'L') loads.push_back(&x);
    if (x.kind == 'C') comp = &x;
  }

  // inner product loop: tile size, tile names
  const Sx& inner = *comp->core;
  if (inner[5].s != "upto" || !is_const_i32(inline_expr(inner[3], comp->env), 0)) return false;
  Poly hi_poly;
  if (!poly_of(cx, inline_expr(inner[4], comp->env), &hi_poly) || hi_poly.size() != 1 || !hi_poly.count(Mono{})) {
    cx.why = "inner loop bound is not a constant tile size";
    return false;
  }
  const long long T = hi_poly[Mono{}] + 1;
  if (T < 1 || T > 32) return false;
  const Poly TX = poly_atom("i:thread_idx_x"), TY = poly_atom("i:thread_idx_y"), PT = poly_const(T);
  Poly ROW, COL;
  if (!poly_of(cx, row, &ROW) || !poly_of(cx, col, &COL)) return false;
  const Poly IV = poly_atom("v" + inner[2].s), TV = poly_atom("v" + outer[2].s);
  std::string aid, tile_a, tile_b;
  {
    const Sx* acc_stmt = &inner[6];
    while ((acc_stmt->is("block") && acc_stmt->size() == 2) || (acc_stmt->is("seq") && acc_stmt->size() == 2)) acc_stmt = &(*acc_stmt)[1];
    const Sx *x, *y;
    if (!match_accumulate(*acc_stmt, &aid, &x, &y) || aid != acc_id) {
      cx.why = "inner loop body is not sum := sum + tile_a[..] * tile_b[..]";
      return false;
    }
    const Sx xi = inline_expr(*x, comp->env), yi = inline_expr(*y, comp->env);
    if (!xi.is("read") || !yi.is("read") || !pl.shared.count(xi[1].s) || !pl.shared.count(yi[1].s) || xi[1].s == yi[1].s) return false;
    const Poly want_a = poly_add(poly_mul(TY, PT), IV), want_b = poly_add(poly_mul(IV, PT), TX);
    if (poly_is(cx, xi[2], want_a) && poly_is(cx, yi[2], want_b)) {
      tile_a = xi[1].s;
      tile_b = yi[1].s;
    } else if (poly_is(cx, yi[2], want_a) && poly_is(cx, xi[2], want_b)) {
      tile_a = yi[1].s;
      tile_b = xi[1].s;
    } else {
      cx.why = "inner product does not read tile_a[ty*T+i] and tile_b[i*T+tx]";
      return false;
    }
  }
  // shared tiles hold T*T floats
  {
    const Sx* s = &body;
    int sized = 0;
    while ((s->is("let") || s->is("letmut")) && s->size() == 6) {
      if (is_shared_let(*s)) {
        const Sx& ac = (*s)[4];
        if (ac.size() != 4 || !is_const_i32(ac[2], T * T)) {
          cx.why = "shared tiles are not tile_size*tile_size long";
          return false;
        }
        ++sized;
      }
      s = &(*s)[5];
    }
    if (sized != 2) return false;
  }
  // the two loads
  const Poly tile_idx = poly_add(poly_mul(TY, PT), TX);
  const Poly M_ = poly_atom("p" + std::to_string(g.m)), N_ = poly_atom("p" + std::to_string(g.n));
  for (const Step* ld : loads) {
    const Sx& sif = *ld->core;
    const Sx cond = inline_expr(sif[1], ld->env);
    const Sx* th = &sif[2];
    const Sx* el = &sif[3];
    auto strip = [](const Sx* q) {
      while ((q->is("block") && q->size() == 2) || (q->is("seq") && q->size() == 2)) q = &(*q)[1];
      return q;
    };
    th = strip(th);
    el = strip(el);
    if (!th->is("assign") || !el->is("assign") || !(*th)[1].is("elem") || !(*el)[1].is("elem") || (*th)[1][1].s != (*el)[1][1].s ||
        !poly_is(cx, inline_expr((*th)[1][2], ld->env), tile_idx) || !poly_is(cx, inline_expr((*el)[1][2], ld->env), tile_idx) ||
        !is_const_f_zero(inline_expr((*el)[2], ld->env))) {
      cx.why = "tile load is not `if in range then tile[ty*T+tx] <- x[..] else tile[ty*T+tx] <- 0.0`";
      return false;
    }
    const std::string tile_name = (*th)[1][1].s;
    const Sx rhs = inline_expr((*th)[2], ld->env);
    int prm;
    const Sx* pidx;
    if (!cx.is_read(rhs, &prm, &pidx)) return false;
    if (tile_name == tile_a && g.a < 0) {
      // a[row*k + t*T + tx], guarded by row < m && t*T+tx < k: k is whatever parameter makes both hold
      const Poly a_col = poly_add(poly_mul(TV, PT), TX);
      int kk = -1;
      for (size_t i = 0; i < plan.params.size() && kk < 0; ++i) {
        if (plan.params[i].is_vec || plan.params[i].elt != "i32") continue;
        const Poly K_ = poly_atom("p" + std::to_string(i));
        if (poly_is(cx, *pidx, poly_add(poly_mul(ROW, K_), a_col)) && guard_is(cx, cond, ROW, M_, a_col, K_)) kk = static_cast<int>(i);
      }
      if (kk < 0) {
        cx.why = "A tile is not loaded from a[row*k + t*T+tx] under row < m && t*T+tx < k";
        return false;
      }
      g.a = prm;
      g.k = kk;
    } else if (tile_name == tile_b && g.b < 0) {
      const Poly b_row = poly_add(poly_mul(TV, PT), TY);
      bool ok = false;
      for (size_t i = 0; i < plan.params.size() && !ok; ++i) {
        if (plan.params[i].is_vec || plan.params[i].elt != "i32") continue;
        const Poly K_ = poly_atom("p" + std::to_string(i));
        if (poly_is(cx, *pidx, poly_add(poly_mul(b_row, N_), COL)) && guard_is(cx, cond, b_row, K_, COL, N_)) {
          ok = true;
          if (g.k >= 0 && g.k != static_cast<int>(i)) ok = false;
          if (g.k < 0) g.k = static_cast<int>(i);
        }
      }
      if (!ok) {
        cx.why = "B tile is not loaded from b[(t*T+ty)*n + col] under t*T+ty < k && col < n";
        return false;
      }
      g.b = prm;
    } else {
      cx.why = "the k-tile loop loads the same tile twice";
      return false;
    }
  }
  if (g.a < 0 || g.b < 0 || g.k < 0) return false;
  // outer loop: t = 0 .. (k + T - 1) / T - 1
  {
    const Poly K_ = poly_atom("p" + std::to_string(g.k));
    const Poly num_tiles = poly_atom("div(" + poly_print(poly_add(K_, poly_const(T - 1))) + "|" + poly_print(PT) + ")");
    if (!is_const_i32(inline_expr(outer[3], pl.env), 0) || !poly_is(cx, inline_expr(outer[4], pl.env), poly_add(num_tiles, poly_const(-1)))) {
      cx.why = "k-tile loop does not run from 0 to (k + T - 1) / T - 1";
      return false;
    }
  }
  if (!match_epilogue(cx, inline_expr(st[2], fin.env), acc_id, out_idx, col, &g)) {
    cx.why = "stored expression is not act(alpha*sum + beta*c[row*n+col] + bias[col])";
    return false;
  }
  g.tile = static_cast<int>(T);
  plan.kind = KIND_GEMM_TILED;
  plan.gemm = g;
  return true;
}

std::string describe_gemm(const KernelPlan& p) {
  const GemmPlan& g = p.gemm;
  std::ostringstream o;
  o << (p.kind == KIND_GEMM_TILED ? "gemm:tiled" : "gemm:naive") << " A=" << p.params[g.a].name
    << " B=" << p.params[g.b].name << " D=" << p.params[g.d].name << " m=" << p.params[g.m].name
    << " n=" << p.params[g.n].name << " k=" << p.params[g.k].name;
  if (g.alpha.param >= 0)
    o << " alpha=" << p.params[g.alpha.param].name;
  else if (g.alpha.value != 1.0)
    o << " alpha=" << g.alpha.value;
  if (g.c >= 0) {
    o << " C=" << p.params[g.c].name << " beta=";
    if (g.beta.param >= 0)
      o << p.params[g.beta.param].name;
    else
      o << g.beta.value;
  }
  if (g.bias >= 0) o << " bias=" << p.params[g.bias].name;
  if (g.act == 1) o << " act=relu";
  if (g.tile) o << " tile=" << g.tile;
  return o.str();
}

bool has_unsupported_stmt(const Sx& s, std::string* what) {
  if (s.atom) return false;
  if (s.is("while") || s.is("return") || s.is("match") || s.is("native")) {
    *what = s[0].s;
    return true;
  }
  for (const Sx& k : s.kids)
    if (has_unsupported_stmt(k, what)) return true;
  return false;
}

// ---------------------------------------------------------------- grammar check
// Every form the grammar in ir.hpp names must have the shape given there: the recogniser and the fusion pass
// index into these lists without further checks.  Forms with a head the grammar does not know pass through
// (their children are not inspected): the recogniser simply does not match them.
bool atom_at(const Sx& e, size_t i) { return i < e.size() && e[i].atom; }

bool bad_form(const Sx& e, std::string* err) {
  std::string t = sx_print(e);
  if (t.size() > 120) t = t.substr(0, 117) + "...";
  *err = "malformed IR form: " + t;
  return false;
}

bool validate_expr(const Sx& e, std::string* err);

bool validate_exprs(const Sx& e, size_t from, std::string* err) {
  for (size_t i = from; i < e.size(); ++i)
    if (!validate_expr(e[i], err)) return false;
  return true;
}

bool validate_expr(const Sx& e, std::string* err) {
  if (e.atom || e.kids.empty() || !e[0].atom) return bad_form(e, err);
  const std::string& h = e[0].s;
  if (h == "const") return (e.size() == 3 && atom_at(e, 2)) || bad_form(e, err);
  if (h == "evar") return (e.size() == 3 && atom_at(e, 1) && atom_at(e, 2)) || bad_form(e, err);
  if (h == "binop") return (e.size() == 4 && atom_at(e, 1) && validate_exprs(e, 2, err)) || (err->empty() ? bad_form(e, err) : false);
  if (h == "unop") return (e.size() == 3 && atom_at(e, 1) && validate_exprs(e, 2, err)) || (err->empty() ? bad_form(e, err) : false);
  if (h == "read") return (e.size() == 3 && atom_at(e, 1) && validate_exprs(e, 2, err)) || (err->empty() ? bad_form(e, err) : false);
  if (h == "intrinsic") {
    if (e.size() < 3 || e[1].atom || !atom_at(e, 2)) return bad_form(e, err);
    for (const Sx& k : e[1].kids)
      if (!k.atom) return bad_form(e, err);
    return validate_exprs(e, 3, err);
  }
  if (h == "cast") return (e.size() == 3 && validate_exprs(e, 2, err)) || (err->empty() ? bad_form(e, err) : false);
  if (h == "if") return (e.size() == 4 && validate_exprs(e, 1, err)) || (err->empty() ? bad_form(e, err) : false);
  if (h == "arraylen") return (e.size() == 2 && atom_at(e, 1)) || bad_form(e, err);
  if (h == "arraycreate")
    return (e.size() == 4 && atom_at(e, 3) && validate_expr(e[2], err)) || (err->empty() ? bad_form(e, err) : false);
  return true;  // a form this grammar does not know
}

bool validate_stmt(const Sx& s, std::string* err) {
  if (s.atom || s.kids.empty() || !s[0].atom) return bad_form(s, err);
  const std::string& h = s[0].s;
  auto fail_or = [&](bool ok) { return ok || (err->empty() ? bad_form(s, err) : false); };
  if (h == "assign") {
    if (s.size() != 3 || s[1].atom) return bad_form(s, err);
    const Sx& lv = s[1];
    if (lv.is("lvar")) {
      if (lv.size() != 3 || !atom_at(lv, 1) || !atom_at(lv, 2)) return bad_form(s, err);
    } else if (lv.is("elem")) {
      if (lv.size() != 3 || !atom_at(lv, 1) || !validate_expr(lv[2], err)) return err->empty() ? bad_form(s, err) : false;
    } else {
      return bad_form(s, err);
    }
    return validate_expr(s[2], err);
  }
  if (h == "seq") {
    for (size_t i = 1; i < s.size(); ++i)
      if (!validate_stmt(s[i], err)) return false;
    return true;
  }
  if (h == "sif")
    return fail_or((s.size() == 3 || s.size() == 4) && validate_expr(s[1], err) && validate_stmt(s[2], err) &&
                   (s.size() == 3 || validate_stmt(s[3], err)));
  if (h == "for")
    return fail_or(s.size() == 7 && atom_at(s, 1) && atom_at(s, 2) && atom_at(s, 5) && (s[5].s == "upto" || s[5].s == "downto") &&
                   validate_expr(s[3], err) && validate_expr(s[4], err) && validate_stmt(s[6], err));
  if (h == "let" || h == "letmut")
    return fail_or(s.size() == 6 && atom_at(s, 1) && atom_at(s, 2) && validate_expr(s[4], err) && validate_stmt(s[5], err));
  if (h == "while") return fail_or(s.size() == 3 && validate_expr(s[1], err) && validate_stmt(s[2], err));
  if (h == "block") return fail_or(s.size() == 2 && validate_stmt(s[1], err));
  if (h == "pragma") return fail_or(s.size() == 3 && validate_stmt(s[2], err));
  if (h == "barrier" || h == "warpbarrier" || h == "memfence" || h == "empty") return fail_or(s.size() == 1);
  if (h == "return" || h == "expr") return fail_or(s.size() == 2 && validate_expr(s[1], err));
  return true;  // a form this grammar does not know
}

// ---------------------------------------------------------------- binding check
// A kernel that is executed must refer only to what it declares: variables bound by a parameter, a let or a
// loop in scope (compared by id, as the reference's IR does), arrays that are vector parameters or shared
// arrays created by a let in scope.  The recogniser inlines lets on demand and never looks at a binding
// nothing uses, so without this pass dead code could name anything.
struct Scope {
  std::set<std::string> vars;    // variable ids
  std::set<std::string> arrays;  // array names
};

bool unbound(const std::string& what, const std::string& name, std::string* err) {
  *err = "the kernel refers to " + what + " '" + name + "', which it does not declare";
  return false;
}

bool check_expr_bindings(const Sx& e, const Scope& sc, std::string* err) {
  if (e.atom || e.kids.empty()) return true;
  if (e.is("evar") && e.size() == 3 && e[2].atom) {
    if (!sc.vars.count(e[2].s)) return unbound("variable", e[1].s, err);
    return true;
  }
  if ((e.is("read") && e.size() == 3 && e[1].atom) || (e.is("arraylen") && e.size() == 2 && e[1].atom)) {
    if (!sc.arrays.count(e[1].s)) return unbound("array", e[1].s, err);
  }
  for (size_t i = 1; i < e.size(); ++i)
    if (!check_expr_bindings(e[i], sc, err)) return false;
  return true;
}

bool check_stmt_bindings(const Sx& s, Scope sc, std::string* err) {
  if (s.atom || s.kids.empty()) return true;
  if ((s.is("let") || s.is("letmut")) && s.size() == 6) {
    if (!check_expr_bindings(s[4], sc, err)) return false;
    if (s[4].is("arraycreate")) sc.arrays.insert(s[1].s);
    sc.vars.insert(s[2].s);
    return check_stmt_bindings(s[5], sc, err);
  }
  if (s.is("for") && s.size() == 7) {
    if (!check_expr_bindings(s[3], sc, err) || !check_expr_bindings(s[4], sc, err)) return false;
    sc.vars.insert(s[2].s);
    return check_stmt_bindings(s[6], sc, err);
  }
  if (s.is("assign") && s.size() == 3 && !s[1].atom) {
    const Sx& lv = s[1];
    if (lv.is("lvar") && lv.size() == 3 && !sc.vars.count(lv[2].s)) return unbound("variable", lv[1].s, err);
    if (lv.is("elem") && lv.size() == 3) {
      if (!sc.arrays.count(lv[1].s)) return unbound("array", lv[1].s, err);
      if (!check_expr_bindings(lv[2], sc, err)) return false;
    }
    return check_expr_bindings(s[2], sc, err);
  }
  if (s.is("seq") || s.is("block") || s.is("pragma")) {
    for (size_t i = 1; i < s.size(); ++i)
      if (!s[i].atom && !(s.is("pragma") && i == 1) && !check_stmt_bindings(s[i], sc, err)) return false;
    return true;
  }
  if (s.is("sif") && s.size() >= 3) {
    if (!check_expr_bindings(s[1], sc, err)) return false;
    for (size_t i = 2; i < s.size(); ++i)
      if (!check_stmt_bindings(s[i], sc, err)) return false;
    return true;
  }
  if ((s.is("expr") || s.is("return")) && s.size() == 2) return check_expr_bindings(s[1], sc, err);
  return true;
}

}  // namespace

bool parse_kernel_form(const std::string& text, Sx* root, KernelPlan* plan, const Sx** body, std::string* err) {
  if (!sx_parse(text, root, err)) return false;
  if (!root->is("kernel") || root->size() != 4 || !(*root)[1].atom || !(*root)[2].is("params") || !(*root)[3].is("body") ||
      (*root)[3].size() != 2) {
    *err = "expected (kernel NAME (params ...) (body STMT))";
    return false;
  }
  plan->name = (*root)[1].s;
  plan->params.clear();
  const Sx& ps = (*root)[2];
  for (size_t i = 1; i < ps.size(); ++i) {
    const Sx& p = ps[i];
    if (!(p.is("vec") || p.is("scalar")) || p.size() != 4 || !p[1].atom || !p[2].atom) {
      *err = "malformed parameter: " + sx_print(p);
      return false;
    }
    ParamInfo pi;
    pi.name = p[1].s;
    pi.id = atoi(p[2].s.c_str());
    pi.is_vec = p.is("vec");
    pi.elt = p[3].atom ? p[3].s : sx_print(p[3]);
    plan->params.push_back(pi);
  }
  *body = &(*root)[3][1];
  err->clear();
  return validate_stmt(**body, err);
}

int ir_compile(const std::string& text, KernelPlan* plan, std::string* err) {
  Sx root;
  const Sx* body = nullptr;
  std::string perr;
  if (!parse_kernel_form(text, &root, plan, &body, &perr)) {
    if (err) *err = perr;
    return SB200_ERR_PARSE;
  }
  std::string what;
  if (has_unsupported_stmt(*body, &what)) {
    if (err) *err = "unsupported construct in kernel '" + plan->name + "': " + what;
    return SB200_ERR_UNSUPPORTED;
  }
  {
    Scope sc;
    for (const ParamInfo& pi : plan->params) {
      sc.vars.insert(std::to_string(pi.id));
      if (pi.is_vec) sc.arrays.insert(pi.name);
    }
    std::string berr;
    if (!check_stmt_bindings(*body, sc, &berr)) {
      if (err) *err = berr;
      return SB200_ERR_PARSE;
    }
  }
  Ctx cx{plan, ""};
  std::string reasons;
  if (match_map(cx, *body)) return 0;
  reasons += "map: " + cx.why;
  cx.why.clear();
  if (match_gemm_naive(cx, *body)) {
    plan->description = describe_gemm(*plan);
    return 0;
  }
  reasons += "; naive gemm: " + (cx.why.empty() ? std::string("shape mismatch") : cx.why);
  cx.why.clear();
  if (match_gemm_tiled(cx, *body)) {
    plan->description = describe_gemm(*plan);
    return 0;
  }
  reasons += "; tiled gemm: " + (cx.why.empty() ? std::string("shape mismatch") : cx.why);
  cx.why.clear();
  if (match_block_reduce(cx, *body)) return 0;
  reasons += "; block reduction: " + (cx.why.empty() ? std::string("shape mismatch") : cx.why);
  cx.why.clear();
  if (match_map_generic(cx, *body)) return 0;
  reasons += "; generic map: " + cx.why;
  if (err)
    *err = "unsupported construct in kernel '" + plan->name +
           "': body is neither a GEMM nor a supported element-wise map (" + reasons + ")";
  plan->kind = 0;
  return SB200_ERR_UNSUPPORTED;
}

}  // namespace sb200
