// fusion.cc — vertical fusion of element-wise kernels on IR text.
//
// Restates the behaviour of the reference's host-side fusion pass
// (sarek/sarek/Sarek_fusion.ml) on the S-expression form of the IR:
//   expr_equal            :32-46     structural equality, variables by id
//   collect_reads/writes  :170-262   (array, index) pairs, newest first
//   analyze_pattern       :296-322   OneToOne / Stencil offsets / Gather
//   find_write_expr       :360-378   gives up inside if / for / while
//   can_fuse              :401-431
//   fuse                  :459-547   substitute, drop the intermediate,
//                                    append producer parameters, "<name>_fused"
//   fuse_pipeline         :570-598   greedy left to right
//   should_fuse           :1068-1098 Fuse / DontFuse / MaybeFuse with reason
//   auto_fuse_pipeline    :1133-1165
//   fuse_reduction        :609-766   map -> fold, try_fuse
//   fuse_stencil          :772-1030  shifted producer expressions, try_fuse_all
// A consumer that reads the intermediate more than once is classified as a
// stencil exactly as in the reference, so can_fuse refuses it while a direct
// fuse, fuse_stencil and try_fuse_all rewrite every read.
#include <algorithm>
#include <functional>
#include <map>
#include <set>

#include "../../include/sb200.h"
#include "ir.hpp"

namespace sb200 {

bool parse_kernel_form(const std::string& text, Sx* root, KernelPlan* plan, const Sx** body, std::string* err);

namespace {

struct Kernel {
  Sx root;  // (kernel NAME (params ...) (body STMT))
  std::string name() const { return root[1].s; }
  const Sx& params() const { return root[2]; }
  const Sx& body() const { return root[3][1]; }
};

bool load_kernel(const std::string& text, Kernel* k, std::string* err) {
  KernelPlan plan;
  const Sx* body;
  return parse_kernel_form(text, &k->root, &plan, &body, err);
}

// structural equality with variables compared by id only; forms the
// reference's expr_equal does not know (if, cast, ...) never compare equal
bool expr_equal(const Sx& a, const Sx& b) {
  if (a.atom || b.atom || a.kids.empty() || b.kids.empty() || !a[0].atom || !b[0].atom || a[0].s != b[0].s) return false;
  const std::string& h = a[0].s;
  if (h == "const") return a.size() == 3 && b.size() == 3 && a[1].s == b[1].s && a[2].s == b[2].s;
  if (h == "evar") return a.size() >= 3 && b.size() >= 3 && a[2].s == b[2].s;
  if (h == "binop") return a.size() == 4 && b.size() == 4 && a[1].s == b[1].s && expr_equal(a[2], b[2]) && expr_equal(a[3], b[3]);
  if (h == "unop") return a.size() == 3 && b.size() == 3 && a[1].s == b[1].s && expr_equal(a[2], b[2]);
  if (h == "read") return a.size() == 3 && b.size() == 3 && a[1].s == b[1].s && expr_equal(a[2], b[2]);
  if (h == "intrinsic") {
    if (a.size() != b.size() || a.size() < 3 || !sx_equal(a[1], b[1]) || a[2].s != b[2].s) return false;
    for (size_t i = 3; i < a.size(); ++i)
      if (!expr_equal(a[i], b[i])) return false;
    return true;
  }
  return false;
}

using Access = std::pair<std::string, Sx>;  // (array, index)
using AccessList = std::vector<Access>;     // front = most recently found (the reference conses)

void push_front(AccessList* l, Access a) { l->insert(l->begin(), std::move(a)); }

void reads_expr(const Sx& e, AccessList* acc) {
  if (e.atom || e.kids.empty()) return;
  const std::string& h = e[0].s;
  if (h == "read" && e.size() == 3) {
    // (arr, idx) :: collect idx  — the read itself ends up in front of its index's reads
    reads_expr(e[2], acc);
    push_front(acc, {e[1].s, e[2]});
  } else if (h == "binop" && e.size() == 4) {
    reads_expr(e[2], acc);
    reads_expr(e[3], acc);
  } else if (h == "unop" && e.size() == 3) {
    reads_expr(e[2], acc);
  } else if (h == "intrinsic") {
    for (size_t i = 3; i < e.size(); ++i) reads_expr(e[i], acc);
  } else if (h == "cast" && e.size() == 3) {
    reads_expr(e[2], acc);
  } else if (h == "if" && e.size() == 4) {
    reads_expr(e[1], acc);
    reads_expr(e[2], acc);
    reads_expr(e[3], acc);
  }
}

void reads_stmt(const Sx& s, AccessList* acc) {
  if (s.atom || s.kids.empty()) return;
  const std::string& h = s[0].s;
  if (h == "assign" && s.size() == 3) {
    if (s[1].is("elem") && s[1].size() == 3) reads_expr(s[1][2], acc);
    reads_expr(s[2], acc);
  } else if (h == "seq") {
    for (size_t i = 1; i < s.size(); ++i) reads_stmt(s[i], acc);
  } else if (h == "sif") {
    reads_expr(s[1], acc);
    for (size_t i = 2; i < s.size(); ++i) reads_stmt(s[i], acc);
  } else if (h == "while" && s.size() == 3) {
    reads_expr(s[1], acc);
    reads_stmt(s[2], acc);
  } else if (h == "for" && s.size() == 7) {
    reads_expr(s[3], acc);
    reads_expr(s[4], acc);
    reads_stmt(s[6], acc);
  } else if ((h == "return" || h == "expr") && s.size() == 2) {
    reads_expr(s[1], acc);
  } else if ((h == "let" || h == "letmut") && s.size() == 6) {
    reads_expr(s[4], acc);
    reads_stmt(s[5], acc);
  } else if (h == "pragma" && s.size() == 3) {
    reads_stmt(s[2], acc);
  } else if (h == "block" && s.size() == 2) {
    reads_stmt(s[1], acc);
  }
}

void writes_stmt(const Sx& s, AccessList* acc) {
  if (s.atom || s.kids.empty()) return;
  const std::string& h = s[0].s;
  if (h == "assign" && s.size() == 3) {
    if (s[1].is("elem") && s[1].size() == 3) push_front(acc, {s[1][1].s, s[1][2]});
  } else if (h == "seq") {
    for (size_t i = 1; i < s.size(); ++i) writes_stmt(s[i], acc);
  } else if (h == "sif") {
    for (size_t i = 2; i < s.size(); ++i) writes_stmt(s[i], acc);
  } else if (h == "while" && s.size() == 3) {
    writes_stmt(s[2], acc);
  } else if (h == "for" && s.size() == 7) {
    writes_stmt(s[6], acc);
  } else if ((h == "let" || h == "letmut") && s.size() == 6) {
    writes_stmt(s[5], acc);
  } else if (h == "pragma" && s.size() == 3) {
    writes_stmt(s[2], acc);
  } else if (h == "block" && s.size() == 2) {
    writes_stmt(s[1], acc);
  }
}

bool has_barrier(const Sx& s) {
  if (s.atom) return false;
  if (s.is("barrier") || s.is("warpbarrier")) return true;
  for (const Sx& k : s.kids)
    if (has_barrier(k)) return true;
  return false;
}

enum PatternKind { P_ONE_TO_ONE, P_STENCIL, P_GATHER, P_UNKNOWN };
struct Pattern {
  PatternKind kind = P_UNKNOWN;
  Sx index;                  // OneToOne
  std::vector<int> offsets;  // Stencil
};

bool const_i32(const Sx& e, int* v) {
  if (e.is("const") && e.size() == 3 && e[1].s == "i32") {
    *v = atoi(e[2].s.c_str());
    return true;
  }
  return false;
}

// idx = base + const | base - const | const + base
bool extract_offset(const Sx& idx, Sx* base, int* off) {
  if (!idx.is("binop") || idx.size() != 4) return false;
  int n;
  if (idx[1].s == "add" && const_i32(idx[3], &n)) {
    *base = idx[2];
    *off = n;
    return true;
  }
  if (idx[1].s == "sub" && const_i32(idx[3], &n)) {
    *base = idx[2];
    *off = -n;
    return true;
  }
  if (idx[1].s == "add" && const_i32(idx[2], &n)) {
    *base = idx[3];
    *off = n;
    return true;
  }
  return false;
}

Pattern analyze_pattern(const AccessList& all, const std::string& arr) {
  std::vector<const Sx*> idxs;
  for (const Access& a : all)
    if (a.first == arr) idxs.push_back(&a.second);
  Pattern p;
  if (idxs.empty()) return p;
  if (idxs.size() == 1) {
    p.kind = P_ONE_TO_ONE;
    p.index = *idxs[0];
    return p;
  }
  std::vector<std::pair<Sx, int>> ob;
  for (const Sx* i : idxs) {
    Sx base;
    int off;
    if (extract_offset(*i, &base, &off))
      ob.emplace_back(base, off);
    else if (i->is("evar") || i->is("intrinsic"))
      ob.emplace_back(*i, 0);
  }
  if (ob.size() != idxs.size()) {
    p.kind = P_GATHER;
    return p;
  }
  for (size_t i = 1; i < ob.size(); ++i)
    if (!expr_equal(ob[i].first, ob[0].first)) {
      p.kind = P_GATHER;
      return p;
    }
  std::set<int> offs;
  for (auto& x : ob) offs.insert(x.second);
  p.kind = P_STENCIL;
  p.offsets.assign(offs.begin(), offs.end());
  return p;
}

struct Info {
  AccessList reads, writes;
  bool barriers = false;
  std::vector<std::string> read_arrays, write_arrays;  // sorted, unique
};

Info analyze(const Kernel& k) {
  Info in;
  reads_stmt(k.body(), &in.reads);
  writes_stmt(k.body(), &in.writes);
  in.barriers = has_barrier(k.body());
  std::set<std::string> r, w;
  for (auto& a : in.reads) r.insert(a.first);
  for (auto& a : in.writes) w.insert(a.first);
  in.read_arrays.assign(r.begin(), r.end());
  in.write_arrays.assign(w.begin(), w.end());
  return in;
}

bool contains(const std::vector<std::string>& v, const std::string& s) { return std::find(v.begin(), v.end(), s) != v.end(); }

bool can_fuse_k(const Kernel& prod, const Kernel& cons, const std::string& inter) {
  Info pi = analyze(prod), ci = analyze(cons);
  if (!contains(pi.write_arrays, inter) || !contains(ci.read_arrays, inter)) return false;
  if (analyze_pattern(pi.writes, inter).kind != P_ONE_TO_ONE) return false;
  if (analyze_pattern(ci.reads, inter).kind != P_ONE_TO_ONE) return false;
  return !pi.barriers && !ci.barriers;
}

// the expression stored to arr[idx]; nullptr inside conditionals and loops
const Sx* find_write_expr(const Sx& s, const std::string& arr, const Sx& idx) {
  if (s.atom || s.kids.empty()) return nullptr;
  const std::string& h = s[0].s;
  if (h == "assign" && s.size() == 3) {
    if (s[1].is("elem") && s[1].size() == 3 && s[1][1].s == arr && expr_equal(s[1][2], idx)) return &s[2];
    return nullptr;
  }
  if (h == "seq") {
    for (size_t i = 1; i < s.size(); ++i)
      if (const Sx* e = find_write_expr(s[i], arr, idx)) return e;
    return nullptr;
  }
  if ((h == "let" || h == "letmut") && s.size() == 6) return find_write_expr(s[5], arr, idx);
  if (h == "pragma" && s.size() == 3) return find_write_expr(s[2], arr, idx);
  if (h == "block" && s.size() == 2) return find_write_expr(s[1], arr, idx);
  return nullptr;
}

Sx subst_expr(const Sx& e, const std::string& arr, const Sx& idx, const Sx& repl) {
  if (e.atom) return e;
  if (e.is("read") && e.size() == 3) {
    if (e[1].s == arr && expr_equal(e[2], idx)) return repl;
    return Sx::L({e[0], e[1], subst_expr(e[2], arr, idx, repl)});
  }
  if (e.is("evar") || e.is("const") || e.is("arraylen")) return e;
  Sx o;
  for (const Sx& k : e.kids) o.kids.push_back(k.atom ? k : subst_expr(k, arr, idx, repl));
  return o;
}

Sx subst_stmt(const Sx& s, const std::string& arr, const Sx& idx, const Sx& repl) {
  if (s.atom || s.kids.empty()) return s;
  const std::string& h = s[0].s;
  if (h == "assign" && s.size() == 3) {
    Sx lv = s[1];
    if (lv.is("elem") && lv.size() == 3) lv = Sx::L({lv[0], lv[1], subst_expr(lv[2], arr, idx, repl)});
    return Sx::L({s[0], lv, subst_expr(s[2], arr, idx, repl)});
  }
  if (h == "seq" || h == "block" || h == "pragma") {
    Sx o;
    for (size_t i = 0; i < s.size(); ++i) o.kids.push_back((i == 0 || s[i].atom || (h == "pragma" && i == 1)) ? s[i] : subst_stmt(s[i], arr, idx, repl));
    return o;
  }
  if (h == "sif") {
    Sx o = Sx::L({s[0], subst_expr(s[1], arr, idx, repl)});
    for (size_t i = 2; i < s.size(); ++i) o.kids.push_back(subst_stmt(s[i], arr, idx, repl));
    return o;
  }
  if (h == "while" && s.size() == 3) return Sx::L({s[0], subst_expr(s[1], arr, idx, repl), subst_stmt(s[2], arr, idx, repl)});
  if (h == "for" && s.size() == 7)
    return Sx::L({s[0], s[1], s[2], subst_expr(s[3], arr, idx, repl), subst_expr(s[4], arr, idx, repl), s[5],
                  subst_stmt(s[6], arr, idx, repl)});
  if ((h == "let" || h == "letmut") && s.size() == 6)
    return Sx::L({s[0], s[1], s[2], s[3], subst_expr(s[4], arr, idx, repl), subst_stmt(s[5], arr, idx, repl)});
  if ((h == "return" || h == "expr") && s.size() == 2) return Sx::L({s[0], subst_expr(s[1], arr, idx, repl)});
  return s;
}

Kernel fuse_k(const Kernel& prod, const Kernel& cons, const std::string& inter) {
  AccessList cr;
  reads_stmt(cons.body(), &cr);
  const Sx* inter_idx = nullptr;
  for (const Access& a : cr)
    if (a.first == inter) {
      inter_idx = &a.second;
      break;
    }
  if (!inter_idx) return cons;
  const Sx* repl = find_write_expr(prod.body(), inter, *inter_idx);
  if (!repl) return cons;
  Sx body = subst_stmt(cons.body(), inter, *inter_idx, *repl);
  Sx params = Sx::L({Sx::A("params")});
  std::set<std::string> names;
  for (size_t i = 1; i < cons.params().size(); ++i) {
    const Sx& p = cons.params()[i];
    if (p[1].s == inter) continue;
    params.kids.push_back(p);
    names.insert(p[1].s);
  }
  for (size_t i = 1; i < prod.params().size(); ++i) {
    const Sx& p = prod.params()[i];
    if (p[1].s == inter || names.count(p[1].s)) continue;
    params.kids.push_back(p);
  }
  Kernel out;
  out.root = Sx::L({Sx::A("kernel"), Sx::A(cons.name() + "_fused"), params, Sx::L({Sx::A("body"), body})});
  return out;
}

// ---- reduction fusion (Sarek_fusion.ml:609-770) ---------------------------
// for i = a to b: acc = acc op arr[i]  (or arr[i] op acc); returns the operator
bool detect_reduction(const Sx& s, std::string* op, std::string* arr, std::string* loop_id) {
  if (!s.is("for") || s.size() != 7 || s[5].s != "upto") return false;
  const Sx& body = s[6];
  if (!body.is("assign") || body.size() != 3 || !body[1].is("lvar") || body[1].size() < 3) return false;
  const std::string acc = body[1][2].s;
  const Sx& e = body[2];
  if (!e.is("binop") || e.size() != 4) return false;
  auto is_acc = [&](const Sx& x) { return x.is("evar") && x.size() >= 3 && x[2].s == acc; };
  auto is_elem = [&](const Sx& x) {
    return x.is("read") && x.size() == 3 && x[2].is("evar") && x[2].size() >= 3 && x[2][2].s == s[2].s;
  };
  const Sx* rd = nullptr;
  if (is_acc(e[2]) && is_elem(e[3])) rd = &e[3];
  else if (is_elem(e[2]) && is_acc(e[3])) rd = &e[2];
  if (!rd) return false;
  *op = e[1].s;
  *arr = (*rd)[1].s;
  *loop_id = s[2].s;
  return true;
}

// the reference looks at the body itself and at the direct children of a top-level seq only
bool is_reduction_kernel(const Kernel& k, const std::string& arr, std::string* op) {
  std::function<bool(const Sx&)> find = [&](const Sx& s) -> bool {
    if (s.is("seq")) {
      for (size_t i = 1; i < s.size(); ++i)
        if (find(s[i])) return true;
      return false;
    }
    std::string o, a, l;
    return detect_reduction(s, &o, &a, &l) && a == arr && ((*op = o), true);
  };
  return find(k.body());
}

bool can_fuse_reduction_k(const Kernel& map_k, const Kernel& red_k, const std::string& inter) {
  Info mi = analyze(map_k), ri = analyze(red_k);
  if (!contains(mi.write_arrays, inter) || analyze_pattern(mi.writes, inter).kind != P_ONE_TO_ONE) return false;
  std::string op;
  if (!is_reduction_kernel(red_k, inter, &op)) return false;
  return !mi.barriers && !ri.barriers;
}

Sx merged_params(const Kernel& prod, const Kernel& cons, const std::string& inter) {
  Sx params = Sx::L({Sx::A("params")});
  std::set<std::string> names;
  for (size_t i = 1; i < cons.params().size(); ++i) {
    const Sx& p = cons.params()[i];
    if (p[1].s == inter) continue;
    params.kids.push_back(p);
    names.insert(p[1].s);
  }
  for (size_t i = 1; i < prod.params().size(); ++i) {
    const Sx& p = prod.params()[i];
    if (p[1].s == inter || names.count(p[1].s)) continue;
    params.kids.push_back(p);
  }
  return params;
}

Kernel fuse_reduction_k(const Kernel& map_k, const Kernel& red_k, const std::string& inter) {
  AccessList w;
  writes_stmt(map_k.body(), &w);
  const Sx* idx = nullptr;
  for (const Access& a : w)
    if (a.first == inter) {
      idx = &a.second;
      break;
    }
  if (!idx) return red_k;
  const Sx* repl = find_write_expr(map_k.body(), inter, *idx);
  if (!repl) return red_k;
  std::function<Sx(const Sx&)> tr = [&](const Sx& s) -> Sx {
    if (s.atom || s.kids.empty()) return s;
    if (s.is("for") && s.size() == 7) {
      std::string op, arr, loop_id;
      if (detect_reduction(s, &op, &arr, &loop_id) && arr == inter) {
        // arr[loop_var] -> the map's expression, as written (the reference does not re-index it)
        Sx loop_var = Sx::L({Sx::A("evar"), s[1], s[2]});
        return Sx::L({s[0], s[1], s[2], s[3], s[4], s[5], subst_stmt(s[6], inter, loop_var, *repl)});
      }
      return Sx::L({s[0], s[1], s[2], s[3], s[4], s[5], tr(s[6])});
    }
    if (s.is("seq")) {
      Sx o = Sx::L({s[0]});
      for (size_t i = 1; i < s.size(); ++i) o.kids.push_back(tr(s[i]));
      return o;
    }
    if (s.is("sif")) {
      Sx o = Sx::L({s[0], s[1]});
      for (size_t i = 2; i < s.size(); ++i) o.kids.push_back(tr(s[i]));
      return o;
    }
    if (s.is("while") && s.size() == 3) return Sx::L({s[0], s[1], tr(s[2])});
    return s;
  };
  Kernel out;
  out.root = Sx::L({Sx::A("kernel"), Sx::A(red_k.name() + "_fused"), merged_params(map_k, red_k, inter),
                    Sx::L({Sx::A("body"), tr(red_k.body())})});
  return out;
}

// ---- stencil fusion (Sarek_fusion.ml:772-1018) ------------------------------
bool can_fuse_stencil_k(const Kernel& prod, const Kernel& cons, const std::string& inter) {
  Info pi = analyze(prod), ci = analyze(cons);
  if (!contains(pi.write_arrays, inter)) return false;
  if (!contains(ci.read_arrays, inter)) return false;
  PatternKind k = analyze_pattern(ci.reads, inter).kind;
  if (k != P_STENCIL && k != P_ONE_TO_ONE) return false;
  return !pi.barriers && !ci.barriers;
}

Sx shift_expr(const Sx& e, int offset) {
  if (offset == 0 || e.atom || e.kids.empty()) return e;
  auto shift_idx = [&](const Sx& idx) {
    return Sx::L({Sx::A("binop"), Sx::A(offset > 0 ? "add" : "sub"), idx,
                  Sx::L({Sx::A("const"), Sx::A("i32"), Sx::A(std::to_string(offset > 0 ? offset : -offset))})});
  };
  if (e.is("read") && e.size() == 3) return Sx::L({e[0], e[1], shift_idx(e[2])});
  if (e.is("binop") && e.size() == 4) return Sx::L({e[0], e[1], shift_expr(e[2], offset), shift_expr(e[3], offset)});
  if (e.is("unop") && e.size() == 3) return Sx::L({e[0], e[1], shift_expr(e[2], offset)});
  if (e.is("cast") && e.size() == 3) return Sx::L({e[0], e[1], shift_expr(e[2], offset)});
  if (e.is("intrinsic")) {
    Sx o = Sx::L({e[0], e[1], e[2]});
    for (size_t i = 3; i < e.size(); ++i) o.kids.push_back(shift_expr(e[i], offset));
    return o;
  }
  return e;
}

Sx subst_stencil(const Sx& e, const std::string& arr, const Sx& base_idx, const Sx& prod_expr) {
  if (e.atom || e.kids.empty()) return e;
  if (e.is("read") && e.size() == 3 && e[1].s == arr) {
    Sx base;
    int off;
    if (extract_offset(e[2], &base, &off)) {
      if (expr_equal(base, base_idx)) return shift_expr(prod_expr, off);
      return e;
    }
    if (expr_equal(e[2], base_idx)) return prod_expr;
    return e;
  }
  if (e.is("binop") && e.size() == 4)
    return Sx::L({e[0], e[1], subst_stencil(e[2], arr, base_idx, prod_expr), subst_stencil(e[3], arr, base_idx, prod_expr)});
  if (e.is("unop") && e.size() == 3) return Sx::L({e[0], e[1], subst_stencil(e[2], arr, base_idx, prod_expr)});
  if (e.is("cast") && e.size() == 3) return Sx::L({e[0], e[1], subst_stencil(e[2], arr, base_idx, prod_expr)});
  if (e.is("intrinsic")) {
    Sx o = Sx::L({e[0], e[1], e[2]});
    for (size_t i = 3; i < e.size(); ++i) o.kids.push_back(subst_stencil(e[i], arr, base_idx, prod_expr));
    return o;
  }
  return e;
}

Kernel fuse_stencil_k(const Kernel& prod, const Kernel& cons, const std::string& inter) {
  AccessList w;
  writes_stmt(prod.body(), &w);
  const Sx* widx = nullptr;
  for (const Access& a : w)
    if (a.first == inter) {
      widx = &a.second;
      break;
    }
  if (!widx) return cons;
  const Sx* repl = find_write_expr(prod.body(), inter, *widx);
  if (!repl) return cons;
  std::function<Sx(const Sx&)> tr = [&](const Sx& s) -> Sx {
    if (s.atom || s.kids.empty()) return s;
    if (s.is("assign") && s.size() == 3) return Sx::L({s[0], s[1], subst_stencil(s[2], inter, *widx, *repl)});
    if (s.is("seq")) {
      Sx o = Sx::L({s[0]});
      for (size_t i = 1; i < s.size(); ++i) o.kids.push_back(tr(s[i]));
      return o;
    }
    if (s.is("sif")) {
      Sx o = Sx::L({s[0], subst_stencil(s[1], inter, *widx, *repl)});
      for (size_t i = 2; i < s.size(); ++i) o.kids.push_back(tr(s[i]));
      return o;
    }
    if (s.is("while") && s.size() == 3) return Sx::L({s[0], subst_stencil(s[1], inter, *widx, *repl), tr(s[2])});
    if (s.is("for") && s.size() == 7) return Sx::L({s[0], s[1], s[2], s[3], s[4], s[5], tr(s[6])});
    return s;  // the reference leaves let / block bodies untouched here
  };
  Kernel out;
  out.root = Sx::L({Sx::A("kernel"), Sx::A(cons.name() + "_stencil_fused"), merged_params(prod, cons, inter),
                    Sx::L({Sx::A("body"), tr(cons.body())})});
  return out;
}

// ---- guarded fusion (an extension of this backend; no counterpart in the reference) ----------
// The reference's own benchmark kernels have the form
//   let tid = global_thread_id in if tid < n then out.(tid) <- e
// which its pass cannot fuse: find_write_expr gives up inside a conditional (:370-375) and two
// kernels never share the id of their `tid` (:38).  Here both kernels are normalised first:
// index lets (pure, free of array reads) are inlined, so that both index the intermediate by
// the same intrinsic expression, and else-less guards are peeled off.  Fusion then needs
//   * no barrier in either kernel;
//   * every read of the intermediate in the consumer at the producer's store index;
//   * the producer unguarded, or guarded exactly as the consumer (parameters compared by name,
//     the reference's convention for "the same argument"), so that the consumer never reads an
//     element the producer would not have written;
//   * a producer expression built from parameters only.
// The result is the consumer's guarded body with the reads replaced, named <consumer>_fused,
// parameters merged as fuse does.  Each replaced read of a float32 intermediate is wrapped in
// (intrinsic (B200) stored_f32 e): "e as the vector would have held it", so the fused kernel rounds
// where the unfused pair did.
using VarEnv = std::map<std::string, Sx>;  // variable id -> defining expression (already inlined)

Sx inline_vars(const Sx& e, const VarEnv& env) {
  if (e.atom) return e;
  if (e.is("evar") && e.size() >= 3) {
    auto it = env.find(e[2].s);
    return it == env.end() ? e : it->second;
  }
  Sx o;
  o.kids.reserve(e.kids.size());
  for (const Sx& k : e.kids) o.kids.push_back(inline_vars(k, env));
  return o;
}

bool has_read(const Sx& e) {
  if (e.atom) return false;
  if (e.is("read")) return true;
  for (const Sx& k : e.kids)
    if (has_read(k)) return true;
  return false;
}

struct Normal {
  std::vector<Sx> guards;  // outermost first, index lets inlined
  Sx inner;                // the guarded statement, index lets inlined
};

Normal normalise(const Sx& body) {
  Normal n;
  VarEnv env;
  const Sx* s = &body;
  for (;;) {
    if (s->is("let") && s->size() == 6 && !(*s)[4].is("arraycreate") && !has_read((*s)[4])) {
      env[(*s)[2].s] = inline_vars((*s)[4], env);
      s = &(*s)[5];
    } else if (s->is("block") && s->size() == 2) {
      s = &(*s)[1];
    } else if (s->is("pragma") && s->size() == 3) {
      s = &(*s)[2];
    } else if (s->is("seq") && s->size() == 2) {
      s = &(*s)[1];
    } else if (s->is("sif") && s->size() == 3) {
      n.guards.push_back(inline_vars((*s)[1], env));
      s = &(*s)[2];
    } else {
      break;
    }
  }
  n.inner = inline_vars(*s, env);
  return n;
}

// structural equality with variables compared by NAME (parameters of two different kernels)
bool equal_by_name(const Sx& a, const Sx& b) {
  if (a.atom || b.atom) return a.atom && b.atom && a.s == b.s;
  if (a.is("evar") && b.is("evar")) return a.size() >= 2 && b.size() >= 2 && a[1].s == b[1].s;
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (!equal_by_name(a[i], b[i])) return false;
  return true;
}

const Sx* find_param(const Kernel& k, const std::string& name) {
  for (size_t i = 1; i < k.params().size(); ++i)
    if (k.params()[i].size() >= 3 && k.params()[i][1].s == name) return &k.params()[i];
  return nullptr;
}

// Producer variables become the consumer's where both kernels have a parameter of that name;
// false when the expression uses anything that is not a producer parameter.
bool rebind_params(const Sx& e, const Kernel& prod, const Kernel& cons, Sx* out, std::string* why) {
  if (e.atom) {
    *out = e;
    return true;
  }
  if (e.is("evar") && e.size() >= 3) {
    const Sx* pp = find_param(prod, e[1].s);
    if (!pp || (*pp)[2].s != e[2].s) {
      *why = "the producer's stored expression uses the local variable '" + e[1].s + "'";
      return false;
    }
    const Sx* cp = find_param(cons, e[1].s);
    *out = cp ? Sx::L({e[0], e[1], (*cp)[2]}) : e;
    return true;
  }
  Sx o;
  for (const Sx& k : e.kids) {
    Sx r;
    if (!rebind_params(k, prod, cons, &r, why)) return false;
    o.kids.push_back(r);
  }
  *out = o;
  return true;
}

bool fuse_guarded_k(const Kernel& prod, const Kernel& cons, const std::string& inter, Kernel* out, std::string* why) {
  if (has_barrier(prod.body()) || has_barrier(cons.body())) {
    *why = "a barrier prevents fusion";
    return false;
  }
  Normal np = normalise(prod.body()), nc = normalise(cons.body());
  AccessList pw, cr, gr;
  writes_stmt(np.inner, &pw);
  reads_stmt(nc.inner, &cr);
  for (const Sx& g : nc.guards) reads_expr(g, &gr);
  for (const Sx& g : np.guards) reads_expr(g, &gr);
  for (const Access& a : gr)
    if (a.first == inter) {
      *why = "a guard reads the intermediate";
      return false;
    }
  const Sx* widx = nullptr;
  int nwrites = 0;
  for (const Access& a : pw)
    if (a.first == inter) {
      widx = &a.second;
      ++nwrites;
    }
  if (nwrites != 1) {
    *why = nwrites ? "the producer stores the intermediate more than once" : "the producer does not store the intermediate";
    return false;
  }
  int nreads = 0;
  for (const Access& a : cr)
    if (a.first == inter) {
      ++nreads;
      if (!expr_equal(a.second, *widx)) {
        *why = "the consumer reads the intermediate at an index other than the producer's store index";
        return false;
      }
    }
  if (!nreads) {
    *why = "the consumer does not read the intermediate";
    return false;
  }
  AccessList cw;
  writes_stmt(nc.inner, &cw);
  for (const Access& a : cw)
    if (a.first == inter) {
      *why = "the consumer stores to the intermediate";
      return false;
    }
  if (!np.guards.empty()) {
    bool same = np.guards.size() == nc.guards.size();
    for (size_t i = 0; same && i < np.guards.size(); ++i) same = equal_by_name(np.guards[i], nc.guards[i]);
    if (!same) {
      *why = "the producer's guard differs from the consumer's: the consumer could read elements the producer skips";
      return false;
    }
  }
  const Sx* stored = find_write_expr(np.inner, inter, *widx);
  if (!stored) {
    *why = "the producer's store of the intermediate is inside a conditional or a loop";
    return false;
  }
  Sx repl;
  if (!rebind_params(*stored, prod, cons, &repl, why)) return false;
  // The unfused kernels round the intermediate to float32 when they store it; the mark keeps that rounding
  // in the fused kernel (generated code evaluates in double), so fused and unfused runs agree bit for bit.
  const Sx* ip = find_param(prod, inter);
  if (ip && ip->size() >= 4 && (*ip)[3].atom && (*ip)[3].s == "f32")
    repl = Sx::L({Sx::A("intrinsic"), Sx::L({Sx::A("B200")}), Sx::A("stored_f32"), repl});
  Sx body = subst_stmt(nc.inner, inter, *widx, repl);
  for (size_t i = nc.guards.size(); i-- > 0;) body = Sx::L({Sx::A("sif"), nc.guards[i], body});
  out->root = Sx::L({Sx::A("kernel"), Sx::A(cons.name() + "_fused"), merged_params(prod, cons, inter),
                     Sx::L({Sx::A("body"), body})});
  return true;
}

// try_fuse (:759-766): reduction, else plain.  try_fuse_all (:1022-1030): reduction, stencil, plain.
bool try_fuse_k(const Kernel& p, const Kernel& c, const std::string& inter, bool with_stencil, Kernel* out) {
  if (can_fuse_reduction_k(p, c, inter)) {
    *out = fuse_reduction_k(p, c, inter);
    return true;
  }
  if (with_stencil && can_fuse_stencil_k(p, c, inter)) {
    *out = fuse_stencil_k(p, c, inter);
    return true;
  }
  if (can_fuse_k(p, c, inter)) {
    *out = fuse_k(p, c, inter);
    return true;
  }
  return false;
}

struct Hint {
  const char* decision;
  const char* reason;
};

Hint should_fuse_k(const Kernel& prod, const Kernel& cons, const std::string& inter) {
  Info pi = analyze(prod), ci = analyze(cons);
  if (pi.barriers || ci.barriers) return {"DontFuse", "Barrier prevents fusion"};
  const bool pw = contains(pi.write_arrays, inter), cr = contains(ci.read_arrays, inter);
  Pattern w = analyze_pattern(pi.writes, inter), r = analyze_pattern(ci.reads, inter);
  if (pw && cr && w.kind == P_ONE_TO_ONE) {
    if (r.kind == P_ONE_TO_ONE) return {"Fuse", "Element-wise producer/consumer"};
    if (r.kind == P_STENCIL)
      return r.offsets.size() <= 3 ? Hint{"MaybeFuse", "Small stencil - profile to decide"}
                                   : Hint{"DontFuse", "Large stencil radius - keep separate"};
    if (r.kind == P_GATHER) return {"DontFuse", "Gather pattern - keep separate"};
  }
  return {"MaybeFuse", "Unknown pattern - profile to decide"};
}

std::vector<std::string> candidates(const Info& cur, const Info& next) {
  std::vector<std::string> out;
  for (const std::string& a : cur.write_arrays)
    if (contains(next.read_arrays, a)) out.push_back(a);
  return out;
}

}  // namespace

int ir_can_fuse(const std::string& producer, const std::string& consumer, const std::string& inter, bool* ok,
                std::string* err) {
  Kernel p, c;
  if (!load_kernel(producer, &p, err) || !load_kernel(consumer, &c, err)) return SB200_ERR_PARSE;
  *ok = can_fuse_k(p, c, inter);
  return SB200_OK;
}

int ir_fuse(const std::string& producer, const std::string& consumer, const std::string& inter, std::string* out,
            std::string* err) {
  Kernel p, c;
  if (!load_kernel(producer, &p, err) || !load_kernel(consumer, &c, err)) return SB200_ERR_PARSE;
  *out = sx_print(fuse_k(p, c, inter).root);
  return SB200_OK;
}

int ir_fuse_pipeline(const std::vector<std::string>& kernels, std::string* out, std::vector<std::string>* eliminated,
                     std::string* err) {
  if (kernels.empty()) {
    *err = "fuse_pipeline: empty pipeline";
    return SB200_ERR_INVALID_VALUE;
  }
  std::vector<Kernel> ks(kernels.size());
  for (size_t i = 0; i < kernels.size(); ++i)
    if (!load_kernel(kernels[i], &ks[i], err)) return SB200_ERR_PARSE;
  Kernel cur = ks[0];
  eliminated->clear();
  for (size_t i = 1; i < ks.size(); ++i) {
    std::vector<std::string> c = candidates(analyze(cur), analyze(ks[i]));
    if (!c.empty() && can_fuse_k(cur, ks[i], c[0])) {
      cur = fuse_k(cur, ks[i], c[0]);
      eliminated->insert(eliminated->begin(), c[0]);  // the reference conses: newest first
    } else {
      cur = ks[i];
    }
  }
  *out = sx_print(cur.root);
  return SB200_OK;
}

int ir_should_fuse(const std::string& producer, const std::string& consumer, const std::string& inter,
                   std::string* decision, std::string* reason, std::string* err) {
  Kernel p, c;
  if (!load_kernel(producer, &p, err) || !load_kernel(consumer, &c, err)) return SB200_ERR_PARSE;
  Hint h = should_fuse_k(p, c, inter);
  *decision = h.decision;
  *reason = h.reason;
  return SB200_OK;
}

int ir_auto_fuse_pipeline(const std::vector<std::string>& kernels, std::string* out, std::vector<std::string>* eliminated,
                          std::vector<std::string>* skipped, std::string* err) {
  if (kernels.empty()) {
    *err = "auto_fuse_pipeline: empty pipeline";
    return SB200_ERR_INVALID_VALUE;
  }
  std::vector<Kernel> ks(kernels.size());
  for (size_t i = 0; i < kernels.size(); ++i)
    if (!load_kernel(kernels[i], &ks[i], err)) return SB200_ERR_PARSE;
  Kernel cur = ks[0];
  eliminated->clear();
  skipped->clear();
  for (size_t i = 1; i < ks.size(); ++i) {
    std::vector<std::string> c = candidates(analyze(cur), analyze(ks[i]));
    if (c.empty()) {
      cur = ks[i];
      continue;
    }
    Hint h = should_fuse_k(cur, ks[i], c[0]);
    Kernel fused;
    if (std::string(h.decision) == "Fuse" && try_fuse_k(cur, ks[i], c[0], false, &fused)) {
      cur = fused;
      eliminated->insert(eliminated->begin(), c[0]);
    } else {
      skipped->insert(skipped->begin(), h.reason);
      cur = ks[i];
    }
  }
  *out = sx_print(cur.root);
  return SB200_OK;
}

// kind: 0 plain (can_fuse / fuse), 1 reduction, 2 stencil, 3 try_fuse, 4 try_fuse_all, 5 guarded (this backend's)
int ir_can_fuse_as(const std::string& producer, const std::string& consumer, const std::string& inter, int kind, bool* ok,
                   std::string* err) {
  Kernel p, c;
  if (!load_kernel(producer, &p, err) || !load_kernel(consumer, &c, err)) return SB200_ERR_PARSE;
  Kernel tmp;
  switch (kind) {
    case 0: *ok = can_fuse_k(p, c, inter); break;
    case 1: *ok = can_fuse_reduction_k(p, c, inter); break;
    case 2: *ok = can_fuse_stencil_k(p, c, inter); break;
    case 3: *ok = try_fuse_k(p, c, inter, false, &tmp); break;
    case 4: *ok = try_fuse_k(p, c, inter, true, &tmp); break;
    case 5: *ok = fuse_guarded_k(p, c, inter, &tmp, err); break;
    default: *err = "unknown fusion kind"; return SB200_ERR_INVALID_VALUE;
  }
  return SB200_OK;
}

int ir_fuse_as(const std::string& producer, const std::string& consumer, const std::string& inter, int kind, std::string* out,
               bool* fused, std::string* err) {
  Kernel p, c, r;
  if (!load_kernel(producer, &p, err) || !load_kernel(consumer, &c, err)) return SB200_ERR_PARSE;
  *fused = true;
  switch (kind) {
    case 0: r = fuse_k(p, c, inter); break;
    case 1: r = fuse_reduction_k(p, c, inter); break;
    case 2: r = fuse_stencil_k(p, c, inter); break;
    case 3: *fused = try_fuse_k(p, c, inter, false, &r); break;
    case 4: *fused = try_fuse_k(p, c, inter, true, &r); break;
    case 5: *fused = fuse_guarded_k(p, c, inter, &r, err); break;
    default: *err = "unknown fusion kind"; return SB200_ERR_INVALID_VALUE;
  }
  *out = *fused ? sx_print(r.root) : std::string();
  return SB200_OK;
}

// fuse_pipeline with a chosen fusion form per step (greedy, left to right, first candidate array as the
// reference's fuse_pipeline does, :570-598); kind as in ir_fuse_as.  With kind 5 a chain of guarded benchmark-form
// kernels collapses into one kernel.
int ir_fuse_pipeline_as(const std::vector<std::string>& kernels, int kind, std::string* out, std::vector<std::string>* eliminated,
                        std::string* err) {
  if (kernels.empty()) {
    *err = "fuse_pipeline: empty pipeline";
    return SB200_ERR_INVALID_VALUE;
  }
  if (kind < 0 || kind > 5) {
    *err = "unknown fusion kind";
    return SB200_ERR_INVALID_VALUE;
  }
  std::vector<Kernel> ks(kernels.size());
  for (size_t i = 0; i < kernels.size(); ++i)
    if (!load_kernel(kernels[i], &ks[i], err)) return SB200_ERR_PARSE;
  Kernel cur = ks[0];
  eliminated->clear();
  for (size_t i = 1; i < ks.size(); ++i) {
    std::vector<std::string> c = candidates(analyze(cur), analyze(ks[i]));
    Kernel fused;
    bool ok = false;
    if (!c.empty()) {
      std::string why;
      switch (kind) {
        case 0: ok = can_fuse_k(cur, ks[i], c[0]); if (ok) fused = fuse_k(cur, ks[i], c[0]); break;
        case 1: ok = can_fuse_reduction_k(cur, ks[i], c[0]); if (ok) fused = fuse_reduction_k(cur, ks[i], c[0]); break;
        case 2: ok = can_fuse_stencil_k(cur, ks[i], c[0]); if (ok) fused = fuse_stencil_k(cur, ks[i], c[0]); break;
        case 3: ok = try_fuse_k(cur, ks[i], c[0], false, &fused); break;
        case 4: ok = try_fuse_k(cur, ks[i], c[0], true, &fused); break;
        case 5: ok = fuse_guarded_k(cur, ks[i], c[0], &fused, &why); break;
      }
    }
    if (ok) {
      cur = fused;
      eliminated->insert(eliminated->begin(), c[0]);
    } else {
      cur = ks[i];
    }
  }
  *out = sx_print(cur.root);
  return SB200_OK;
}

// One line per array: "read|write NAME one_to_one|stencil[o1,o2]|gather|unknown", then "barriers yes|no".
int ir_analyze(const std::string& kernel, std::string* report, std::string* err) {
  Kernel k;
  if (!load_kernel(kernel, &k, err)) return SB200_ERR_PARSE;
  Info in = analyze(k);
  auto fmt = [](const Pattern& p) {
    switch (p.kind) {
      case P_ONE_TO_ONE: return std::string("one_to_one");
      case P_GATHER: return std::string("gather");
      case P_STENCIL: {
        std::string s = "stencil[";
        for (size_t i = 0; i < p.offsets.size(); ++i) s += (i ? "," : "") + std::to_string(p.offsets[i]);
        return s + "]";
      }
      default: return std::string("unknown");
    }
  };
  std::string r;
  for (auto& a : in.read_arrays) r += "read " + a + " " + fmt(analyze_pattern(in.reads, a)) + "\n";
  for (auto& a : in.write_arrays) r += "write " + a + " " + fmt(analyze_pattern(in.writes, a)) + "\n";
  r += std::string("barriers ") + (in.barriers ? "yes" : "no") + "\n";
  *report = r;
  return SB200_OK;
}

}  // namespace sb200
