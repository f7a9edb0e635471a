// ir.hpp — Sarek kernel IR as S-expression text: parser, printer, and the
// recogniser that maps a kernel body onto one of this backend's operators.
//
// The text form mirrors the constructors of spoc/ir/Sarek_ir_types.ml:80-133:
//
//   kernel := (kernel NAME (params PARAM*) (body STMT))
//   PARAM  := (vec NAME ID ELT) | (scalar NAME ID ELT)         DParam
//   ELT    := f32 | f64 | i32 | i64 | bool | unit | (array ELT SPACE) | (vecof ELT)
//   EXPR   := (const ELT VALUE)                               EConst
//           | (evar NAME ID)                                  EVar
//           | (binop OP EXPR EXPR)     OP: add sub mul div mod eq ne lt le gt ge
//                                          and or shl shr band bor bxor
//           | (unop OP EXPR)           OP: neg not bnot
//           | (read ARR EXPR)                                 EArrayRead
//           | (intrinsic (PATH*) NAME EXPR*)                  EIntrinsic
//           | (cast ELT EXPR) | (if EXPR EXPR EXPR)           ECast, EIf
//           | (arraylen ARR) | (arraycreate ELT EXPR SPACE)   EArrayLen, EArrayCreate
//   LV     := (lvar NAME ID) | (elem ARR EXPR)                LVar, LArrayElem
//   STMT   := (assign LV EXPR) | (seq STMT*) | (sif EXPR STMT [STMT])
//           | (for NAME ID EXPR EXPR upto|downto STMT)        SFor (bounds inclusive)
//           | (let NAME ID ELT EXPR STMT) | (letmut NAME ID ELT EXPR STMT)
//           | (while EXPR STMT) | (block STMT) | (pragma (STR*) STMT)
//           | (barrier) | (warpbarrier) | (memfence) | (empty)
//           | (return EXPR) | (expr EXPR)
//
// Host-only code: no CUDA here, so it is unit-tested without a GPU.
#pragma once
#include <memory>
#include <string>
#include <vector>

namespace sb200 {

struct Sx {
  bool atom = false;
  std::string s;         // atom text
  std::vector<Sx> kids;  // list elements
  static Sx A(const std::string& t) { Sx x; x.atom = true; x.s = t; return x; }
  static Sx L(std::vector<Sx> k) { Sx x; x.kids = std::move(k); return x; }
  bool is(const char* head) const { return !atom && !kids.empty() && kids[0].atom && kids[0].s == head; }
  const Sx& operator[](size_t i) const { return kids[i]; }
  size_t size() const { return kids.size(); }
};

bool sx_parse(const std::string& text, Sx* out, std::string* err);
std::string sx_print(const Sx& x);
bool sx_equal(const Sx& a, const Sx& b);

struct ParamInfo {
  std::string name;
  int id = 0;
  bool is_vec = false;
  std::string elt;  // "f32", "i32", ...
};

// A coefficient that is either a literal or a float scalar parameter.
struct Coef {
  int param = -1;  // index into params, or -1
  double value = 0.0;
};

enum { OP_VECADD = 0, OP_TRIAD = 1, OP_CHAIN = 2, OP_CHAIN_KEEP = 3, OP_GENERIC = 4 };
enum { IDX_GLOBAL = 0, IDX_THREAD_X = 1 };
enum { KIND_MAP = 1, KIND_GEMM_NAIVE = 2, KIND_GEMM_TILED = 3, KIND_BLOCK_REDUCE = 4 };

struct MapPlan {
  int op = -1;
  int out0 = -1, out1 = -1, in0 = -1, in1 = -1;  // param indices
  Coef scalar;
  int n_param = -1;  // guard `idx < n`; -1 when the body is unguarded
  int index_kind = IDX_GLOBAL;
};

// An element-wise map that is none of the ahead-of-time shapes: the expression is
// emitted as CUDA source into the vectorised map skeleton and compiled at run time.
struct GenericMap {
  std::vector<int> inputs;   // float32 vector params read at the element index
  std::vector<int> outputs;  // float32 vector params stored, in store order
  std::vector<int> scalars;  // scalar params used by the expression (passed as double / long long)
  std::string source;        // complete CUDA translation unit (kernels sb200_map_vec, sb200_map_scalar)
};

struct GemmPlan {
  int a = -1, b = -1, d = -1;  // param indices of A, B and the output
  int m = -1, n = -1, k = -1;  // scalar params
  Coef alpha;                  // default 1
  Coef beta;                   // coefficient of the C term
  int c = -1;                  // param read at row*n+col in the epilogue, or -1
  int bias = -1;               // param read at col in the epilogue, or -1
  int act = 0;                 // 0 none, 1 relu
  int tile = 0;                // tiled shape: the kernel's tile size (16)
};

// Block-level tree reduction with a fused map (the reduce_sum / dot_product kernel shape):
// out[block] = sum over the block's elements of f(inputs[gid]), zero past n.  Inputs, scalars and
// the generated source live in KernelPlan::generic; outputs[0] is the per-block result vector.
struct ReducePlan {
  int n_param = -1;
  int block = 0;  // the kernel's block size (shared array length)
};

struct KernelPlan {
  std::string name;
  std::vector<ParamInfo> params;
  int kind = 0;
  MapPlan map;
  GenericMap generic;  // when map.op == OP_GENERIC, or kind == KIND_BLOCK_REDUCE
  ReducePlan reduce;
  GemmPlan gemm;
  std::string description;
};

// Returns 0 or a negative SB200_ERR_* (PARSE, UNSUPPORTED); *err explains.
int ir_compile(const std::string& text, KernelPlan* plan, std::string* err);

// Fusion of element-wise kernels on IR text (sarek/sarek/Sarek_fusion.ml).
int ir_can_fuse(const std::string& producer, const std::string& consumer, const std::string& inter, bool* ok,
                std::string* err);
int ir_fuse(const std::string& producer, const std::string& consumer, const std::string& inter, std::string* out,
            std::string* err);
int ir_fuse_pipeline(const std::vector<std::string>& kernels, std::string* out, std::vector<std::string>* eliminated,
                     std::string* err);
int ir_should_fuse(const std::string& producer, const std::string& consumer, const std::string& inter,
                   std::string* decision, std::string* reason, std::string* err);
int ir_auto_fuse_pipeline(const std::vector<std::string>& kernels, std::string* out, std::vector<std::string>* eliminated,
                          std::vector<std::string>* skipped, std::string* err);
int ir_analyze(const std::string& kernel, std::string* report, std::string* err);
// kind: 0 plain, 1 reduction (fuse_reduction), 2 stencil (fuse_stencil), 3 try_fuse, 4 try_fuse_all
int ir_can_fuse_as(const std::string& producer, const std::string& consumer, const std::string& inter, int kind, bool* ok,
                   std::string* err);
int ir_fuse_as(const std::string& producer, const std::string& consumer, const std::string& inter, int kind, std::string* out,
               bool* fused, std::string* err);

int ir_fuse_pipeline_as(const std::vector<std::string>& kernels, int kind, std::string* out, std::vector<std::string>* eliminated,
                        std::string* err);

}  // namespace sb200
