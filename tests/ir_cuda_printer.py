"""IR text -> CUDA C, the way the reference's CUDA backend prints a kernel.

Test infrastructure only.  The backend consumes Sarek kernels as S-expression
text (grammar in spoc_b200/csrc/ir.hpp); the recogniser, the fusion pass and the
GPU tests are all fed text built by spoc_b200/sarek_ir.py.  To pin that text to
something the reference itself holds, this module renders it as CUDA C following
the reference's printer rule by rule (sarek-cuda/Sarek_ir_cuda.ml:37-63 types and
parameters, :67-95 thread intrinsics, :99-246 expressions, :417-433 l-values,
:437-607 statements, :669-680 array declarations, :687-706 parameters,
:871-929 kernel frame), and tests/test_ir_golden.py compares the result byte for
byte with the `## CUDA C` blocks of the reference's generated-code files
(benchmarks/descriptions/generated/*_generated.md, which its CI regenerates and
diffs, .github/workflows/ci.yml:150-184).
"""
from __future__ import annotations

import re

_TOKEN = re.compile(r"\(|\)|[^\s()]+")


def parse(text: str):
    """S-expression text -> nested lists of strings."""
    stack, cur = [], None
    root = None
    for tok in _TOKEN.findall(text):
        if tok == "(":
            new = []
            if cur is not None:
                cur.append(new)
                stack.append(cur)
            cur = new
        elif tok == ")":
            if stack:
                cur = stack.pop()
            else:
                root, cur = cur, None
        else:
            cur.append(tok)
    assert root is not None and cur is None, "unbalanced S-expression"
    return root


_CTYPE = {"i32": "int", "i64": "long long", "f32": "float", "f64": "double", "bool": "int", "unit": "void"}


def ctype(elt) -> str:
    if isinstance(elt, list):  # (array ELT SPACE) | (vecof ELT)
        return ctype(elt[1]) + "*"
    return _CTYPE[elt]


_THREAD = {
    "thread_id_x": "threadIdx.x", "thread_idx_x": "threadIdx.x", "thread_id_y": "threadIdx.y", "thread_idx_y": "threadIdx.y",
    "thread_id_z": "threadIdx.z", "thread_idx_z": "threadIdx.z", "block_id_x": "blockIdx.x", "block_idx_x": "blockIdx.x",
    "block_id_y": "blockIdx.y", "block_idx_y": "blockIdx.y", "block_id_z": "blockIdx.z", "block_idx_z": "blockIdx.z",
    "block_dim_x": "blockDim.x", "block_dim_y": "blockDim.y", "block_dim_z": "blockDim.z",
    "grid_dim_x": "gridDim.x", "grid_dim_y": "gridDim.y", "grid_dim_z": "gridDim.z",
    "global_thread_id": "(threadIdx.x + blockIdx.x * blockDim.x)", "global_idx": "(threadIdx.x + blockIdx.x * blockDim.x)",
    "global_idx_x": "(threadIdx.x + blockIdx.x * blockDim.x)", "global_idx_y": "(threadIdx.y + blockIdx.y * blockDim.y)",
    "global_idx_z": "(threadIdx.z + blockIdx.z * blockDim.z)", "global_size": "(blockDim.x * gridDim.x)",
}
_BINOP = {"add": " + ", "sub": " - ", "mul": " * ", "div": " / ", "mod": " % ", "eq": " == ", "ne": " != ", "lt": " < ",
          "le": " <= ", "gt": " > ", "ge": " >= ", "and": " && ", "or": " || ", "shl": " << ", "shr": " >> ",
          "band": " & ", "bor": " | ", "bxor": " ^ "}
_UNOP = {"neg": "-", "not": "!", "bnot": "~"}
_MATH = {"sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh", "exp", "exp2", "log", "log2", "log10", "sqrt",
         "rsqrt", "cbrt", "floor", "ceil", "round", "trunc", "fabs", "atan2", "pow", "fma", "min", "max"}


def _float_literal(text: str) -> str:
    s = "%.17g" % float(text)
    if "." not in s and "e" not in s:
        s += ".0"
    return s


def expr(e) -> str:
    h = e[0]
    if h == "const":
        t, v = e[1], e[2]
        if t == "i32":
            return str(int(v))
        if t == "i64":
            return str(int(v)) + "LL"
        if t == "f32":
            return _float_literal(v) + "f"
        if t == "f64":
            return "%.17g" % float(v)
        if t == "bool":
            return "1" if v == "true" else "0"
        return "(void)0"
    if h == "evar":
        return e[1]
    if h == "binop":
        return "(" + expr(e[2]) + _BINOP[e[1]] + expr(e[3]) + ")"
    if h == "unop":
        return "(" + _UNOP[e[1]] + expr(e[2]) + ")"
    if h == "read":
        return e[1] + "[" + expr(e[2]) + "]"
    if h == "intrinsic":
        name, args = e[2], e[3:]
        if name in _THREAD:
            return _THREAD[name]
        if name in _MATH:
            return name + "(" + ", ".join(expr(a) for a in args) + ")"
        if name == "block_barrier":
            return "__syncthreads()"
        raise ValueError(f"intrinsic {name} is printed through the reference's registry templates, which this printer does not carry")
    if h == "cast":
        return "(" + ctype(e[1]) + ")" + expr(e[2])
    if h == "if":
        return "(" + expr(e[1]) + " ? " + expr(e[2]) + " : " + expr(e[3]) + ")"
    if h == "arraylen":
        return "sarek_" + e[1] + "_length"
    raise ValueError(f"unprintable expression {h}")


def lvalue(lv) -> str:
    if lv[0] == "lvar":
        return lv[1]
    return lv[1] + "[" + expr(lv[2]) + "]"


def stmt(s, ind: str, out: list) -> None:
    h = s[0]
    if h == "empty":
        return
    if h == "seq":
        for x in s[1:]:
            stmt(x, ind, out)
    elif h == "assign":
        out.append(ind + lvalue(s[1]) + " = " + expr(s[2]) + ";\n")
    elif h == "sif":
        out.append(ind + "if (" + expr(s[1]) + ") {\n")
        stmt(s[2], ind + "  ", out)
        out.append(ind + "}")
        if len(s) > 3:
            out.append(" else {\n")
            stmt(s[3], ind + "  ", out)
            out.append(ind + "}\n")
        else:
            out.append("\n")
    elif h == "while":
        out.append(ind + "while (" + expr(s[1]) + ") {\n")
        stmt(s[2], ind + "  ", out)
        out.append(ind + "}\n")
    elif h == "for":
        name, lo, hi, direction, body = s[1], s[3], s[4], s[5], s[6]
        op, incr = ("<=", "++") if direction == "upto" else (">=", "--")
        out.append(f"{ind}for (int {name} = {expr(lo)}; {name} {op} {expr(hi)}; {name}{incr}) {{\n")
        stmt(body, ind + "  ", out)
        out.append(ind + "}\n")
    elif h == "return":
        out.append(ind + "return " + expr(s[1]) + ";\n")
    elif h == "barrier":
        out.append(ind + "__syncthreads();\n")
    elif h == "warpbarrier":
        out.append(ind + "__syncwarp();\n")
    elif h == "memfence":
        out.append(ind + "__threadfence();\n")
    elif h == "expr":
        out.append(ind + expr(s[1]) + ";\n")
    elif h in ("let", "letmut"):
        name, elt, e, body = s[1], s[3], s[4], s[5]
        if h == "let" and isinstance(e, list) and e[0] == "arraycreate":
            space = "__shared__ " if e[3] == "shared" else ""
            out.append(f"{ind}{space}{ctype(e[1])} {name}[{expr(e[2])}];\n")
        else:
            out.append(f"{ind}{ctype(elt)} {name} = {expr(e)};\n")
        stmt(body, ind, out)
    elif h == "pragma":
        out.append(ind + "#pragma " + " ".join(s[1]) + "\n")
        stmt(s[2], ind, out)
    elif h == "block":
        out.append(ind + "{\n")
        stmt(s[1], ind + "  ", out)
        out.append(ind + "}\n")
    else:
        raise ValueError(f"unprintable statement {h}")


def cuda_source(ir_text: str) -> str:
    """The complete CUDA translation unit the reference's generate_with_types yields for this kernel (no custom
    types, no helper functions, no kernel-level locals: none of the path's kernels has any)."""
    k = parse(ir_text)
    assert k[0] == "kernel" and k[2][0] == "params" and k[3][0] == "body"
    params = []
    for p in k[2][1:]:
        kind, name, elt = p[0], p[1], p[3]
        if kind == "vec":
            params.append(f"{ctype(elt)}* __restrict__ {name}, int sarek_{name}_length")
        else:
            params.append(f"{ctype(elt)} {name}")
    out = ['\nextern "C" {\n', "__global__ void " + k[1] + "(" + ", ".join(params) + ") {\n"]
    stmt(k[3][1], "  ", out)
    out.append("}\n}\n")
    return "".join(out)
