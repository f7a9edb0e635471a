"""Sarek kernel IR in the S-expression text form the backend consumes.

The OCaml plugin's ``generate_source`` prints a ``Sarek_ir_types.kernel``
(spoc/ir/Sarek_ir_types.ml:80-133,230-245) in this form; the grammar is given in
``spoc_b200/csrc/ir.hpp``.  This module builds the same text from Python for
the kernels of the reference's benchmarks and tests, following how the PPX
lowers them (sarek/ppx/Sarek_lower_ir.ml:274-526,577-702): ``let`` -> ``SLet``,
``mut`` -> ``SLetMut``, ``v.(i) <- e`` -> ``SAssign(LArrayElem ..)``,
``for`` bounds inclusive, ``let%shared`` -> ``SLet`` of an ``EArrayCreate``,
``let%superstep`` -> ``SSeq [SBlock body; SBarrier; cont]``.
"""
from __future__ import annotations

import itertools
from typing import Iterable, Sequence

__all__ = [
    "sx", "Builder", "vector_add_ir", "stream_triad_ir", "matmul_naive_ir", "matmul_tiled_ir",
    "triad_producer_ir", "square_add_consumer_ir", "chain_fused_ir", "generic_example_ir",
    "block_reduce_ir", "square_add_guarded_ir", "vector_copy_ir",
]


def sx(*items) -> str:
    """Render nested tuples / lists / atoms as one S-expression."""
    def r(x) -> str:
        if isinstance(x, (tuple, list)):
            return "(" + " ".join(r(i) for i in x) + ")"
        if isinstance(x, bool):
            return "true" if x else "false"
        if isinstance(x, float):
            return repr(x)
        return str(x)
    return r(items if len(items) != 1 else items[0])


class Builder:
    """Allocates variable ids the way the PPX does (one counter per kernel)."""

    def __init__(self) -> None:
        self._ids = itertools.count(1)
        self.vars: dict[str, int] = {}

    def new(self, name: str) -> int:
        i = next(self._ids)
        self.vars[name] = i
        return i

    def evar(self, name: str):
        return ("evar", name, self.vars[name])

    @staticmethod
    def c_i32(v: int):
        return ("const", "i32", int(v))

    @staticmethod
    def c_f32(v: float):
        return ("const", "f32", repr(float(v)))

    @staticmethod
    def intr(name: str, *args):
        return ("intrinsic", ("Gpu",), name) + tuple(args)

    @staticmethod
    def binop(op: str, a, b):
        return ("binop", op, a, b)

    @staticmethod
    def read(arr: str, idx):
        return ("read", arr, idx)

    def let(self, name: str, elt, e, body_fn):
        i = self.new(name)
        return ("let", name, i, elt, e, body_fn())

    def letmut(self, name: str, elt, e, body_fn):
        i = self.new(name)
        return ("letmut", name, i, elt, e, body_fn())

    def params(self, spec: Sequence[tuple[str, str, str]]):
        out = ["params"]
        for kind, name, elt in spec:
            out.append((kind, name, self.new(name), elt))
        return tuple(out)


def _kernel(name: str, params, body) -> str:
    return sx(("kernel", name, params, ("body", body)))


def vector_add_ir(name: str = "sarek_kern") -> str:
    """benchmarks/bench_vector_add.ml:47-55."""
    b = Builder()
    p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "c", "f32"), ("scalar", "n", "i32")])
    body = b.let("tid", "i32", b.intr("global_thread_id"), lambda: (
        "sif", b.binop("lt", b.evar("tid"), b.evar("n")),
        ("assign", ("elem", "c", b.evar("tid")),
         b.binop("add", b.read("a", b.evar("tid")), b.read("b", b.evar("tid"))))))
    return _kernel(name, p, body)


def vector_copy_ir(name: str = "sarek_kern") -> str:
    """benchmarks/bench_vector_copy.ml:22-30: b.(tid) <- a.(tid) under the guard tid < n."""
    b = Builder()
    p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("scalar", "n", "i32")])
    body = b.let("tid", "i32", b.intr("global_thread_id"), lambda: (
        "sif", b.binop("lt", b.evar("tid"), b.evar("n")),
        ("assign", ("elem", "b", b.evar("tid")), b.read("a", b.evar("tid")))))
    return _kernel(name, p, body)


def stream_triad_ir(name: str = "sarek_kern") -> str:
    """benchmarks/bench_stream_triad.ml:22-31."""
    b = Builder()
    p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "c", "f32"),
                  ("scalar", "scalar", "f32"), ("scalar", "n", "i32")])
    body = b.let("tid", "i32", b.intr("global_thread_id"), lambda: (
        "sif", b.binop("lt", b.evar("tid"), b.evar("n")),
        ("assign", ("elem", "a", b.evar("tid")),
         b.binop("add", b.read("b", b.evar("tid")),
                 b.binop("mul", b.read("c", b.evar("tid")), b.evar("scalar"))))))
    return _kernel(name, p, body)


def _epilogue_expr(b: Builder, sum_e, idx, col, epilogue):
    """epilogue = None | dict(alpha, beta, c, bias, relu): the stored expression
    relu(alpha *. sum +. beta *. c.(row*n+col) +. bias.(col))."""
    if not epilogue:
        return sum_e
    e = sum_e
    if epilogue.get("alpha") is not None:
        e = b.binop("mul", b.c_f32(epilogue["alpha"]), e)
    if epilogue.get("c"):
        e = b.binop("add", e, b.binop("mul", b.c_f32(epilogue.get("beta", 1.0)), b.read(epilogue["c"], idx)))
    if epilogue.get("bias"):
        e = b.binop("add", e, b.read(epilogue["bias"], col))
    if epilogue.get("relu"):
        e = ("if", b.binop("gt", e, b.c_f32(0.0)), e, b.c_f32(0.0))
    return e


def _gemm_params(b: Builder, epilogue):
    spec = [("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "c", "f32")]
    out_name = "c"
    if epilogue:
        # D = epi(A.B, C, bias): the accumulate-into matrix is read as `c`, the result is `d`
        spec = [("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "c", "f32"), ("vec", "bias", "f32"),
                ("vec", "d", "f32")]
        out_name = "d"
    spec += [("scalar", "m", "i32"), ("scalar", "n", "i32"), ("scalar", "k", "i32")]
    return b.params(spec), out_name


def matmul_naive_ir(name: str = "sarek_kern", epilogue: dict | None = None) -> str:
    """benchmarks/bench_matrix_mul.ml:55-73 (optionally with a fused epilogue store)."""
    b = Builder()
    p, out = _gemm_params(b, epilogue)

    def body_sum():
        i_id = b.new("i")
        idx_a = b.binop("add", b.binop("mul", b.evar("row"), b.evar("k")), ("evar", "i", i_id))
        idx_b = b.binop("add", b.binop("mul", ("evar", "i", i_id), b.evar("n")), b.evar("col"))
        loop = ("for", "i", i_id, b.c_i32(0), b.binop("sub", b.evar("k"), b.c_i32(1)), "upto",
                ("assign", ("lvar", "sum", b.vars["sum"]),
                 b.binop("add", b.evar("sum"), b.binop("mul", b.read("a", idx_a), b.read("b", idx_b)))))
        idx_c = b.binop("add", b.binop("mul", b.evar("row"), b.evar("n")), b.evar("col"))
        store = ("assign", ("elem", out, idx_c), _epilogue_expr(b, b.evar("sum"), idx_c, b.evar("col"), epilogue))
        return ("seq", loop, store)

    body = b.let("tid", "i32", b.intr("global_thread_id"), lambda:
        b.let("row", "i32", b.binop("div", b.evar("tid"), b.evar("n")), lambda:
        b.let("col", "i32", b.binop("mod", b.evar("tid"), b.evar("n")), lambda: (
            "sif", b.binop("and", b.binop("lt", b.evar("row"), b.evar("m")), b.binop("lt", b.evar("col"), b.evar("n"))),
            b.letmut("sum", "f32", b.c_f32(0.0), body_sum)))))
    return _kernel(name, p, body)


def matmul_tiled_ir(name: str = "sarek_kern", epilogue: dict | None = None, tile: int = 16) -> str:
    """benchmarks/bench_matrix_mul_tiled.ml:55-94 (optionally with a fused epilogue store)."""
    b = Builder()
    p, out = _gemm_params(b, epilogue)
    shared_t = ("array", "f32", "shared")

    def tile_idx(r, c):
        return b.binop("add", b.binop("mul", r, b.evar("tile_size")), c)

    def k_loop():
        t_id = b.new("t")
        t = ("evar", "t", t_id)

        def load_a():
            return b.let("a_col", "i32", b.binop("add", b.binop("mul", t, b.evar("tile_size")), b.evar("tx")), lambda: (
                "sif", b.binop("and", b.binop("lt", b.evar("row"), b.evar("m")), b.binop("lt", b.evar("a_col"), b.evar("k"))),
                ("assign", ("elem", "tile_a", tile_idx(b.evar("ty"), b.evar("tx"))),
                 b.read("a", b.binop("add", b.binop("mul", b.evar("row"), b.evar("k")), b.evar("a_col")))),
                ("assign", ("elem", "tile_a", tile_idx(b.evar("ty"), b.evar("tx"))), b.c_f32(0.0))))

        def load_b():
            return b.let("b_row", "i32", b.binop("add", b.binop("mul", t, b.evar("tile_size")), b.evar("ty")), lambda: (
                "sif", b.binop("and", b.binop("lt", b.evar("b_row"), b.evar("k")), b.binop("lt", b.evar("col"), b.evar("n"))),
                ("assign", ("elem", "tile_b", tile_idx(b.evar("ty"), b.evar("tx"))),
                 b.read("b", b.binop("add", b.binop("mul", b.evar("b_row"), b.evar("n")), b.evar("col")))),
                ("assign", ("elem", "tile_b", tile_idx(b.evar("ty"), b.evar("tx"))), b.c_f32(0.0))))

        def compute():
            i_id = b.new("i")
            i = ("evar", "i", i_id)
            return ("for", "i", i_id, b.c_i32(0), b.binop("sub", b.evar("tile_size"), b.c_i32(1)), "upto",
                    ("assign", ("lvar", "sum", b.vars["sum"]),
                     b.binop("add", b.evar("sum"),
                             b.binop("mul", b.read("tile_a", tile_idx(b.evar("ty"), i)),
                                     b.read("tile_b", tile_idx(i, b.evar("tx")))))))

        la, lb, cp = load_a(), load_b(), compute()
        steps = ("seq", ("block", la), ("barrier",),
                 ("seq", ("block", lb), ("barrier",),
                  ("seq", ("block", cp), ("barrier",), ("empty",))))
        return ("for", "t", t_id, b.c_i32(0), b.binop("sub", b.evar("num_tiles"), b.c_i32(1)), "upto", steps)

    def after_sum():
        loop = k_loop()
        idx_c = b.binop("add", b.binop("mul", b.evar("row"), b.evar("n")), b.evar("col"))
        store = ("sif", b.binop("and", b.binop("lt", b.evar("row"), b.evar("m")), b.binop("lt", b.evar("col"), b.evar("n"))),
                 ("assign", ("elem", out, idx_c), _epilogue_expr(b, b.evar("sum"), idx_c, b.evar("col"), epilogue)))
        return ("seq", loop, store)

    ts2 = tile * tile
    body = b.let("tile_a", shared_t, ("arraycreate", "f32", b.c_i32(ts2), "shared"), lambda:
        b.let("tile_b", shared_t, ("arraycreate", "f32", b.c_i32(ts2), "shared"), lambda:
        b.let("tx", "i32", b.intr("thread_idx_x"), lambda:
        b.let("ty", "i32", b.intr("thread_idx_y"), lambda:
        b.let("row", "i32", b.binop("add", b.evar("ty"), b.binop("mul", b.intr("block_dim_y"), b.intr("block_idx_y"))), lambda:
        b.let("col", "i32", b.binop("add", b.evar("tx"), b.binop("mul", b.intr("block_dim_x"), b.intr("block_idx_x"))), lambda:
        b.let("tile_size", "i32", b.c_i32(tile), lambda:
        b.let("num_tiles", "i32",
              b.binop("div", b.binop("sub", b.binop("add", b.evar("k"), b.evar("tile_size")), b.c_i32(1)), b.evar("tile_size")), lambda:
        b.letmut("sum", "f32", b.c_f32(0.0), after_sum)))))))))
    return _kernel(name, p, body)


# ---- the two-kernel chain a = b + 3c ; d = a*a + b and its fusion ----------------
# Bodies are unguarded straight-line stores indexed by the intrinsic itself, the
# form the reference's fusion pass can analyse (sarek/sarek/Sarek_fusion.ml:360-378).

def triad_producer_ir(scalar: float = 3.0, index: str = "global_thread_id") -> str:
    b = Builder()
    p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "c", "f32")])
    idx = b.intr(index)
    body = ("assign", ("elem", "a", idx),
            b.binop("add", b.read("b", idx), b.binop("mul", b.c_f32(scalar), b.read("c", idx))))
    return _kernel("triad", p, body)


def square_add_consumer_ir(index: str = "global_thread_id") -> str:
    b = Builder()
    p = b.params([("vec", "d", "f32"), ("vec", "a", "f32"), ("vec", "b", "f32")])
    idx = b.intr(index)
    body = ("assign", ("elem", "d", idx),
            b.binop("add", b.binop("mul", b.read("a", idx), b.read("a", idx)), b.read("b", idx)))
    return _kernel("square_add", p, body)


def chain_fused_ir(scalar: float = 3.0, index: str = "global_thread_id") -> str:
    """What Sarek_fusion.fuse yields for (triad_producer, square_add_consumer, "a"):
    consumer body with both reads of `a` replaced by the producer's expression,
    `a` dropped from the parameters, producer parameters appended, named
    <consumer>_fused (sarek/sarek/Sarek_fusion.ml:482-547)."""
    b = Builder()
    # consumer params d(1) a(2) b(3) keep their ids; the producer's c is appended
    p = ("params", ("vec", "d", 1, "f32"), ("vec", "b", 3, "f32"), ("vec", "c", 3, "f32"))
    idx = b.intr(index)
    t = b.binop("add", b.read("b", idx), b.binop("mul", b.c_f32(scalar), b.read("c", idx)))
    body = ("assign", ("elem", "d", idx), b.binop("add", b.binop("mul", t, t), b.read("b", idx)))
    return _kernel("square_add_fused", p, body)


def square_add_guarded_ir(name: str = "square_add") -> str:
    """d.(tid) <- a.(tid) *. a.(tid) +. b.(tid) in the guarded form of the reference's benchmark kernels
    (let tid = global_thread_id in if tid < n then ..., benchmarks/bench_stream_triad.ml:22-31): the
    consumer that follows stream_triad_ir in the chain a = b + s*c ; d = a*a + b."""
    b = Builder()
    p = b.params([("vec", "d", "f32"), ("vec", "a", "f32"), ("vec", "b", "f32"), ("scalar", "n", "i32")])
    body = b.let("tid", "i32", b.intr("global_thread_id"), lambda: (
        "sif", b.binop("lt", b.evar("tid"), b.evar("n")),
        ("assign", ("elem", "d", b.evar("tid")),
         b.binop("add", b.binop("mul", b.read("a", b.evar("tid")), b.read("a", b.evar("tid"))), b.read("b", b.evar("tid"))))))
    return _kernel(name, p, body)


def generic_example_ir() -> str:
    """A map outside the ahead-of-time shapes, with two stores and a math intrinsic:
         u.(i) <- x.(i) /. (y.(i) +. 2.5) -. sqrt (abs_float (z.(i) *. s))
         v.(i) <- if u.(i) > 0.0 then u.(i) *. x.(i) else -. y.(i)
    guarded by i < n.  The second store reads the value the first one stored."""
    b = Builder()
    p = b.params([("vec", "u", "f32"), ("vec", "v", "f32"), ("vec", "x", "f32"), ("vec", "y", "f32"), ("vec", "z", "f32"),
                  ("scalar", "s", "f32"), ("scalar", "n", "i32")])

    def body():
        i = b.evar("i")
        e1 = b.binop("sub", b.binop("div", b.read("x", i), b.binop("add", b.read("y", i), b.c_f32(2.5))),
                     ("intrinsic", ("Float32",), "sqrt",
                      ("intrinsic", ("Float32",), "abs_float", b.binop("mul", b.read("z", i), b.evar("s")))))
        e2 = ("if", b.binop("gt", b.read("u", i), b.c_f32(0.0)), b.binop("mul", b.read("u", i), b.read("x", i)),
              ("unop", "neg", b.read("y", i)))
        return ("sif", b.binop("lt", i, b.evar("n")), ("seq", ("assign", ("elem", "u", i), e1), ("assign", ("elem", "v", i), e2)))

    return _kernel("generic_example", p, b.let("i", "i32", b.intr("global_thread_id"), body))


def block_reduce_ir(kind: str = "dot", block: int = 256, name: str | None = None, final_superstep: bool | None = None) -> str:
    """The shared-memory tree reductions of the reference: kind "sum" is reduce_sum_kernel
    (benchmarks/bench_reduction.ml:62-105), kind "dot" is dot_product_kernel
    (benchmarks/bench_dot_product.ml:17-57).  One let%superstep per line of the source:
    load, then reduce<block/2> ... reduce1, then the final guarded store.  The reference's generated code shows
    the final store of reduce_sum as a superstep of its own (a block followed by a barrier,
    benchmarks/descriptions/generated/reduction_generated.md) and that of dot_product as a plain statement
    (dot_product_generated.md); final_superstep selects the form and defaults to that difference."""
    if final_superstep is None:
        final_superstep = kind != "dot"
    b = Builder()
    if kind == "dot":
        p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "output", "f32"), ("scalar", "n", "i32")])
    else:
        p = b.params([("vec", "input", "f32"), ("vec", "output", "f32"), ("scalar", "n", "i32")])

    def steps():
        tid, gid = b.evar("tid"), b.evar("gid")
        elem = b.binop("mul", b.read("a", gid), b.read("b", gid)) if kind == "dot" else b.read("input", gid)
        load = ("sif", b.binop("lt", gid, b.evar("n")), ("assign", ("elem", "sdata", tid), elem),
                ("assign", ("elem", "sdata", tid), b.c_f32(0.0)))
        final = ("sif", b.binop("eq", tid, b.c_i32(0)),
                 ("assign", ("elem", "output", b.intr("block_idx_x")), b.read("sdata", b.c_i32(0))))
        chain = ("seq", ("block", final), ("barrier",), ("empty",)) if final_superstep else final
        c = 1
        tree = []
        while c < block:
            tree.append(c)
            c *= 2
        for c in tree:          # innermost continuation first: reduce1 wraps final, reduce2 wraps that, ...
            step = ("sif", b.binop("lt", tid, b.c_i32(c)),
                    ("assign", ("elem", "sdata", tid),
                     b.binop("add", b.read("sdata", tid), b.read("sdata", b.binop("add", tid, b.c_i32(c))))))
            chain = ("seq", ("block", step), ("barrier",), chain)
        return ("seq", ("block", load), ("barrier",), chain)

    body = b.let("sdata", ("array", "f32", "shared"), ("arraycreate", "f32", b.c_i32(block), "shared"), lambda:
        b.let("tid", "i32", b.intr("thread_idx_x"), lambda:
        b.let("gid", "i32", b.binop("add", b.intr("thread_idx_x"), b.binop("mul", b.intr("block_dim_x"), b.intr("block_idx_x"))),
              steps)))
    return _kernel(name or ("dot_product" if kind == "dot" else "reduce_sum"), p, body)
