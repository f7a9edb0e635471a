"""A small interpreter of the kernel IR text, for the tests only.

It executes a kernel — the same S-expression text the library is fed and that tests/test_ir_golden.py pins on the
reference's generated CUDA C — thread by thread over a launch geometry, with barriers, under one of two float32
disciplines of the reference:

* "native": what the Native backend's generated OCaml does (sarek/ppx/Sarek_native_gen.ml:96-118,746-772; sarek/core/
  Vector.ml:80-91,139-143; sarek/sarek/Sarek_cpu_runtime.ml:74-109): vector loads widen float32 to double, every
  arithmetic operation is a double operation, mutable accumulators and shared arrays hold doubles, a vector store rounds
  once to float32, int32 arithmetic wraps.
* "interpreter": what the reference's IR interpreter does (sarek/sarek/Sarek_ir_interp.ml:175-211 through
  sarek/sarek/Sarek_float32.ml:89-95): every float32 operation rounds its result to float32.

The CPU oracle (oracle/native_oracle.c) hard-codes the kernels' formulas under the first discipline; this interpreter
derives the result from the IR itself, so agreement between the two (tests/test_oracle_vs_ir_interp.py, bit for bit)
ties the oracle to the pinned IR, and the second discipline is the negative control: it must differ.
"""
from __future__ import annotations

import math

import numpy as np

from tests.ir_cuda_printer import parse

f32 = np.float32


def _wrap32(x: int) -> int:
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x & 0x80000000 else x


class _Thread:
    def __init__(self, interp, block_idx, thread_idx, shared):
        self.I, self.bidx, self.tidx, self.shared = interp, block_idx, thread_idx, shared
        self.env: dict[int, object] = {}

    # ---- expressions -------------------------------------------------------------------------------------
    def intrinsic(self, name, args):
        I = self.I
        bd, gd = I.block, I.grid
        table = {"thread_idx_x": self.tidx[0], "thread_idx_y": self.tidx[1], "thread_idx_z": self.tidx[2],
                 "block_idx_x": self.bidx[0], "block_idx_y": self.bidx[1], "block_idx_z": self.bidx[2],
                 "block_dim_x": bd[0], "block_dim_y": bd[1], "block_dim_z": bd[2],
                 "grid_dim_x": gd[0], "grid_dim_y": gd[1], "grid_dim_z": gd[2],
                 "global_thread_id": self.tidx[0] + self.bidx[0] * bd[0]}
        if name in table:
            return table[name]
        vals = [self.expr(a) for a in args]
        if name == "sqrt":
            return self.fl(math.sqrt(vals[0]))
        if name in ("abs_float", "fabs"):
            return self.fl(abs(vals[0]))
        raise NotImplementedError(f"intrinsic {name}")

    def fl(self, x):
        """Result of a float32 operation under the active discipline."""
        return float(f32(x)) if self.I.per_op_rounding else float(x)

    def expr(self, e):
        h = e[0]
        if h == "const":
            t, v = e[1], e[2]
            if t in ("i32", "i64"):
                return int(v)
            if t == "bool":
                return v == "true"
            # float literals are doubles in Native code; the interpreter holds float32 values
            return float(f32(float(v))) if (self.I.per_op_rounding and t == "f32") else float(v)
        if h == "evar":
            ident = int(e[2])
            if ident in self.env:
                return self.env[ident]
            return self.I.scalars[e[1]]
        if h == "read":
            idx = self.expr(e[2])
            arr = e[1]
            if arr in self.shared:
                return self.shared[arr][idx]
            return float(self.I.vectors[arr][idx])          # float32 -> double, exact
        if h == "binop":
            op = e[1]
            a, b = self.expr(e[2]), self.expr(e[3])
            if op in ("and", "or"):
                return (a and b) if op == "and" else (a or b)
            if op in ("lt", "le", "gt", "ge", "eq", "ne"):
                return {"lt": a < b, "le": a <= b, "gt": a > b, "ge": a >= b, "eq": a == b, "ne": a != b}[op]
            if isinstance(a, int) and isinstance(b, int) and not isinstance(a, bool):
                if op == "add":
                    return _wrap32(a + b)
                if op == "sub":
                    return _wrap32(a - b)
                if op == "mul":
                    return _wrap32(a * b)
                if op in ("div", "mod"):   # OCaml's Int32.div truncates toward zero, rem takes the dividend's sign
                    if b == 0:
                        raise ZeroDivisionError("integer division by zero in the kernel")
                    q = abs(a) // abs(b)
                    q = -q if (a < 0) != (b < 0) else q
                    return _wrap32(q) if op == "div" else _wrap32(a - b * q)
                raise NotImplementedError(op)
            r = {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "div": lambda: a / b}[op]()
            return self.fl(r)
        if h == "unop":
            v = self.expr(e[2])
            return (not v) if e[1] == "not" else (self.fl(-v) if isinstance(v, float) else _wrap32(-v))
        if h == "if":
            return self.expr(e[2]) if self.expr(e[1]) else self.expr(e[3])
        if h == "cast":
            v = self.expr(e[2])
            return float(v) if e[1] in ("f32", "f64") else int(v)
        if h == "intrinsic":
            return self.intrinsic(e[2], e[3:])
        raise NotImplementedError(f"expression {h}")

    # ---- statements: a generator that yields at barriers ------------------------------------------------------
    def stmt(self, s):
        h = s[0]
        if h == "empty":
            return
        if h == "seq":
            for x in s[1:]:
                yield from self.stmt(x)
        elif h == "block":
            yield from self.stmt(s[1])
        elif h == "barrier":
            yield "barrier"
        elif h == "assign":
            lv, val = s[1], self.expr(s[2])
            if lv[0] == "lvar":
                self.env[int(lv[2])] = val
            else:
                idx = self.expr(lv[2])
                if lv[1] in self.shared:
                    self.shared[lv[1]][idx] = val           # shared float arrays hold doubles in Native code
                else:
                    self.I.vectors[lv[1]][idx] = f32(val)    # the one rounding of a vector store
        elif h == "sif":
            if self.expr(s[1]):
                yield from self.stmt(s[2])
            elif len(s) > 3:
                yield from self.stmt(s[3])
        elif h == "for":
            ident, lo, hi, direction, body = int(s[2]), self.expr(s[3]), self.expr(s[4]), s[5], s[6]
            rng = range(lo, hi + 1) if direction == "upto" else range(lo, hi - 1, -1)
            for i in rng:
                self.env[ident] = i
                yield from self.stmt(body)
        elif h in ("let", "letmut"):
            ident, e = int(s[2]), s[4]
            if isinstance(e, list) and e[0] == "arraycreate":
                # one array per block, created by whichever thread gets here first
                if s[1] not in self.shared:
                    n = self.expr(e[2])
                    self.shared[s[1]] = [0.0] * n
            else:
                self.env[ident] = self.expr(e)
            yield from self.stmt(s[5])
        else:
            raise NotImplementedError(f"statement {h}")


class Interp:
    def __init__(self, ir_text: str, vectors: dict[str, np.ndarray], scalars: dict[str, object], grid, block,
                 per_op_rounding: bool = False):
        k = parse(ir_text)
        assert k[0] == "kernel"
        self.params = [(p[0], p[1]) for p in k[2][1:]]
        self.body = k[3][1]
        self.vectors, self.scalars = vectors, dict(scalars)
        if per_op_rounding:
            self.scalars = {n: (float(f32(v)) if isinstance(v, float) else v) for n, v in self.scalars.items()}
        self.grid = tuple(grid) + (1,) * (3 - len(grid))
        self.block = tuple(block) + (1,) * (3 - len(block))
        self.per_op_rounding = per_op_rounding

    def run(self) -> None:
        gx, gy, gz = self.grid
        bx, by, bz = self.block
        for bzz in range(gz):
            for byy in range(gy):
                for bxx in range(gx):
                    shared: dict[str, list] = {}
                    threads = [_Thread(self, (bxx, byy, bzz), (tx, ty, tz), shared)
                               for tz in range(bz) for ty in range(by) for tx in range(bx)]
                    gens = [t.stmt(self.body) for t in threads]
                    live = list(range(len(gens)))
                    while live:                      # all threads of the block advance to the next barrier together
                        nxt = []
                        for i in live:
                            try:
                                next(gens[i])
                                nxt.append(i)
                            except StopIteration:
                                pass
                        assert not nxt or len(nxt) == len(live), "threads of a block disagree about a barrier"
                        live = nxt


def run_kernel(ir_text, vectors, scalars, grid, block, discipline="native") -> None:
    """Executes the kernel in place on `vectors` (name -> float32 array)."""
    Interp(ir_text, vectors, scalars, grid, block, per_op_rounding=(discipline == "interpreter")).run()
