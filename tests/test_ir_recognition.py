"""IR text -> operator recognition, argument binding and the C ABI's behaviour without a GPU."""
import ctypes as C
import os
import re

import pytest

from spoc_b200 import Backend, BackendError, UnsupportedConstruct, dims1d, sarek_ir as S
from spoc_b200 import _lib as L

EPI = dict(alpha=1.5, beta=0.5, c="c", bias="bias", relu=True)


def compile_(ir):
    b = Backend()
    return b.Kernel.compile(b.Device.T(0, "none", 0, (10, 0), 148, 0, 0), name="sarek_kern", source=ir)


@pytest.mark.parametrize("ir,kind,needle", [
    (S.vector_add_ir(), L.KIND_MAP, "map:vector_add guarded idx=global_x"),
    (S.stream_triad_ir(), L.KIND_MAP, "map:stream_triad guarded"),
    (S.chain_fused_ir(), L.KIND_MAP, "map:triad_square_chain unguarded"),
    (S.triad_producer_ir(index="thread_idx_x"), L.KIND_MAP, "idx=thread_idx_x"),
    (S.matmul_naive_ir(), L.KIND_GEMM_NAIVE, "gemm:naive A=a B=b D=c m=m n=n k=k"),
    (S.matmul_tiled_ir(), L.KIND_GEMM_TILED, "gemm:tiled A=a B=b D=c m=m n=n k=k tile=16"),
    (S.matmul_naive_ir(epilogue=EPI), L.KIND_GEMM_NAIVE, "alpha=1.5 C=c beta=0.5 bias=bias act=relu"),
    (S.matmul_tiled_ir(epilogue=EPI), L.KIND_GEMM_TILED, "D=d m=m n=n k=k alpha=1.5 C=c beta=0.5 bias=bias act=relu tile=16"),
    (S.matmul_tiled_ir(epilogue=dict(bias="bias")), L.KIND_GEMM_TILED, "bias=bias tile=16"),
])
def test_reference_kernels_are_recognised(ir, kind, needle):
    k = compile_(ir)
    assert k.kind == kind
    assert needle in k.describe()


def test_other_elementwise_expressions_take_the_generated_kernel_path():
    k = compile_(S.square_add_consumer_ir())       # d = a*a + b: none of the ahead-of-time shapes
    assert k.kind == L.KIND_MAP and "map:generic(jit) inputs=2 outputs=1" in k.describe()
    k = compile_(S.generic_example_ir())
    assert "map:generic(jit) inputs=3 outputs=2 scalars=1 guarded" in k.describe()


@pytest.mark.parametrize("kind,block,inputs", [("dot", 256, 2), ("sum", 256, 1), ("sum", 64, 1)])
def test_block_tree_reductions_are_recognised(kind, block, inputs):
    k = compile_(S.block_reduce_ir(kind, block))
    assert k.kind == L.KIND_BLOCK_REDUCE
    assert f"reduce:block_tree(jit) block={block} inputs={inputs} out=output" in k.describe()


def test_commuted_operands_and_expanded_thread_id_are_recognised():
    b = S.Builder()
    p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("vec", "c", "f32"), ("scalar", "s", "f32"), ("scalar", "n", "i32")])
    tid = b.binop("add", b.binop("mul", b.intr("block_idx_x"), b.intr("block_dim_x")), b.intr("thread_idx_x"))
    body = b.let("i", "i32", tid, lambda: ("sif", b.binop("lt", b.evar("i"), b.evar("n")),
                 ("assign", ("elem", "a", b.evar("i")),
                  b.binop("add", b.binop("mul", b.evar("s"), b.read("c", b.evar("i"))), b.read("b", b.evar("i"))))))
    k = compile_(S.sx(("kernel", "t", p, ("body", body))))
    assert "map:stream_triad guarded idx=global_x" in k.describe()


@pytest.mark.parametrize("ir,why", [
    ("(kernel k (params (vec a 1 f32) (vec b 2 f32)) (body (assign (elem a (intrinsic (Gpu) thread_idx_x)) "
     "(read b (binop add (intrinsic (Gpu) thread_idx_x) (const i32 1))))))", "other than the element index"),   # stencil read
    ("(kernel k (params (vec a 1 f32)) (body (while (const bool true) (empty))))", "while"),
    ("(kernel k (params (vec a 1 i32) (vec b 2 i32)) (body (assign (elem a (intrinsic (Gpu) thread_idx_x)) (read b (intrinsic (Gpu) thread_idx_x)))))", "float32"),
])
def test_unrecognised_kernels_raise_unsupported_construct(ir, why):
    with pytest.raises(UnsupportedConstruct) as e:
        compile_(ir)
    assert e.value.code == L.ERR_UNSUPPORTED and why in e.value.message


@pytest.mark.parametrize("text", ["", "(kernel", "(kernel k (params) (body (empty))) trailing", "(notakernel)", "(kernel k (params (vec a)) (body (empty)))"])
def test_malformed_ir_is_a_parse_error(text):
    with pytest.raises(BackendError) as e:
        compile_(text)
    assert e.value.code == L.ERR_PARSE


def test_argument_binding_errors_are_reported_before_any_device_work():
    b = Backend()
    k = compile_(S.stream_triad_ir())
    buf = b.Memory.Buffer(0, 4096, 16, 4)

    def launch(build):
        ka = b.Kernel.create_args()
        build(ka)
        b.Kernel.launch(k, args=ka, grid=dims1d(1), block=dims1d(32))

    def good_prefix(ka):
        for _ in range(3):
            b.Kernel.set_arg_buffer(ka, 0, buf)
            b.Kernel.set_arg_int32(ka, 0, 16)

    with pytest.raises(BackendError) as e:   # too few
        launch(good_prefix)
    assert e.value.code == L.ERR_ARGS

    def wrong_scalar(ka):
        good_prefix(ka)
        b.Kernel.set_arg_int32(ka, 0, 3)     # scalar is float32
        b.Kernel.set_arg_int32(ka, 0, 16)
    with pytest.raises(BackendError) as e:
        launch(wrong_scalar)
    assert e.value.code == L.ERR_ARGS

    def missing_length(ka):
        b.Kernel.set_arg_buffer(ka, 0, buf)
        b.Kernel.set_arg_buffer(ka, 0, buf)
    with pytest.raises(BackendError) as e:
        launch(missing_length)
    assert e.value.code == L.ERR_ARGS

    def too_many(ka):
        good_prefix(ka)
        b.Kernel.set_arg_float32(ka, 0, 3.0)
        b.Kernel.set_arg_int32(ka, 0, 16)
        b.Kernel.set_arg_int32(ka, 0, 16)
    with pytest.raises(BackendError) as e:
        launch(too_many)
    assert e.value.code == L.ERR_ARGS


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(os.path.dirname(L.HERE), "include", "sb200.h")).read()
    declared = set(re.findall(r"SB200_API\s+(?:const\s+)?\w+\s*\*?\s*(sb200_\w+)\s*\(", header))
    assert len(declared) >= 45
    lib = L.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in sb200.h but not exported"
    assert declared == set(L.SIGNATURES), declared ^ set(L.SIGNATURES)
    assert lib.sb200_version() == 100


def test_no_gpu_means_errors_not_fallbacks():
    """Without a device the library reports it; nothing computes on the CPU."""
    b = Backend()
    if b.Device.count() > 0:
        pytest.skip("a GPU is present")
    lib = L.load()
    assert not b.is_available()
    assert lib.sb200_init() == L.ERR_NO_DEVICE
    assert lib.sb200_vector_add_f32(0, 0, 16, 16, 16, 4) == L.ERR_NO_DEVICE
    assert lib.sb200_gemm_f32(0, 0, 3, 4, 4, 4, 16, 4, 16, 4, 16, 4, 1.0, 0, 0, 0.0, 0, 0) == L.ERR_NO_DEVICE
    assert lib.sb200_gemm_f32_noalloc(0, 0, 3, 4, 4, 4, 16, 4, 16, 4, 16, 4, 1.0, 0, 0, 0.0, 0, 0) == L.ERR_NO_DEVICE
    p = C.c_uint64(0)
    assert lib.sb200_mem_alloc(0, 64, C.byref(p)) == L.ERR_NO_DEVICE
    assert b"CUDA" in lib.sb200_last_error_string() or b"device" in lib.sb200_last_error_string()
    n = C.c_uint64(0)
    assert lib.sb200_gemm_workspace_bytes(3, 8192, 8192, 8192, C.byref(n)) == 0 and n.value == 4 * 8192 * 8192 * 4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "libsarek_b200.so"))
    with pytest.raises(L.LibraryMissing):
        L.load()


def test_mode_setting():
    b = Backend()
    b.set_mode(L.MODE_TF32)
    assert b.get_mode() == L.MODE_TF32
    b.set_mode(L.MODE_3XTF32)
    assert b.get_mode() == L.MODE_3XTF32
    for mode in (L.MODE_3XF16, L.MODE_F16, L.MODE_3XMIXED, L.MODE_3XTF32):
        b.set_mode(mode)
        assert b.get_mode() == mode
    with pytest.raises(BackendError):
        b.set_mode(6)


@pytest.mark.parametrize("find,replace", [
    ("(elem c (evar tid 5))", "(elem (evar tid 5))"),            # array name missing
    ("(read a (evar tid 5))", "(read a)"),                       # index missing
    ("(binop add ", "(binop add add "),                          # an atom where an expression belongs
    ("(evar n 4)", "(evar n)"),
    ("(let tid 5 i32 ", "(let tid 5 "),
    ("(sif ", "(sif) (sif "),                                     # a condition-less if, and a let with two bodies
    ("(intrinsic (Gpu) global_thread_id)", "(intrinsic Gpu global_thread_id)"),
])
def test_malformed_forms_are_parse_errors(find, replace):
    """Every form is checked against the grammar before the recogniser or the fusion pass indexes into it."""
    from spoc_b200 import fusion as F
    ir = S.vector_add_ir()
    assert find in ir
    bad = ir.replace(find, replace, 1)
    with pytest.raises(BackendError) as e:
        compile_(bad)
    assert e.value.code == L.ERR_PARSE and "malformed IR form" in str(e.value)
    with pytest.raises(BackendError):
        F.analyze(bad)
    with pytest.raises(BackendError):
        F.fuse_guarded(bad, S.square_add_guarded_ir(), "c")


def test_forms_outside_the_grammar_are_unsupported_not_malformed():
    ir = S.vector_add_ir().replace("(sif ", "(seq (match (evar n 4) (case 0 (empty))) (sif ", 1).replace("))))", ")))))", 1)
    with pytest.raises(UnsupportedConstruct):
        compile_(ir)


@pytest.mark.parametrize("find,replace,needle", [
    ("(let tid 5 i32 (intrinsic (Gpu) global_thread_id) ", "(let dead 9 f32 (read y (evar tid 5)) (let tid 5 i32 (intrinsic (Gpu) global_thread_id) ", None),
    ("(read a (evar tid 5))", "(read zz (evar tid 5))", "array 'zz'"),
    ("(elem c (evar tid 5))", "(elem out (evar tid 5))", "array 'out'"),
    ("(evar n 4)", "(evar n 44)", "variable 'n'"),
])
def test_kernels_must_declare_what_they_use(find, replace, needle):
    """Even in a binding nothing uses: the recogniser never looks at dead lets, the binding check does."""
    ir = S.vector_add_ir()
    assert find in ir
    bad = ir.replace(find, replace, 1)
    if needle is None:
        bad += ")"                      # the extra let needs its closing parenthesis
        needle = "array 'y'"            # read by a binding that nothing uses
    with pytest.raises(BackendError) as e:
        compile_(bad)
    assert e.value.code == L.ERR_PARSE and needle in str(e.value) and "does not declare" in str(e.value)


TILED_WRONG = [
    # (what, find, replace): each changes what the kernel computes while keeping its overall look
    ("A read with the wrong row stride", "(read a (binop add (binop mul (evar row 11) (evar k 6)) (evar a_col 17)))",
     "(read a (binop add (binop mul (evar row 11) (evar n 5)) (evar a_col 17)))"),
    ("A column taken from ty", "(let a_col 17 i32 (binop add (binop mul (evar t 16) (evar tile_size 13)) (evar tx 9))",
     "(let a_col 17 i32 (binop add (binop mul (evar t 16) (evar tile_size 13)) (evar ty 10))"),
    ("B row guard against n", "(binop lt (evar b_row 18) (evar k 6))", "(binop lt (evar b_row 18) (evar n 5))"),
    ("A guard dropped to one half", "(binop and (binop lt (evar row 11) (evar m 4)) (binop lt (evar a_col 17) (evar k 6)))",
     "(binop and (binop lt (evar row 11) (evar m 4)) (binop lt (evar row 11) (evar m 4)))"),
    ("tile_b stored transposed", "(assign (elem tile_b (binop add (binop mul (evar ty 10) (evar tile_size 13)) (evar tx 9))) (read b",
     "(assign (elem tile_b (binop add (binop mul (evar tx 9) (evar tile_size 13)) (evar ty 10))) (read b"),
    ("inner product walks tile_a by column", "(read tile_a (binop add (binop mul (evar ty 10) (evar tile_size 13)) (evar i 19)))",
     "(read tile_a (binop add (binop mul (evar i 19) (evar tile_size 13)) (evar ty 10)))"),
    ("one k-tile too few", "(for t 16 (const i32 0) (binop sub (evar num_tiles 14) (const i32 1)) upto",
     "(for t 16 (const i32 0) (binop sub (evar num_tiles 14) (const i32 2)) upto"),
    ("k-tiles start at 1", "(for t 16 (const i32 0) ", "(for t 16 (const i32 1) "),
    ("inner loop one short", "(for i 19 (const i32 0) (binop sub (evar tile_size 13) (const i32 1)) upto",
     "(for i 19 (const i32 0) (binop sub (evar tile_size 13) (const i32 2)) upto"),
    ("barrier between the loads and the product missing",
     "(const f32 0.0))))) (barrier) (seq (block (for i 19", "(const f32 0.0))))) (empty) (seq (block (for i 19"),
    ("out-of-range elements of A not zeroed", "(evar tx 9))) (const f32 0.0))))) (barrier) (seq (block (let b_row",
     "(evar tx 9))) (const f32 1.0))))) (barrier) (seq (block (let b_row"),
    ("shared tile too small", "(let tile_a 7 (array f32 shared) (arraycreate f32 (const i32 256) shared)",
     "(let tile_a 7 (array f32 shared) (arraycreate f32 (const i32 128) shared)"),
    ("row taken from the x index", "(let row 11 i32 (binop add (evar ty 10) (binop mul (intrinsic (Gpu) block_dim_y) (intrinsic (Gpu) block_idx_y)))",
     "(let row 11 i32 (binop add (evar tx 9) (binop mul (intrinsic (Gpu) block_dim_x) (intrinsic (Gpu) block_idx_x)))"),
]


@pytest.mark.parametrize("what,find,replace", TILED_WRONG, ids=[w for w, _, _ in TILED_WRONG])
def test_tiled_kernels_that_compute_something_else_are_not_taken_for_gemm(what, find, replace):
    ir = S.matmul_tiled_ir()
    assert ir.count(find) >= 1, what
    with pytest.raises(UnsupportedConstruct):
        compile_(ir.replace(find, replace, 1))


def test_equivalent_spellings_of_the_tiled_kernel_are_recognised():
    ir = S.matmul_tiled_ir()
    same = [
        # index arithmetic commuted and the global indices taken from the intrinsics
        ir.replace("(binop add (binop mul (evar row 11) (evar k 6)) (evar a_col 17))", "(binop add (evar a_col 17) (binop mul (evar k 6) (evar row 11)))"),
        ir.replace("(let row 11 i32 (binop add (evar ty 10) (binop mul (intrinsic (Gpu) block_dim_y) (intrinsic (Gpu) block_idx_y)))",
                   "(let row 11 i32 (intrinsic (Gpu) global_idx_y)"),
        ir.replace("(binop add (binop mul (evar t 16) (evar tile_size 13)) (evar ty 10))", "(binop add (evar ty 10) (binop mul (const i32 16) (evar t 16)))"),
        ir.replace("(binop and (binop lt (evar b_row 18) (evar k 6)) (binop lt (evar col 12) (evar n 5)))",
                   "(binop and (binop lt (evar col 12) (evar n 5)) (binop lt (evar b_row 18) (evar k 6)))"),
        ir.replace("(binop mul (read tile_a (binop add (binop mul (evar ty 10) (evar tile_size 13)) (evar i 19))) (read tile_b (binop add (binop mul (evar i 19) (evar tile_size 13)) (evar tx 9))))",
                   "(binop mul (read tile_b (binop add (evar tx 9) (binop mul (evar tile_size 13) (evar i 19)))) (read tile_a (binop add (evar i 19) (binop mul (evar tile_size 13) (evar ty 10)))))"),
    ]
    for text in same:
        assert text != ir
        k = compile_(text)
        assert k.kind == L.KIND_GEMM_TILED and "tile=16" in k.describe()


def test_reduction_whose_shared_array_is_too_short_is_rejected():
    ir = S.block_reduce_ir("sum", 64)
    assert "(arraycreate f32 (const i32 64) shared)" in ir
    with pytest.raises(UnsupportedConstruct):
        compile_(ir.replace("(arraycreate f32 (const i32 64) shared)", "(arraycreate f32 (const i32 32) shared)"))


def _parse_sx(text):
    toks = text.replace("(", " ( ").replace(")", " ) ").split()
    pos = 0

    def rd():
        nonlocal pos
        if toks[pos] == "(":
            pos += 1
            out = []
            while toks[pos] != ")":
                out.append(rd())
            pos += 1
            return out
        pos += 1
        return toks[pos - 1]
    return rd()


def _show_sx(x):
    return "(" + " ".join(_show_sx(i) for i in x) + ")" if isinstance(x, list) else x


def _subtrees(x, heads, acc, parent=None, idx=None):
    if isinstance(x, list):
        if x and isinstance(x[0], str) and x[0] in heads and parent is not None:
            acc.append((parent, idx))
        for i, k in enumerate(x):
            _subtrees(k, heads, acc, x, i)
    return acc


@pytest.mark.parametrize("seed", [0, 1])
def test_mutated_kernels_never_crash_the_entry_points(seed):
    """Seeded mutation fuzz of the text entry points: characters and tokens dropped, swapped or inserted, and
    sub-expressions / statements of one reference kernel grafted into another.  Every call must come back with
    success, SB200_ERR_UNSUPPORTED or SB200_ERR_PARSE (a crash would take the test process down)."""
    import copy
    import random
    from spoc_b200 import fusion as F
    lib = L.load()
    rnd = random.Random(seed)
    texts = [S.vector_add_ir(), S.stream_triad_ir(), S.matmul_naive_ir(), S.matmul_tiled_ir(), S.chain_fused_ir(), S.generic_example_ir(),
             S.block_reduce_ir("dot"), S.square_add_guarded_ir(), S.matmul_tiled_ir(epilogue=EPI)]
    trees = [_parse_sx(t) for t in texts]
    exprs = {"const", "evar", "binop", "unop", "read", "intrinsic", "if"}
    stmts = {"assign", "seq", "sif", "for", "let", "letmut", "block", "barrier", "empty"}
    out = C.create_string_buffer(1 << 20)
    seen = set()
    for it in range(400):
        if it % 2:
            t = rnd.choice(texts)
            toks = t.replace("(", " ( ").replace(")", " ) ").split()
            k = rnd.randrange(5)
            if k == 0:
                t = t[:rnd.randrange(1, len(t))]
            elif k == 1:
                del toks[rnd.randrange(len(toks))]
                t = " ".join(toks)
            elif k == 2:
                i, j = rnd.randrange(len(toks)), rnd.randrange(len(toks))
                toks[i], toks[j] = toks[j], toks[i]
                t = " ".join(toks)
            elif k == 3:
                toks.insert(rnd.randrange(len(toks)), rnd.choice(["(", ")", "evar", "read", "-1", "()", "f32", "let", "99999999999999999999"]))
                t = " ".join(toks)
            else:
                i = rnd.randrange(len(toks))
                t = " ".join(toks[:i] + toks[min(len(toks), i + rnd.randrange(1, 30)):])
        else:
            tree = copy.deepcopy(rnd.choice(trees))
            for _ in range(rnd.randrange(1, 4)):
                heads = rnd.choice([exprs, stmts])
                here, donor = _subtrees(tree[3], heads, []), _subtrees(copy.deepcopy(rnd.choice(trees))[3], heads, [])
                if here and donor:
                    (p, i), (dp, di) = rnd.choice(here), rnd.choice(donor)
                    p[i] = dp[di]
            t = _show_sx(tree)
        h = C.c_uint64(0)
        rc = lib.sb200_kernel_compile(0, t.encode(), b"k", C.byref(h))
        assert rc in (0, L.ERR_UNSUPPORTED, L.ERR_PARSE), (rc, t[:200])
        seen.add(rc)
        if rc == 0:
            assert lib.sb200_kernel_destroy(h.value) == 0
        assert lib.sb200_ir_analyze(t.encode(), out, 1 << 20) in (0, L.ERR_PARSE)
        other = rnd.choice(texts).encode()
        fused = C.c_int(0)
        for kind in range(6):
            for a, b in ((t.encode(), other), (other, t.encode())):
                assert lib.sb200_ir_fuse_as(a, b, rnd.choice([b"a", b"c", b"d", b"sdata"]), kind, out, 1 << 20, C.byref(fused)) in (0, L.ERR_PARSE)
    assert seen == {0, L.ERR_UNSUPPORTED, L.ERR_PARSE}
