"""The fusion pass on IR text against the behaviour the reference's own tests pin
(sarek/tests/unit/test_fusion.ml, sarek/tests/e2e/test_fusion_api.ml)."""
import pytest

from spoc_b200 import fusion as F
from spoc_b200 import sarek_ir as S

TX = ("intrinsic", ("Gpu",), "thread_idx_x")


def kern(name, body, params=()):
    return S.sx(("kernel", name, ("params",) + tuple(params), ("body", body)))


def c_i32(v):
    return ("const", "i32", v)


def scale(name, dst, src, op, k):
    return kern(name, ("assign", ("elem", dst, TX), ("binop", op, ("read", src, TX), c_i32(k))),
                [("vec", dst, 1, "i32"), ("vec", src, 2, "i32")])


PRODUCER = scale("producer", "temp", "input", "mul", 2)
CONSUMER = scale("consumer", "output", "temp", "add", 1)


def test_analyze_one_to_one():          # test_fusion.ml:21-46
    info = F.analyze(scale("scale", "output", "input", "mul", 2))
    assert info["reads"] == {"input": "one_to_one"} and info["writes"] == {"output": "one_to_one"}
    assert not info["has_barriers"]


def test_analyze_with_barrier():        # test_fusion.ml:49-76
    body = ("seq", ("assign", ("elem", "shared", TX), ("read", "input", TX)), ("barrier",),
            ("assign", ("elem", "output", TX), ("read", "shared", TX)))
    assert F.analyze(kern("with_barrier", body))["has_barriers"]


def test_can_fuse_compatible_and_barrier():   # test_fusion.ml:79-156
    assert F.can_fuse(PRODUCER, CONSUMER, "temp")
    with_barrier = kern("producer", ("seq", ("assign", ("elem", "temp", TX), ("read", "input", TX)), ("barrier",)))
    assert not F.can_fuse(with_barrier, CONSUMER, "temp")
    assert not F.can_fuse(PRODUCER, CONSUMER, "other")


def test_fuse_simple():                 # test_fusion.ml:159-202
    fused = F.fuse(PRODUCER, CONSUMER, "temp")
    assert fused.startswith("(kernel consumer_fused ")
    info = F.analyze(fused)
    assert "temp" not in info["reads"] and "input" in info["reads"] and "output" in info["writes"]
    # the intermediate leaves the parameter list, the producer's input joins it
    assert "(vec temp" not in fused and "(vec input" in fused
    # output[i] = (input[i] * 2) + 1
    assert "(binop add (binop mul (read input" in fused


def test_fuse_pipeline_eliminates_both_intermediates():   # test_fusion.ml:205-267, test_fusion_api.ml:52-81
    k1, k2, k3 = scale("k1", "a", "input", "mul", 2), scale("k2", "b", "a", "add", 1), scale("k3", "output", "b", "mul", 3)
    fused, eliminated = F.fuse_pipeline([k1, k2, k3])
    assert set(eliminated) == {"a", "b"} and eliminated == ["b", "a"]   # newest first, like the reference's cons
    info = F.analyze(fused)
    assert "input" in info["reads"] and "output" in info["writes"] and "a" not in info["reads"] and "b" not in info["reads"]
    assert fused.startswith("(kernel k3_fused ")   # consumer name + "_fused" at each step: k2_fused, then k3_fused
    single, none = F.fuse_pipeline([k1])
    assert none == [] and single.startswith("(kernel k1 ")


def test_fuse_leaves_consumer_alone_when_write_is_conditional():   # find_write_expr, Sarek_fusion.ml:360-378
    guarded = kern("producer", ("sif", ("binop", "lt", TX, c_i32(10)), ("assign", ("elem", "temp", TX), ("read", "input", TX))))
    out = F.fuse(guarded, CONSUMER, "temp")
    assert out.startswith("(kernel consumer ") and "(read temp" in out


def stencil_consumer(offsets):
    e = None
    for o in offsets:
        idx = TX if o == 0 else ("binop", "add" if o > 0 else "sub", TX, c_i32(abs(o)))
        r = ("read", "temp", idx)
        e = r if e is None else ("binop", "add", e, r)
    return kern("consumer", ("assign", ("elem", "output", TX), e))


def test_should_fuse_decisions():       # test_fusion.ml:712-833
    assert F.should_fuse(PRODUCER, CONSUMER, "temp")[0] == "Fuse"
    with_barrier = kern("producer", ("seq", ("assign", ("elem", "temp", TX), ("read", "input", TX)), ("barrier",)))
    assert F.should_fuse(with_barrier, CONSUMER, "temp") == ("DontFuse", "Barrier prevents fusion")
    assert F.should_fuse(PRODUCER, stencil_consumer([-1, 0, 1]), "temp")[0] == "MaybeFuse"
    assert F.should_fuse(PRODUCER, stencil_consumer([-2, -1, 0, 1, 2]), "temp")[0] == "DontFuse"
    gather = kern("consumer", ("assign", ("elem", "output", TX),
                               ("binop", "add", ("read", "temp", ("read", "index", TX)), ("read", "temp", TX))))
    assert F.should_fuse(PRODUCER, gather, "temp") == ("DontFuse", "Gather pattern - keep separate")
    assert F.analyze(stencil_consumer([-1, 0, 1]))["reads"]["temp"] == "stencil[-1,0,1]"


def test_auto_fuse_pipeline():          # test_fusion.ml:836-943
    k1, k2, k3 = scale("k1", "a", "input", "mul", 2), scale("k2", "b", "a", "add", 1), scale("k3", "output", "b", "mul", 3)
    fused, eliminated, skipped = F.auto_fuse_pipeline([k1, k2, k3])
    assert set(eliminated) == {"a", "b"} and skipped == []
    k_st = kern("k2", ("assign", ("elem", "output", TX),
                       ("binop", "add", ("read", "temp", ("binop", "sub", TX, c_i32(1))),
                        ("read", "temp", ("binop", "add", TX, c_i32(1))))))
    _, eliminated, skipped = F.auto_fuse_pipeline([PRODUCER, k_st])
    assert eliminated == [] and len(skipped) == 1


def reduce_kernel(arr="temp"):
    loop = ("for", "i", 1, c_i32(0), c_i32(100), "upto",
            ("assign", ("lvar", "sum", 2), ("binop", "add", ("evar", "sum", 2), ("read", arr, ("evar", "i", 1)))))
    return kern("reduce", ("seq", ("assign", ("lvar", "sum", 2), c_i32(0)), loop), [("vec", arr, 5, "i32")])


def test_reduction_fusion():            # test_fusion.ml:298-522
    m = scale("map", "temp", "input", "mul", 2)
    r = reduce_kernel()
    assert F.can_fuse_reduction(m, r, "temp")
    assert not F.can_fuse_reduction(m, reduce_kernel("other"), "temp")
    fused = F.fuse_reduction(m, r, "temp")
    assert fused.startswith("(kernel reduce_fused ")
    assert "temp" not in F.analyze(fused)["reads"] and "(vec temp" not in fused and "(vec input" in fused
    # the fold keeps its structure, with the map's expression at each step
    assert "(binop add (evar sum 2) (binop mul (read input" in fused
    assert F.try_fuse(m, r, "temp") == fused            # try_fuse prefers the reduction form
    assert F.try_fuse(PRODUCER, CONSUMER, "temp") == F.fuse(PRODUCER, CONSUMER, "temp")
    assert F.try_fuse(PRODUCER, stencil_consumer([-1, 1]), "temp") is None


def test_stencil_fusion():              # test_fusion.ml:525-710
    cons = stencil_consumer([-1, 1])
    assert F.can_fuse_stencil(PRODUCER, cons, "temp")
    fused = F.fuse_stencil(PRODUCER, cons, "temp")
    assert fused.startswith("(kernel consumer_stencil_fused ")
    info = F.analyze(fused)
    assert "temp" not in info["reads"] and info["reads"]["input"] == "stencil[-1,1]"
    # temp[i-1] became input[i-1] * 2: the producer's expression shifted by the read's offset
    assert "(binop mul (read input (binop sub (intrinsic (Gpu) thread_idx_x) (const i32 1))) (const i32 2))" in fused
    # try_fuse_all: stencil fusion also takes the one-to-one case, before plain fusion is tried
    out = F.try_fuse_all(PRODUCER, CONSUMER, "temp")
    assert out is not None and out.startswith("(kernel consumer_stencil_fused ")
    gather = kern("consumer", ("assign", ("elem", "output", TX),
                               ("binop", "add", ("read", "temp", ("read", "index", TX)), ("read", "temp", TX))))
    assert F.try_fuse_all(PRODUCER, gather, "temp") is None


def test_config2_chain_through_try_fuse_all():
    """The route that does fuse a = b + 3c ; d = a*a + b automatically: try_fuse_all takes the stencil branch
    (offsets [0]) and yields the same body as a direct fuse."""
    p, c = S.triad_producer_ir(3.0), S.square_add_consumer_ir()
    out = F.try_fuse_all(p, c, "a")
    assert out is not None and out.startswith("(kernel square_add_stencil_fused ")
    assert out.replace("square_add_stencil_fused", "square_add_fused") == F.fuse(p, c, "a")


def test_config2_chain_behaves_like_the_reference():
    """a = b + 3c ; d = a*a + b: the consumer reads `a` twice, which the reference classifies as a
    stencil with offsets [0] (Sarek_fusion.ml:301-322): can_fuse is false, should_fuse says MaybeFuse,
    fuse_pipeline skips it, and a direct fuse rewrites both reads."""
    p, c = S.triad_producer_ir(3.0), S.square_add_consumer_ir()
    assert F.analyze(c)["reads"]["a"] == "stencil[0]"
    assert not F.can_fuse(p, c, "a")
    assert F.should_fuse(p, c, "a")[0] == "MaybeFuse"
    assert F.fuse_pipeline([p, c])[1] == []
    fused = F.fuse(p, c, "a")
    assert "(read a" not in fused and "(vec a" not in fused and fused.startswith("(kernel square_add_fused ")
    assert fused == S.chain_fused_ir(3.0)


def test_errors():
    from spoc_b200 import BackendError
    with pytest.raises(BackendError):
        F.fuse("(kernel", CONSUMER, "temp")
    with pytest.raises(BackendError):
        F.fuse_pipeline([])


# ---- guarded fusion: this backend's extension for the reference's own benchmark kernel form ----

def test_reference_pass_leaves_guarded_benchmark_kernels_unfused():
    """Sarek_fusion.ml:370-375: find_write_expr returns None inside SIf, so fuse gives the consumer back."""
    prod, cons = S.stream_triad_ir("triad"), S.square_add_guarded_ir()
    assert not F.can_fuse(prod, cons, "a")
    for out in (F.fuse(prod, cons, "a"), F.try_fuse_all(prod, cons, "a")):
        assert "(read a" in out and "(read c" not in out     # the consumer comes back, still reading the intermediate


def test_guarded_fusion_of_the_benchmark_kernel_form():
    prod, cons = S.stream_triad_ir("triad"), S.square_add_guarded_ir()
    assert F.can_fuse_guarded(prod, cons, "a")
    fused = F.fuse_guarded(prod, cons, "a")
    assert fused.startswith("(kernel square_add_fused ")
    assert "(read a" not in fused and "(vec a " not in fused        # intermediate eliminated
    assert fused.count("(read c ") == 2 and fused.count("(read b ") == 3
    assert "(sif (binop lt (intrinsic (Gpu) global_thread_id) (evar n 4))" in fused   # consumer's guard and its n
    # parameters: the consumer's without the intermediate, then the producer's that are new by name
    names = [p.split()[1] for p in fused.split("(params ")[1].split("(body")[0].split("(")[1:]]
    assert names == ["d", "b", "n", "c", "scalar"]
    info = F.analyze(fused)
    assert info["writes"] == {"d": "one_to_one"} and set(info["reads"]) == {"b", "c"}


def test_guarded_fusion_accepts_an_unguarded_producer_and_chains():
    prod = S.triad_producer_ir()                   # unguarded store at global_thread_id
    fused = F.fuse_guarded(prod, S.square_add_guarded_ir(), "a")
    assert fused is not None and "(read a" not in fused and "(sif " in fused
    # a three-kernel chain: (triad ; square_add) ; e = d + d
    b = S.Builder()
    p = b.params([("vec", "e", "f32"), ("vec", "d", "f32"), ("scalar", "n", "i32")])
    body = b.let("i", "i32", b.intr("global_thread_id"), lambda: (
        "sif", b.binop("lt", b.evar("i"), b.evar("n")),
        ("assign", ("elem", "e", b.evar("i")), b.binop("add", b.read("d", b.evar("i")), b.read("d", b.evar("i"))))))
    third = S.sx(("kernel", "twice", p, ("body", body)))
    both = F.fuse_guarded(F.fuse_guarded(S.stream_triad_ir("triad"), S.square_add_guarded_ir(), "a"), third, "d")
    assert both is not None and both.startswith("(kernel twice_fused ")
    assert "(read d" not in both and "(read a" not in both and both.count("(read c ") == 4


@pytest.mark.parametrize("case,needle", [
    ("guards_differ", "guard differs"),
    ("other_index", "index other than"),
    ("unguarded_consumer", "guard differs"),
    ("barrier", "barrier"),
    ("not_read", "does not read"),
    ("local_variable", "local variable"),
])
def test_guarded_fusion_refuses_with_a_reason(case, needle):
    prod, cons = S.stream_triad_ir("triad"), S.square_add_guarded_ir()
    if case == "guards_differ":
        cons = cons.replace("(evar n 4)", "(evar m 4)").replace("(scalar n 4 i32)", "(scalar m 4 i32)")
    elif case == "other_index":
        cons = cons.replace("(read a (evar tid 5)) (read a (evar tid 5))",
                            "(read a (evar tid 5)) (read a (binop add (evar tid 5) (const i32 1)))")
    elif case == "unguarded_consumer":
        cons = S.square_add_consumer_ir()
    elif case == "barrier":
        cons = cons.replace("(body ", "(body (seq (barrier) ").replace(")))", "))))", 1)[:-0] if False else \
            S.sx(("kernel", "k", ("params", ("vec", "d", 1, "f32"), ("vec", "a", 2, "f32")),
                  ("body", ("seq", ("barrier",), ("assign", ("elem", "d", TX), ("read", "a", TX))))))
    elif case == "not_read":
        cons = S.vector_add_ir("add").replace("(read a ", "(read z ").replace("(vec a ", "(vec z ")
    elif case == "local_variable":
        # producer:  let x = b[tid] in a[tid] <- x + x   (a let that reads an array stays in place)
        b = S.Builder()
        p = b.params([("vec", "a", "f32"), ("vec", "b", "f32"), ("scalar", "n", "i32")])
        body = b.let("tid", "i32", b.intr("global_thread_id"), lambda: (
            "sif", b.binop("lt", b.evar("tid"), b.evar("n")),
            b.let("x", "f32", b.read("b", b.evar("tid")), lambda:
                  ("assign", ("elem", "a", b.evar("tid")), b.binop("add", b.evar("x"), b.evar("x"))))))
        prod = S.sx(("kernel", "p", p, ("body", body)))
    assert not F.can_fuse_guarded(prod, cons, "a")
    assert needle in F.why_not_fused()
    assert F.fuse_guarded(prod, cons, "a") is None


def test_pipeline_of_guarded_benchmark_kernels_collapses_into_one_kernel():
    b = S.Builder()
    p = b.params([("vec", "e", "f32"), ("vec", "d", "f32"), ("scalar", "n", "i32")])
    body = b.let("i", "i32", b.intr("global_thread_id"), lambda: (
        "sif", b.binop("lt", b.evar("i"), b.evar("n")),
        ("assign", ("elem", "e", b.evar("i")), b.binop("mul", b.read("d", b.evar("i")), b.c_f32(0.5)))))
    third = S.sx(("kernel", "halve", p, ("body", body)))
    chain = [S.stream_triad_ir("triad"), S.square_add_guarded_ir(), third]
    fused, eliminated = F.fuse_pipeline_as(chain, F.GUARDED)
    assert fused.startswith("(kernel halve_fused ") and eliminated == ["d", "a"]       # newest first, as the reference lists them
    assert "(read a" not in fused and "(read d" not in fused
    # the reference's own pipeline fuses nothing here: it hands back the last kernel, still reading d (and, since
    # can_fuse holds for a single guarded read, lists d as eliminated all the same — Sarek_fusion.ml:590-593)
    plain, eliminated = F.fuse_pipeline(chain)
    assert plain.startswith("(kernel halve ") and "(read d" in plain and eliminated == ["d"]
    assert F.fuse_pipeline_as(chain, F.PLAIN) == (plain, eliminated)
