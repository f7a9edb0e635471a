"""GPU parity of the fused-map kernels against the Native-semantics oracle.

Bar: <= 1 ulp on every element (the GPU rounds once per fused multiply-add, the
Native backend rounds a double result once: they differ only in double-rounding
corner cases), bit-exact for vector_add.
"""
import ctypes as C
import os

import numpy as np
import pytest

from spoc_b200 import BackendError, Vector, dims1d, run_vectors, sarek_ir
from spoc_b200 import _lib as L
from spoc_b200.plugin import _check
from tests import oracle_lib as O
from tests.gpu_util import CANARY, Dev, dev_from

pytestmark = pytest.mark.gpu

SIZES = [1, 2, 3, 4, 5, 7, 8, 31, 32, 33, 255, 256, 257, 1023, 1024, 1025, 4099, (1 << 20) + 3]


def _inputs(n, seed=7):
    return O.fill(n, seed, 2), O.fill(n, seed, 3)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("offset", [0, 1, 3])
def test_direct_ops_match_oracle(backend, device, oracle, n, offset):
    lib = L.load()
    b, c = _inputs(n)
    db, dc = dev_from(backend, device, b, offset=offset), dev_from(backend, device, c, offset=offset)
    out, keep = Dev(backend, device, n, offset=offset), Dev(backend, device, n, offset=offset)
    try:
        # vector_add: bit-exact
        _check(lib.sb200_vector_add_f32(device.id, 0, out.ptr, db.ptr, dc.ptr, n))
        ref = np.empty(n, np.float32)
        oracle.so_vector_add(b, c, ref, n)
        assert np.array_equal(out.download(), ref)
        # triad
        out.clear()
        _check(lib.sb200_stream_triad_f32(device.id, 0, out.ptr, db.ptr, dc.ptr, 3.0, n))
        oracle.so_stream_triad(ref, b, c, 3.0, n)
        assert O.ulp_distance(out.download(), ref).max() <= 1
        # fused chain, intermediate eliminated and kept
        out.clear()
        _check(lib.sb200_chain_triad_square_f32(device.id, 0, out.ptr, 0, db.ptr, dc.ptr, 3.0, n))
        ref_a = np.empty(n, np.float32)
        oracle.so_chain_triad_square(ref, ref_a.ctypes.data_as(C.c_void_p), b, c, 3.0, n)
        got = out.download()
        assert O.ulp_distance(got, ref).max() <= 1
        out.clear()
        _check(lib.sb200_chain_triad_square_f32(device.id, 0, out.ptr, keep.ptr, db.ptr, dc.ptr, 3.0, n))
        assert np.array_equal(out.download(), got)
        assert O.ulp_distance(keep.download(), ref_a).max() <= 1
    finally:
        for d in (db, dc, out, keep):
            d.free()


def test_mixed_alignment_takes_scalar_path(backend, device, oracle):
    lib = L.load()
    n = 5000
    b, c = _inputs(n, seed=11)
    db, dc, out = dev_from(backend, device, b, offset=1), dev_from(backend, device, c, offset=2), Dev(backend, device, n, offset=3)
    _check(lib.sb200_stream_triad_f32(device.id, 0, out.ptr, db.ptr, dc.ptr, 3.0, n))
    ref = np.empty(n, np.float32)
    oracle.so_stream_triad(ref, b, c, 3.0, n)
    assert O.ulp_distance(out.download(), ref).max() <= 1


def test_zero_length_and_errors(backend, device):
    lib = L.load()
    assert lib.sb200_vector_add_f32(device.id, 0, 0, 0, 0, 0) == 0
    assert lib.sb200_vector_add_f32(device.id, 0, 0, 0, 0, -1) == L.ERR_INVALID_VALUE
    assert lib.sb200_vector_add_f32(device.id, 0, 0, 0, 0, 8) == L.ERR_INVALID_VALUE


def test_stream_triad_reference_fixture(backend, device):
    """benchmarks/bench_stream_triad.ml:44-49,122: B=(i mod 100)/100, C=((i+1) mod 100)/100,
    scalar 3.0, expected b+c*3 in double from the un-rounded inputs, tolerance 1e-5."""
    n = 100000
    i = np.arange(n)
    b64, c64 = (i % 100) / 100.0, ((i + 1) % 100) / 100.0
    va, vb, vc = Vector.create(backend, n), Vector(backend, b64.astype(np.float32)), Vector(backend, c64.astype(np.float32))
    block, grid = dims1d(256), dims1d((n + 255) // 256)
    run_vectors(backend, device=device, ir=sarek_ir.stream_triad_ir(), args=[va, vb, vc, ("float32", 3.0), ("int32", n)],
                block=block, grid=grid)
    backend.Device.synchronize(device)
    assert va.location == Vector.STALE_CPU and vb.location == Vector.STALE_CPU
    got = va.to_array()
    assert np.max(np.abs(got - (b64 + c64 * 3.0))) <= 1e-5
    for v in (va, vb, vc):
        v.free()


def test_vector_add_reference_fixture(backend, device):
    """sarek/tests/e2e/test_vector_add.ml:31-49: a=i, b=2i, expected 3i, tolerance 1e-3;
    benchmarks/bench_vector_add.ml:68-71: a=i*0.001, b=i*0.002."""
    n = 4096
    i = np.arange(n, dtype=np.float64)
    for a64, b64 in ((i, 2 * i), (i * 0.001, i * 0.002)):
        va, vb, vc = Vector(backend, a64.astype(np.float32)), Vector(backend, b64.astype(np.float32)), Vector.create(backend, n)
        run_vectors(backend, device=device, ir=sarek_ir.vector_add_ir(), args=[va, vb, vc, ("int32", n)], block=dims1d(256),
                    grid=dims1d((n + 255) // 256))
        assert np.max(np.abs(vc.to_array() - (a64 + b64))) <= 1e-3
        for v in (va, vb, vc):
            v.free()


def test_launch_geometry_limits_the_elements_written(backend, device, oracle):
    """The reference kernel writes element tid only for tid < min(n, grid*block)."""
    n = 1000
    b, c = _inputs(n, seed=3)
    ref = np.empty(n, np.float32)
    oracle.so_stream_triad(ref, b, c, 3.0, n)
    for n_arg, blocks in ((600, 4), (1000, 2), (1000, 4)):
        va = Vector(backend, np.full(n, CANARY, np.float32))
        vb, vc = Vector(backend, b.copy()), Vector(backend, c.copy())
        run_vectors(backend, device=device, ir=sarek_ir.stream_triad_ir(), args=[va, vb, vc, ("float32", 3.0), ("int32", n_arg)],
                    block=dims1d(256), grid=dims1d(blocks))
        got = va.to_array()
        covered = min(n_arg, blocks * 256)
        assert O.ulp_distance(got[:covered], ref[:covered]).max() <= 1
        assert np.all(got[covered:] == CANARY)
        for v in (va, vb, vc):
            v.free()


def test_launch_past_vector_length_is_rejected(backend, device):
    n = 100
    va, vb, vc = Vector.create(backend, n), Vector.create(backend, n), Vector.create(backend, n // 2)
    with pytest.raises(BackendError) as e:
        run_vectors(backend, device=device, ir=sarek_ir.stream_triad_ir(), args=[va, vb, vc, ("float32", 3.0), ("int32", n)],
                    block=dims1d(128), grid=dims1d(1))
    assert e.value.code == L.ERR_BOUNDS
    for v in (va, vb, vc):
        v.free()


def test_length_larger_than_the_buffer_is_rejected(backend, device):
    """The caller states each vector's length; for a buffer the library allocated a length beyond the allocation is
    refused before anything is launched."""
    import ctypes as C
    from spoc_b200.plugin import RSA_Buffer, RSA_Float32, RSA_Int32
    n = 256
    bufs = [backend.Memory.alloc(device, n, np.float32) for _ in range(3)]
    short = backend.Memory.alloc(device, n // 2, np.float32)
    try:
        args = []
        for b, stated in ((bufs[0], n), (bufs[1], n), (short, n)):         # the third vector claims n elements in n/2
            args += [RSA_Buffer(b, stated), RSA_Int32(stated)]
        args += [RSA_Float32(3.0), RSA_Int32(n)]
        with pytest.raises(BackendError) as e:
            backend.run_source(source=sarek_ir.stream_triad_ir(), lang=backend.supported_source_langs[0], kernel_name="sarek_kern",
                               block=dims1d(256), grid=dims1d(1), shared_mem=0, args=args)
        assert e.value.code == L.ERR_BOUNDS and "the buffer it lies in ends after 512" in str(e.value)
    finally:
        for b in bufs + [short]:
            backend.Memory.free(b)


def test_fused_chain_ir_runs_in_one_pass(backend, device, oracle):
    """The kernel Sarek_fusion.fuse builds from a = b + 3c ; d = a*a + b (sarek/sarek/Sarek_fusion.ml:482-547),
    against Native's result of the two unfused kernels."""
    n = 256 * 782  # unguarded body: the launch must not cover more elements than the vectors hold
    b, c = _inputs(n, seed=5)
    vd, vb, vc = Vector.create(backend, n), Vector(backend, b.copy()), Vector(backend, c.copy())
    before = backend.launch_count()
    run_vectors(backend, device=device, ir=sarek_ir.chain_fused_ir(3.0), args=[vd, vb, vc], block=dims1d(256),
                grid=dims1d((n + 255) // 256 ))
    launches = backend.launch_count() - before
    got = vd.to_array()
    ref = np.empty(n, np.float32)
    oracle.so_chain_triad_square(ref, None, b, c, 3.0, n)
    assert launches <= 3
    d = O.ulp_distance(got, ref)
    assert d.max() <= 1
    assert (d == 0).mean() > 0.99
    for v in (vd, vb, vc):
        v.free()


def test_full_size_chain_every_element(backend, device, oracle):
    """N = 2^28 (the benchmark size), every element: the fused pass d = (b + 3c)^2 + b against the oracle's two
    unfused kernels (<= 1 ulp), the same pass with the intermediate kept (d2 must equal d bit for bit, a <= 1 ulp
    from the oracle's intermediate), and the device generator against the host generator (bit for bit).  The
    vectors are walked in chunks of 2^24 elements so that host memory stays bounded."""
    lib = L.load()
    n = 1 << 28
    bufs = [backend.Memory.alloc(device, n, np.float32) for _ in range(5)]
    b, c, d, a, d2 = bufs
    try:
        _check(lib.sb200_fill_f32(device.id, 0, b.ptr, n, 20260101, 2, 0, 1.0, 0))
        _check(lib.sb200_fill_f32(device.id, 0, c.ptr, n, 20260101, 3, 0, 1.0, 0))
        _check(lib.sb200_chain_triad_square_f32(device.id, 0, d.ptr, 0, b.ptr, c.ptr, 3.0, n))
        _check(lib.sb200_chain_triad_square_f32(device.id, 0, d2.ptr, a.ptr, b.ptr, c.ptr, 3.0, n))
        backend.Device.synchronize(device)
        blk = 1 << 24
        workers = max(1, (os.cpu_count() or 2) - 1)
        got = {k: np.empty(blk, np.float32) for k in "bcda2"}
        exact = total = 0
        for start in range(0, n, blk):
            hb, hc = O.fill(blk, 20260101, 2, first=start), O.fill(blk, 20260101, 3, first=start)
            for key, src in (("b", b), ("c", c), ("d", d), ("a", a), ("2", d2)):
                _check(lib.sb200_memcpy_dtoh(device.id, got[key].ctypes.data_as(C.c_void_p), src.ptr + 4 * start, 4 * blk))
            assert np.array_equal(got["b"], hb) and np.array_equal(got["c"], hc), "device fill differs from the host generator"
            ref, ref_a = np.empty(blk, np.float32), np.empty(blk, np.float32)
            oracle.so_par_chain_triad_square(ref, ref_a, hb, hc, 3.0, blk, workers)
            assert np.array_equal(got["d"], got["2"]), "eliminating the intermediate changed the result"
            dist = O.ulp_distance(got["d"], ref)
            assert dist.max() <= 1 and O.ulp_distance(got["a"], ref_a).max() <= 1
            exact += int((dist == 0).sum())
            total += blk
        assert exact / total > 0.99
    finally:
        for x in bufs:
            backend.Memory.free(x)


@pytest.mark.parametrize("n", [1, 5, 1000, 65537])
def test_generated_map_kernel_is_bit_exact_against_native_semantics(backend, device, n):
    """A map that is none of the ahead-of-time shapes is compiled at run time; it evaluates in double and
    rounds once per store like the Native backend, so it must match a float64 evaluation bit for bit."""
    rng = np.random.default_rng(n)
    x, y, z = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    vu, vv = Vector(backend, np.full(n, CANARY, np.float32)), Vector(backend, np.full(n, CANARY, np.float32))
    vx, vy, vz = Vector(backend, x.copy()), Vector(backend, y.copy()), Vector(backend, z.copy())
    s = 0.75
    before = backend.launch_count()
    run_vectors(backend, device=device, ir=sarek_ir.generic_example_ir(), args=[vu, vv, vx, vy, vz, ("float32", s), ("int32", n)],
                block=dims1d(256), grid=dims1d((n + 255) // 256))
    assert backend.launch_count() > before
    X, Y, Z = x.astype(np.float64), y.astype(np.float64), z.astype(np.float64)
    u = (X / (Y + 2.5) - np.sqrt(np.abs(Z * s))).astype(np.float32)
    U = u.astype(np.float64)
    v = np.where(U > 0.0, U * X, -Y).astype(np.float32)
    assert np.array_equal(vu.to_array(), u)
    assert np.array_equal(vv.to_array(), v)
    for t in (vu, vv, vx, vy, vz):
        t.free()


def test_unfused_consumer_runs_through_the_generated_path(backend, device):
    n = 4096
    a, b = O.fill(n, 31, 1), O.fill(n, 31, 2)
    vd, va, vb = Vector.create(backend, n), Vector(backend, a.copy()), Vector(backend, b.copy())
    run_vectors(backend, device=device, ir=sarek_ir.square_add_consumer_ir(), args=[vd, va, vb], block=dims1d(256), grid=dims1d(n // 256))
    want = (a.astype(np.float64) * a.astype(np.float64) + b.astype(np.float64)).astype(np.float32)
    assert np.array_equal(vd.to_array(), want)
    for t in (vd, va, vb):
        t.free()


@pytest.mark.parametrize("n", [1, 255, 1000, 256 * 40, 100003])
def test_guarded_benchmark_kernels_fused_by_the_backend(backend, device, oracle, n):
    """stream_triad followed by a guarded consumer, the kernel form of the reference's benchmarks
    (benchmarks/bench_stream_triad.ml:22-31), run unfused (two launches) and fused by the backend's
    guarded fusion (one launch); both against Native's result of the two kernels in sequence."""
    from spoc_b200 import fusion as F
    b, c = _inputs(n, seed=11)
    grid = dims1d((n + 255) // 256)               # the launch covers more threads than elements: the guard matters
    va, vd = Vector.create(backend, n), Vector.create(backend, n)
    vb, vc = Vector(backend, b.copy()), Vector(backend, c.copy())
    run_vectors(backend, device=device, ir=sarek_ir.stream_triad_ir("triad"), args=[va, vb, vc, ("float32", 3.0), ("int32", n)],
                block=dims1d(256), grid=grid)
    run_vectors(backend, device=device, ir=sarek_ir.square_add_guarded_ir(), args=[vd, va, vb, ("int32", n)],
                block=dims1d(256), grid=grid)
    unfused = vd.to_array().copy()
    fused_ir = F.fuse_guarded(sarek_ir.stream_triad_ir("triad"), sarek_ir.square_add_guarded_ir(), "a")
    assert fused_ir is not None
    vf = Vector.create(backend, n)
    before = backend.launch_count()
    run_vectors(backend, device=device, ir=fused_ir, args=[vf, vb, ("int32", n), vc, ("float32", 3.0)],
                block=dims1d(256), grid=grid, kernel_name="square_add_fused")
    assert backend.launch_count() - before <= 3   # vector body + scalar head/tail, never two passes over the data
    fused = vf.to_array()
    ref = np.empty(n, np.float32)
    oracle.so_chain_triad_square(ref, None, b, c, 3.0, n)
    assert O.ulp_distance(unfused, ref).max() <= 1
    assert O.ulp_distance(fused, ref).max() <= 1
    for v in (va, vd, vb, vc, vf):
        v.free()


@pytest.mark.parametrize("n", [5, 1000, 70001])
def test_pipeline_of_three_guarded_kernels_fused_matches_the_unfused_sequence_bit_for_bit(backend, device, n):
    """a = b + s*c ; d = a*a + b ; e = d*0.5 + a... as three guarded kernels and as the one generated kernel the
    backend's guarded pipeline fusion builds: the eliminated stores are marked, so the fused kernel rounds where the
    unfused kernels stored, and both agree with Native's result of the sequence to the last bit."""
    from spoc_b200 import fusion as F
    S = sarek_ir
    bld = S.Builder()
    p = bld.params([("vec", "e", "f32"), ("vec", "d", "f32"), ("vec", "c", "f32"), ("scalar", "n", "i32")])
    body = bld.let("i", "i32", bld.intr("global_thread_id"), lambda: (
        "sif", bld.binop("lt", bld.evar("i"), bld.evar("n")),
        ("assign", ("elem", "e", bld.evar("i")),
         bld.binop("sub", bld.binop("div", bld.read("d", bld.evar("i")), bld.c_f32(3.0)), bld.read("c", bld.evar("i"))))))
    third = S.sx(("kernel", "third", p, ("body", body)))
    b, c = _inputs(n, seed=13)
    grid = dims1d((n + 255) // 256)
    va, vd, ve = (Vector.create(backend, n) for _ in range(3))
    vb, vc = Vector(backend, b.copy()), Vector(backend, c.copy())
    run_vectors(backend, device=device, ir=S.stream_triad_ir("triad"), args=[va, vb, vc, ("float32", 3.0), ("int32", n)],
                block=dims1d(256), grid=grid)
    run_vectors(backend, device=device, ir=S.square_add_guarded_ir(),
                args=[vd, va, vb, ("int32", n)], block=dims1d(256), grid=grid)
    run_vectors(backend, device=device, ir=third, args=[ve, vd, vc, ("int32", n)], block=dims1d(256), grid=grid, kernel_name="third")
    unfused = ve.to_array().copy()
    fused_ir, eliminated = F.fuse_pipeline_as([S.stream_triad_ir("triad"), S.square_add_guarded_ir(), third], F.GUARDED)
    assert eliminated == ["d", "a"] and fused_ir.count("stored_f32") == 3      # a twice (read twice), d once
    # parameters of the fused kernel: third's without d, then the new ones of the kernel in front of it
    names = [q.split()[1] for q in fused_ir.split("(params ")[1].split("(body")[0].split("(")[1:]]
    assert names == ["e", "c", "n", "b", "scalar"]
    vf = Vector.create(backend, n)
    before = backend.launch_count()
    run_vectors(backend, device=device, ir=fused_ir, args=[vf, vc, ("int32", n), vb, ("float32", 3.0)],
                block=dims1d(256), grid=grid, kernel_name="third_fused")
    assert backend.launch_count() - before <= 3
    fused = vf.to_array()
    # Native's result of the three kernels in sequence: double arithmetic, one rounding per store
    a64 = (b.astype(np.float64) + c.astype(np.float64) * 3.0).astype(np.float32).astype(np.float64)
    d64 = (a64 * a64 + b.astype(np.float64)).astype(np.float32).astype(np.float64)
    ref = (d64 / 3.0 - c.astype(np.float64)).astype(np.float32)
    assert np.array_equal(fused, ref)
    assert O.ulp_distance(unfused, ref).max() <= 1     # the unfused run goes through the fused-multiply-add operators
    for v in (va, vd, ve, vb, vc, vf):
        v.free()


def _random_expression(rng, bld, depth):
    """A random float32 expression over x, y, z and the scalar s, with the function that evaluates it in float64."""
    f32 = ("Float32",)
    if depth == 0 or rng.random() < 0.15:
        k = int(rng.integers(0, 3))
        if k == 0:
            name = "xyz"[int(rng.integers(0, 3))]
            return bld.read(name, bld.evar("i")), (lambda env, name=name: env[name])
        if k == 1:
            v = round(float(rng.uniform(-2, 2)), 3)
            return bld.c_f32(v), (lambda env, v=v: np.float64(v))
        return bld.evar("s"), (lambda env: env["s"])
    op = str(rng.choice(["add", "sub", "mul", "div", "neg", "if", "sqrtabs", "fabs"]))
    sub = lambda: _random_expression(rng, bld, depth - 1)
    if op in ("add", "sub", "mul"):
        (ea, fa), (eb, fb) = sub(), sub()
        fn = {"add": np.add, "sub": np.subtract, "mul": np.multiply}[op]
        return bld.binop(op, ea, eb), (lambda env: fn(fa(env), fb(env)))
    if op == "div":
        (ea, fa), (eb, fb) = sub(), sub()
        return (bld.binop("div", ea, bld.binop("add", ("intrinsic", f32, "abs_float", eb), bld.c_f32(1.5))),
                lambda env: fa(env) / (np.abs(fb(env)) + 1.5))
    if op == "neg":
        ea, fa = sub()
        return ("unop", "neg", ea), (lambda env: -fa(env))
    if op == "fabs":
        ea, fa = sub()
        return ("intrinsic", f32, "abs_float", ea), (lambda env: np.abs(fa(env)))
    if op == "sqrtabs":
        ea, fa = sub()
        return ("intrinsic", f32, "sqrt", ("intrinsic", f32, "abs_float", ea)), (lambda env: np.sqrt(np.abs(fa(env))))
    (ec, fc), (ea, fa), (eb, fb) = sub(), sub(), sub()
    return ("if", bld.binop("gt", ec, bld.c_f32(0.25)), ea, eb), (lambda env: np.where(fc(env) > 0.25, fa(env), fb(env)))


@pytest.mark.parametrize("seed", [1, 2])
def test_random_expressions_on_the_generated_path_are_bit_exact(backend, device, seed):
    """Twelve seeded random expression trees per seed (+ - * / neg abs sqrt if, constants, a scalar parameter), guarded,
    against the same tree evaluated in float64 and rounded once — the Native backend's rule."""
    rng = np.random.default_rng(seed)
    for case in range(12):
        n = int(rng.choice([1, 7, 255, 1000, 4099, 70001]))
        bld = sarek_ir.Builder()
        p = bld.params([("vec", "o", "f32"), ("vec", "x", "f32"), ("vec", "y", "f32"), ("vec", "z", "f32"),
                        ("scalar", "s", "f32"), ("scalar", "n", "i32")])
        made = {}

        def body():
            e, made["f"] = _random_expression(rng, bld, int(rng.integers(1, 5)))
            return ("sif", bld.binop("lt", bld.evar("i"), bld.evar("n")), ("assign", ("elem", "o", bld.evar("i")), e))

        ir = sarek_ir.sx(("kernel", "rnd", p, ("body", bld.let("i", "i32", bld.intr("global_thread_id"), body))))
        x, y, z = O.fill(n, 100 * seed + case, 1), O.fill(n, 100 * seed + case, 2), O.fill(n, 100 * seed + case, 3)
        sval = float(np.float32(rng.uniform(-3, 3)))
        vo, vx, vy, vz = Vector.create(backend, n), Vector(backend, x.copy()), Vector(backend, y.copy()), Vector(backend, z.copy())
        run_vectors(backend, device=device, ir=ir, args=[vo, vx, vy, vz, ("float32", sval), ("int32", n)], block=dims1d(256),
                    grid=dims1d((n + 255) // 256), kernel_name="rnd")
        env = {"x": x.astype(np.float64), "y": y.astype(np.float64), "z": z.astype(np.float64), "s": np.float64(sval)}
        ref = np.broadcast_to(np.asarray(made["f"](env), dtype=np.float64), (n,)).astype(np.float32)
        assert np.array_equal(vo.to_array(), ref), ir
        for v in (vo, vx, vy, vz):
            v.free()


@pytest.mark.parametrize("kind", ["dot", "sum"])
@pytest.mark.parametrize("n,block", [(1000, 256), (256 * 40, 256), (100003, 256), (5000, 64), (70000, 1024)])
def test_block_tree_reduction_is_bit_exact(backend, device, oracle, kind, n, block):
    """reduce_sum / dot_product: one output per block, summed in the reference's tree order in double."""
    import ctypes as C
    a, b = O.fill(n, 41, 1), O.fill(n, 41, 2)
    nblocks = (n + block - 1) // block
    va, vb, vo = Vector(backend, a.copy()), Vector(backend, b.copy()), Vector(backend, np.full(nblocks + 3, CANARY, np.float32))
    args = [va, vb, vo, ("int32", n)] if kind == "dot" else [va, vo, ("int32", n)]
    run_vectors(backend, device=device, ir=sarek_ir.block_reduce_ir(kind, block), args=args, block=dims1d(block), grid=dims1d(nblocks),
                shared_mem=block * 4)
    want = np.empty(nblocks, np.float32)
    oracle.so_block_tree_reduce(a, b.ctypes.data_as(C.c_void_p) if kind == "dot" else None, want, n, nblocks, block)
    got = vo.to_array()
    assert np.array_equal(got[:nblocks], want)
    assert np.all(got[nblocks:] == CANARY)
    for v in (va, vb, vo):
        v.free()


def test_block_reduction_with_wrong_block_size_is_rejected(backend, device):
    n = 1024
    va, vo = Vector.create(backend, n), Vector.create(backend, 8)
    with pytest.raises(BackendError) as e:
        run_vectors(backend, device=device, ir=sarek_ir.block_reduce_ir("sum", 256), args=[va, vo, ("int32", n)], block=dims1d(128),
                    grid=dims1d(8))
    assert e.value.code == L.ERR_ARGS
    va.free()
    vo.free()
