"""SB200_MODE_3XMIXED: the three-term split with the main term on the TF32 pipe and the two cross terms on the fp16 pipe.

What must hold: the bound of 3xTF32 mode (1e-5*sqrt(K) against the Native-semantics oracle); an error no worse than
3xTF32's own against a float64 product; exact equivariance under power-of-two scalings of A and B (the plan only moves
exponents, so the panels, the MMAs and the rescaling are the same numbers); and operands the mode cannot take — huge
magnitudes, infinities, NaNs — computed by the plain 3xTF32 kernels in the same call, bit for bit.
"""
import math

import numpy as np
import pytest

from spoc_b200 import _lib as L
from tests import oracle_lib as O
from tests.gpu_util import Dev, dev_from, gemm

pytestmark = pytest.mark.gpu

MIX, PLAIN = L.MODE_3XMIXED, L.MODE_3XTF32


@pytest.fixture(autouse=True)
def low_threshold():
    """The mode takes products from 2^34 multiply-adds by default; the tests lower that to 2^28 to keep their sizes small."""
    L.load().sb200_set_mixed_min_macs(1 << 28)
    yield
    L.load().sb200_set_mixed_min_macs(0)


def bound(K, scale=1.0):
    return max(1e-5 * math.sqrt(K), 1e-6) * scale


def run(backend, device, mode, M, N, K, a, b, **epi):
    A, B, D = dev_from(backend, device, a), dev_from(backend, device, b), Dev(backend, device, M * N)
    extra = []
    try:
        kw = {}
        if "c" in epi:
            Cm, Bi = dev_from(backend, device, epi["c"]), dev_from(backend, device, epi["bias"])
            extra = [Cm, Bi]
            kw = dict(alpha=1.5, C_=Cm, beta=0.5, bias=Bi, act=1)
        gemm(backend, device, mode, M, N, K, A, B, D, **kw)
        return D.download().reshape(M, N)
    finally:
        for x in [A, B, D] + extra:
            x.free()


# every shape has at least 2^28 multiply-adds (below the threshold the mode hands over to 3xTF32 on the host side)
# and rows TMA can address (K and N multiples of 4) except the last three, which take the 3xTF32 route
SHAPES = [(1024, 1024, 256), (1024, 1000, 300), (257, 4096, 260), (2048, 520, 264), (300, 1032, 1000), (4096, 64, 1024),
          (512, 516, 1028), (1500, 1500, 128), (2048, 2048, 2048), (300, 1031, 1000), (512, 512, 1025), (1500, 1500, 127)]


@pytest.mark.parametrize("shape", SHAPES)
def test_plain_product_matches_oracle_and_3xtf32(backend, device, shape):
    M, N, K = shape
    a, b = O.fill(M * K, 61, 1), O.fill(K * N, 61, 2)
    got = run(backend, device, MIX, M, N, K, a, b)
    rows = np.unique(np.linspace(0, M - 1, 24).astype(int))
    ref = np.vstack([O.gemm(a, b, M, N, K, r0=int(r), r1=int(r) + 1) for r in rows])
    assert O.gemm_rel_error(got[rows], ref) <= bound(K)
    # against an exact product the mixed mode errs no more than 3xTF32 does (same three terms, same roundings of the
    # operands; only the order of the fp32 accumulation differs)
    plain = run(backend, device, PLAIN, M, N, K, a, b)
    exact = a.reshape(M, K)[rows].astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    scale = np.abs(a.reshape(M, K)[rows]).astype(np.float64) @ np.abs(b.reshape(K, N)).astype(np.float64)
    err_mix = (np.abs(got[rows] - exact) / scale).max()
    err_plain = (np.abs(plain[rows] - exact) / scale).max()
    assert err_mix <= 1.5 * err_plain + 2e-8, (err_mix, err_plain)
    assert err_mix < 4e-6       # far inside TF32's 5e-5..5e-4: the cross terms are there


@pytest.mark.parametrize("shape", [(1024, 1024, 256), (700, 1100, 520)])
def test_fused_epilogue_matches_oracle(backend, device, shape):
    M, N, K = shape
    a, b, c = O.fill(M * K, 62, 1), O.fill(K * N, 62, 2), O.fill(M * N, 62, 3)
    bias = O.fill(N, 62, 4, kind=1)
    got = run(backend, device, MIX, M, N, K, a, b, c=c, bias=bias)
    rows = np.unique(np.linspace(0, M - 1, 16).astype(int))
    ref = np.vstack([O.gemm(a, b, M, N, K, 1.5, 0.5, c, bias, 1, r0=int(r), r1=int(r) + 1) for r in rows])
    assert O.gemm_rel_error(got[rows], ref) <= bound(K, 1.5 * math.sqrt(2))


@pytest.mark.parametrize("pa,pb", [(0, 0), (3, -2), (10, 8), (19, 19), (-8, -9), (-20, -15), (30, -30), (-40, 45), (-17, -17)])
def test_power_of_two_scalings_commute_with_the_product(backend, device, pa, pb):
    """(2^pa A)(2^pb B) = 2^(pa+pb) (A B) bit for bit: the total rescaling runs from 0 (product of the maxima near 2^39)
    through one to four rescale stages as the magnitudes shrink, and every plan must yield the same numbers."""
    M, N, K = 1024, 1024, 256
    a, b = O.fill(M * K, 63, 1), O.fill(K * N, 63, 2)
    base = run(backend, device, MIX, M, N, K, a, b)
    scaled = run(backend, device, MIX, M, N, K, np.ldexp(a, pa), np.ldexp(b, pb))
    assert np.array_equal(scaled.view(np.uint32), np.ldexp(base, pa + pb).view(np.uint32))


def test_small_magnitudes_shrink_the_panels_but_keep_the_bound(backend, device):
    """Product of the maxima below 2^-36: the plan caps the rescaling at 75 bits and lets the panels peak lower."""
    M, N, K = 1024, 1024, 256
    a, b = O.fill(M * K, 64, 1), O.fill(K * N, 64, 2)
    for pa, pb in ((-25, -25), (-28, -28)):
        a2, b2 = np.ldexp(a, pa), np.ldexp(b, pb)
        got = run(backend, device, MIX, M, N, K, a2, b2)
        exact = a2[:16 * K].reshape(16, K).astype(np.float64) @ b2.reshape(K, N).astype(np.float64)
        scale = np.abs(a2[:16 * K].reshape(16, K)).astype(np.float64) @ np.abs(b2.reshape(K, N)).astype(np.float64)
        assert (np.abs(got[:16] - exact) / scale).max() < 4e-6


@pytest.mark.parametrize("case", ["huge", "tiny", "inf", "nan"])
def test_operands_the_mode_declines_are_computed_by_3xtf32(backend, device, case):
    M, N, K = 1024, 1024, 256
    a, b = O.fill(M * K, 65, 1), O.fill(K * N, 65, 2)
    if case == "huge":
        a, b = np.ldexp(a, 25), np.ldexp(b, 20)          # maxima's product beyond 2^39
    elif case == "tiny":
        a, b = np.ldexp(a, -35), np.ldexp(b, -35)        # below 2^-58
    elif case == "inf":
        a = a.copy()
        a[5 * K + 7] = np.inf
    else:
        b = b.copy()
        b[3 * N + 11] = np.nan
    with np.errstate(invalid="ignore"):
        got, want = run(backend, device, MIX, M, N, K, a, b), run(backend, device, PLAIN, M, N, K, a, b)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_zero_matrices(backend, device):
    M, N, K = 1024, 1024, 256
    a, b = O.fill(M * K, 66, 1), O.fill(K * N, 66, 2)
    assert not run(backend, device, MIX, M, N, K, np.zeros_like(a), b).any()
    assert not run(backend, device, MIX, M, N, K, a, np.zeros_like(b)).any()


def test_wide_dynamic_range_degrades_no_further_than_tf32(backend, device):
    """Elements far below their matrix's largest lose their cross terms at worst: every product keeps TF32's accuracy,
    and those within 2^29 of the largest keep 3xTF32's."""
    M, N, K = 1024, 1024, 256
    rng = np.random.default_rng(7)
    a = (O.fill(M * K, 67, 1) * np.exp2(rng.integers(-45, 1, M * K))).astype(np.float32)
    b = (O.fill(K * N, 67, 2) * np.exp2(rng.integers(-45, 1, K * N))).astype(np.float32)
    got = run(backend, device, MIX, M, N, K, a, b)
    exact = a[:32 * K].reshape(32, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    scale = np.abs(a[:32 * K].reshape(32, K)).astype(np.float64) @ np.abs(b.reshape(K, N)).astype(np.float64)
    assert (np.abs(got[:32] - exact) / scale).max() < 2.0 ** -10
    # restricted to 2^-20..1 the result is fp32-grade again
    a = (O.fill(M * K, 67, 1) * np.exp2(rng.integers(-20, 1, M * K))).astype(np.float32)
    b = (O.fill(K * N, 67, 2) * np.exp2(rng.integers(-20, 1, K * N))).astype(np.float32)
    got = run(backend, device, MIX, M, N, K, a, b)
    exact = a[:32 * K].reshape(32, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    scale = np.abs(a[:32 * K].reshape(32, K)).astype(np.float64) @ np.abs(b.reshape(K, N)).astype(np.float64)
    assert (np.abs(got[:32] - exact) / scale).max() < 4e-6


def test_small_products_and_unaligned_operands_take_the_3xtf32_route(backend, device):
    for (M, N, K), offset in (((256, 256, 256), 0), ((1024, 1024, 256), 1)):
        a, b = O.fill(M * K, 68, 1), O.fill(K * N, 68, 2)
        outs = []
        for mode in (MIX, PLAIN):
            A, B, D = dev_from(backend, device, a, offset=offset), dev_from(backend, device, b), Dev(backend, device, M * N)
            try:
                gemm(backend, device, mode, M, N, K, A, B, D)
                outs.append(D.download())
            finally:
                for x in (A, B, D):
                    x.free()
        assert np.array_equal(outs[0], outs[1])
