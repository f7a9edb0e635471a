"""The plan of SB200_MODE_3XMIXED (spoc_b200/csrc/gemm_tcgen05.cuh, mix_plan), checked on the CPU through
sb200_mixed_plan: from the largest magnitudes of A and B it fixes the power-of-two scales of the fp16 panels and how the
accumulated cross terms get back to true units (rescale stages of 2^-15 each plus the first main-term MMA's scale)."""
import ctypes as C
import math

import numpy as np
import pytest

from spoc_b200 import _lib as L


def plan(max_a, max_b):
    out = (C.c_int32 * 5)()
    assert L.load().sb200_mixed_plan(C.c_float(max_a), C.c_float(max_b), out) == 0
    return dict(ok=out[0], stages=out[1], first=out[2], shift_a=out[3], shift_b=out[4])


def exponent(x):
    return math.frexp(float(np.float32(x)))[1] - 1      # x in [2^e, 2^(e+1))


@pytest.mark.parametrize("ea", range(-40, 30, 7))
@pytest.mark.parametrize("eb", range(-40, 30, 7))
def test_scales_and_rescaling_are_consistent(ea, eb):
    max_a, max_b = 1.37 * 2.0 ** ea, 1.91 * 2.0 ** eb
    p = plan(max_a, max_b)
    total = 39 - ea - eb                                 # rescaling when both panels peak below 2^15
    if total < 0 or min(total, 75) - 9 + ea + eb < 8:
        assert p["ok"] == 0
        return
    assert p["ok"] == 1
    # cross products come out in units of 2^-(shift_a + shift_b + 11); the kernel scales by 2^-(15*stages + first)
    assert p["shift_a"] + p["shift_b"] + 11 == 15 * p["stages"] + p["first"]
    assert 0 <= p["first"] <= 15 and 0 <= p["stages"] <= 4
    if p["stages"] > 0:
        assert p["first"] >= 1                           # no stage that could have been saved
    # the panels of both matrices fit fp16: largest scaled magnitude below 2^15 (high parts; low parts one bit lower)
    assert max_a * 2.0 ** p["shift_a"] < 2.0 ** 15 and max_b * 2.0 ** p["shift_b"] < 2.0 ** 15
    # and use its range: together the two peaks lie within a factor of four of 2^30 unless the rescaling was capped
    if total <= 75:
        assert exponent(max_a * 2.0 ** p["shift_a"]) + exponent(max_b * 2.0 ** p["shift_b"]) == 28


def test_ordinary_magnitudes():
    p = plan(0.99, 0.99)                                  # uniform [-1, 1): exponents -1, -1
    assert p == dict(ok=1, stages=2, first=11, shift_a=15, shift_b=15)
    p = plan(4.7, 0.06)                                   # N(0,1) against N(0, 1/64)
    assert p["ok"] == 1 and p["shift_a"] == 12 and p["shift_b"] == 19


@pytest.mark.parametrize("a,b", [(float("inf"), 1.0), (1.0, float("nan")), (2.0 ** 25, 2.0 ** 20), (2.0 ** -35, 2.0 ** -35)])
def test_declined_operands(a, b):
    assert plan(a, b)["ok"] == 0


def test_zero_matrices_are_taken():
    assert plan(0.0, 3.0)["ok"] == 1 and plan(3.0, 0.0)["ok"] == 1


def test_sign_is_ignored():
    assert plan(-0.99, 0.5) == plan(0.99, 0.5)
