"""How the library routes a product (kernel, tile, scratch, launches) — host logic, no GPU needed."""
import ctypes as C

import pytest

from spoc_b200 import _lib as L

SMS = 148


def describe(mode, M, N, K, addressable=1, sms=SMS):
    out = C.create_string_buffer(256)
    assert L.load().sb200_gemm_describe(mode, M, N, K, addressable, sms, out, 256) == 0
    return dict(kv.split("=") for kv in out.value.decode().split()[2:]) | {"kernel": " ".join(out.value.decode().split()[:2])}


@pytest.mark.parametrize("mode", [L.MODE_3XTF32, L.MODE_TF32])
def test_benchmark_configurations_take_the_large_tile(mode):
    for shape in [(8192, 8192, 8192), (32768 // 8, 32768, 32768), (65536 // 8, 4096, 4096), (4096, 4096, 4096), (2048, 2048, 2048)]:
        d = describe(mode, *shape)
        assert d["kernel"] == "pair direct" and d["tile"] == "256x256", (shape, d)
        assert d["launches"] == ("2" if mode == L.MODE_3XTF32 else "1")
    d = describe(L.MODE_TF32, 8192, 8192, 8192)
    assert d["stages"] == "6" and d["tiles"] == "1024" and d["waves"] == "14" and d["workspace"] == "0"
    d = describe(L.MODE_3XTF32, 8192, 8192, 8192)
    assert d["stages"] == "3" and d["workspace"] == str(2 * 8192 * 8192 * 4)     # the two low-part panels


def test_problems_with_few_tiles_take_narrower_tiles():
    assert describe(L.MODE_TF32, 1024, 1024, 1024)["tile"] == "256x64"
    assert describe(L.MODE_TF32, 256, 256, 256)["tile"] == "256x64"
    assert describe(L.MODE_3XTF32, 1536, 1536, 1536)["tile"] == "256x128"
    assert describe(L.MODE_TF32, 1792, 1792, 1792)["tile"] == "256x256"
    d = describe(L.MODE_TF32, 1024, 1024, 1024)
    assert d["stages"] == "8" and d["tiles"] == "64" and d["waves"] == "1"


def test_operands_tma_cannot_address_go_through_panels():
    d = describe(L.MODE_3XTF32, 700, 900, 1000, addressable=0)
    assert d["kernel"] == "pair panels" and d["launches"] == "3"
    kp = 1024
    assert int(d["workspace"]) == 2 * ((700 * kp * 4 + 1023) // 1024 * 1024 + (900 * kp * 4 + 1023) // 1024 * 1024)
    # at most 128 rows: the single-CTA kernel from panels, or the pair kernel when it can read the operands directly
    assert describe(L.MODE_TF32, 100, 300, 500, addressable=0)["kernel"] == "single panels"
    assert describe(L.MODE_TF32, 100, 300, 500, addressable=1)["kernel"] == "pair direct"


def test_degenerate_and_bad_arguments():
    out = C.create_string_buffer(64)
    lib = L.load()
    assert lib.sb200_gemm_describe(L.MODE_TF32, 0, 5, 5, 1, SMS, out, 64) == 0 and out.value == b"nothing to do"
    assert lib.sb200_gemm_describe(L.MODE_TF32, 5, 5, 0, 1, SMS, out, 64) == 0 and b"gemm_k0_kernel" in out.value
    assert lib.sb200_gemm_describe(7, 5, 5, 5, 1, SMS, out, 64) == L.ERR_INVALID_VALUE
    assert lib.sb200_gemm_describe(L.MODE_TF32, 5, 5, 5, 1, 0, out, 64) == L.ERR_INVALID_VALUE
    assert lib.sb200_set_gemm_tile_n(96) == L.ERR_INVALID_VALUE
    assert lib.sb200_set_gemm_tile_n(128) == 0
    assert describe(L.MODE_TF32, 8192, 8192, 8192)["tile"] == "256x128"
    assert lib.sb200_set_gemm_tile_n(0) == 0
