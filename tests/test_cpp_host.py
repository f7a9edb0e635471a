"""Builds and runs the C++ host-side mirror of the plugin (spoc_b200/host/sarek_b200.hpp) through its
own C++ test program, tests/cpp/test_host_plugin.cc."""
import os
import subprocess

import pytest

from spoc_b200 import _lib as L
from spoc_b200 import sarek_ir as S
from spoc_b200.build import build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    build_library()
    work = tmp_path_factory.mktemp("cpp_host")
    exe = str(work / "test_host_plugin")
    libdir = os.path.dirname(L.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", os.path.join(ROOT, "tests", "cpp", "test_host_plugin.cc"), "-o", exe,
           f"-L{libdir}", "-lsarek_b200", f"-Wl,-rpath,{libdir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    irdir = work / "ir"
    irdir.mkdir()
    for name, text in {"vector_add": S.vector_add_ir(), "stream_triad": S.stream_triad_ir(), "matmul_naive": S.matmul_naive_ir(),
                       "matmul_tiled": S.matmul_tiled_ir(), "dot_product": S.block_reduce_ir("dot"),
                       "triad_producer": S.triad_producer_ir(), "square_add_consumer": S.square_add_consumer_ir(),
                       "square_add_guarded": S.square_add_guarded_ir()}.items():
        (irdir / f"{name}.ir").write_text(text)
    return exe, str(irdir)


def test_cpp_host_side_without_a_gpu(program):
    exe, irdir = program
    res = subprocess.run([exe, "cpu", irdir], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "ALL PASSED" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_host_side_on_the_gpu(program):
    exe, irdir = program
    res = subprocess.run([exe, "gpu", irdir], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "ALL PASSED" in res.stdout, res.stdout + res.stderr
