"""The reference's own unit tests for this path, re-expressed in C++ against the
drop-in `namespace lh` front end (include/lh_dropin) with all-host buffers."""
import os
import subprocess

import pytest

from longhornai_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_dropin.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "_build", "test_dropin")


def compile_test():
    _cabi.load()
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    libdir = os.path.dirname(_cabi.LIB_PATH)
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include", "lh_dropin"),
                           SRC, "-o", EXE, "-L" + libdir, "-llhb200", "-Wl,-rpath," + libdir])


def test_dropin_headers_compile_and_link():
    compile_test()


@pytest.mark.gpu
def test_reference_unit_tests_pass_on_the_gpu_dropin():
    compile_test()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failures" in r.stdout
