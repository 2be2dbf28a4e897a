"""Runs the C++ host-mirror test (tests/cpp/test_compat.cpp): the brotensor /
brodiffusion entry points of include/brotensor and include/brodiffusion over
the C ABI, against the oracle, in the style of the reference's own tests."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "test_compat")


@pytest.mark.gpu
def test_cpp_host_mirror(bd, oracle):
    src = os.path.join(ROOT, "tests", "cpp", "test_compat.cpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < os.path.getmtime(src):
        subprocess.check_call(["sh", os.path.join(ROOT, "tests", "cpp", "build.sh")])
    res = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    print(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "test_compat: ok" in res.stdout


def test_cpp_headers_compile_without_a_gpu():
    """The mirror headers are self-contained C++17 (host compile only)."""
    code = ('#include "brodiffusion/dit/common.h"\n#include "brodiffusion/fused_transformer.h"\n'
            "int main() { return 0; }\n")
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "t.cpp")
        open(p, "w").write(code)
        subprocess.check_call(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"),
                               "-I", "/usr/local/cuda/include", p])
