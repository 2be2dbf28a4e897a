"""The C-ABI shared library loads and exports every entry point that
include/bdattn.h declares; without a GPU every operator fails loudly (there is
no CPU path)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "bdattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bdattn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for required in ("bdattn_sdpa_fwd", "bdattn_rmsnorm_rope", "bdattn_linear_attn_relu_fwd",
                     "bdattn_last_error", "bdattn_device_status", "bdattn_version"):
        assert required in names


def test_library_exports_every_declared_symbol():
    import brodiffusion_b200 as bd
    lib = bd.lib()
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in bdattn.h but not exported: {missing}"
    assert lib.bdattn_version() >= 100


def test_struct_mirrors_match_the_header_layout():
    import brodiffusion_b200 as bd
    # bdattn_sdpa_params: 4 ints + int + 2*8 ... the C compiler's layout is
    # reproduced by ctypes; the sizes below are sizeof() from the header.
    import subprocess, tempfile, textwrap
    src = textwrap.dedent("""
        #include <stdio.h>
        #include "bdattn.h"
        int main(void) { printf("%zu %zu\\n", sizeof(bdattn_sdpa_params), sizeof(bdattn_norm_rope_job)); return 0; }
    """)
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        a, b = map(int, subprocess.check_output([exe]).split())
    assert C.sizeof(bd.SdpaParams) == a
    assert C.sizeof(bd.NormRopeJob) == b


def test_no_cpu_path_without_a_gpu():
    import torch
    import brodiffusion_b200 as bd
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = bd.SdpaParams()
    rc = bd.lib().bdattn_sdpa_fwd(C.byref(p), None)
    assert rc == -1
    assert "CUDA" in bd.last_error() or "sm_100" in bd.last_error()
    with pytest.raises(bd.BdattnError):
        bd.device_status()


def test_missing_library_is_reported(monkeypatch, tmp_path):
    import brodiffusion_b200 as bd
    monkeypatch.setattr(bd, "_lib", None)
    monkeypatch.setattr(bd._build, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(bd.BdattnError, match="missing"):
        bd.lib()
