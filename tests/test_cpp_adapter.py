"""The header-only C++ adapter (include/aila_nf4_linear.hpp) compiles with a plain C++17
compiler, links against the C-ABI library and keeps the reference's error behaviour."""
import os
import shutil
import subprocess

import pytest

from aila_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_adapter_compiles_links_and_reports_errors(tmp_path):
    gxx = shutil.which("g++", path="/usr/bin:/bin") or shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    if not os.path.exists(_lib.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    exe = tmp_path / "adapter_example"
    libdir = os.path.dirname(_lib.LIB_PATH)
    cmd = [gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "adapter_example.cpp"), "-o", str(exe),
           "-L", libdir, "-laila_nf4", f"-Wl,-rpath,{libdir}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "init failed as expected" in r.stdout or "adapter ok on a GPU" in r.stdout
