"""Builds and runs tests/cpp/test_host_mirror.cc: the reference's own test style (load_library /
function / set_buffer / dispatch / commit().wait()) against the C++ host layer include/vpq_host.hpp."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_host_mirror.cc")
OUT = os.path.join(ROOT, "tests", "cpp", "build", "test_host_mirror")


def _build(vpq):
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    libdir = os.path.dirname(vpq.lib_path())
    cmd = [shutil.which("g++") or "g++", "-std=c++17", "-O1", SRC, "-o", OUT, f"-I{ROOT}/include",
           f"-I{cuda}/include", f"-L{libdir}", "-lvpq", f"-L{cuda}/lib64", "-lcudart",
           f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda}/lib64"]
    subprocess.run(cmd, check=True)


def test_host_mirror_compiles(vpq):
    """CPU: the header and the test program compile and link against libvpq.so."""
    _build(vpq)
    assert os.path.exists(OUT)


@pytest.mark.gpu
def test_host_mirror_reference_style_tests(vpq):
    if not os.path.exists(OUT):
        _build(vpq)
    r = subprocess.run([OUT], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "ALL PASSED" in r.stdout
