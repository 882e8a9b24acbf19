"""The README-level C++ interface (include/tile-fusion.h) compiled against the shared library."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def api_test_binary(built_lib, tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cpp") / "api_test")
    libdir = os.path.dirname(built_lib)
    cmd = ["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "api_test.cpp"),
           "-L" + libdir, "-ltilefusion_b200", "-Wl,-rpath," + libdir, "-L/usr/local/cuda/lib64",
           "-Wl,-rpath,/usr/local/cuda/lib64", "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_cpp_inspector(api_test_binary):
    res = subprocess.run([api_test_binary, "inspect"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "OK inspect" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_executors(api_test_binary):
    res = subprocess.run([api_test_binary, "run"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "OK run" in res.stdout, res.stdout + res.stderr
