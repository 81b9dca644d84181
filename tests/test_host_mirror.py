"""Builds and runs the C++ host-mirror test (tests/cpp/host_mirror_test.cpp): the reference's
dispatcher interface in C++ on top of the C ABI."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp):
    exe = os.path.join(tmp, "host_mirror_test")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"),
           "-I/usr/local/cuda/include", "-L/usr/local/cuda/lib64", "-lcudart",
           os.path.join(ROOT, "zeromoe_b200", "libzmoe_b200.so"), os.path.join(ROOT, "oracle", "libzmoe_oracle.so"),
           "-Wl,-rpath," + os.path.join(ROOT, "zeromoe_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle"),
           "-Wl,-rpath,/usr/local/cuda/lib64", "-o", exe]
    subprocess.check_call(cmd)
    return exe


def test_host_mirror_compiles(tmp_path, zlib, oracle):
    _build(str(tmp_path))


@pytest.mark.gpu
def test_host_mirror_runs(tmp_path, zlib, oracle, dev):
    exe = _build(str(tmp_path))
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and r.stdout.count("PASS") >= 8
