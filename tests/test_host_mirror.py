"""Builds and runs the C++ host-mirror test (tests/cpp/host_mirror_test.cpp): the reference's
dispatcher interface in C++ on top of the C ABI."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp, name="host_mirror_test"):
    exe = os.path.join(tmp, name)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", os.path.join(ROOT, "tests", "cpp", name + ".cpp"),
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
    assert "FAIL" not in r.stdout and r.stdout.count("PASS") >= 9


def test_ggml_bridge_recognises_the_expert_chain(tmp_path, zlib, oracle):
    """the bridge header against a stand-in for ggml's declarations: graph-chain recognition (no device)"""
    exe = _build(str(tmp_path), "ggml_bridge_test")
    r = subprocess.run([exe, "--match"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and r.stdout.count("PASS") >= 20


@pytest.mark.gpu
def test_ggml_bridge_runs_the_fused_chain(tmp_path, zlib, oracle, dev):
    exe = _build(str(tmp_path), "ggml_bridge_test")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and r.stdout.count("PASS") >= 28
