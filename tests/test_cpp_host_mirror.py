"""Builds the C++ host mirror test (tests/cpp/kvcache_host_test.cpp over include/EdgeRunnerCUDA.hpp) with g++ and runs
it: the no-device error path on CPU, the reference's KVCacheTests cases on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    from edgerunner_b200 import build
    lib = build.build()
    out = str(tmp_path_factory.mktemp("cpp") / "kvcache_host_test")
    env = dict(os.environ)
    env.pop("CXX", None)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "kvcache_host_test.cpp"), "-o", out,
           "-L", os.path.dirname(lib), "-ler_kv", "-Wl,-rpath," + os.path.dirname(lib)]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    return out


def test_cpp_mirror_without_device(binary):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    r = subprocess.run([binary, "--no-device"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_mirror_kvcache_cases(binary):
    r = subprocess.run([binary], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
