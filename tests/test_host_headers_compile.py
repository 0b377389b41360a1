"""The header-only C++ host classes build from plain C++ (no pybind11) against the C ABI library, as the integration notes show."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    cxx = shutil.which("g++")
    lib_dir = os.path.join(ROOT, "binarybrain_b200", "lib")
    if cxx is None or not os.path.exists(os.path.join(lib_dir, "libbbcu_b200.so")):
        pytest.skip("no g++ or no built library")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    out = tmp_path / "host_example"
    cmd = [cxx, "-std=c++17", "-O1", os.path.join(ROOT, "tests", "host_example.cpp"), "-o", str(out),
           "-I" + os.path.join(ROOT, "binarybrain_b200", "host"), "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include"),
           "-L" + lib_dir, "-lbbcu_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + lib_dir]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert out.exists()
    return out


def test_host_example_compiles_and_links(tmp_path):
    _build(tmp_path)


@pytest.mark.gpu
def test_host_example_runs(tmp_path):
    """Three DifferentiableLut6 layers, forward + backward + Adam, from a plain C++ program."""
    out = _build(tmp_path)
    r = subprocess.run([str(out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
