"""Builds and runs the C++ caller of the C ABI (tests/cxx/tile_check.cpp): the reference's own
GPU-vs-matrixMulCPU check (TileProgramming/kernel.cu:117-159) with this library in place of its
tiled kernel."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tile_check(cb, oracle, tmp_path_factory):
    exe = tmp_path_factory.mktemp("cxx") / "tile_check"
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O2", os.path.join(ROOT, "tests", "cxx", "tile_check.cpp"), "-o", str(exe),
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           "-L", os.path.join(ROOT, "cudaintro_b200"), "-lb200gemm", "-L", os.path.join(ROOT, "oracle"), "-loracle",
           "-L", os.path.join(cuda, "lib64"), "-lcudart",
           f"-Wl,-rpath,{os.path.join(ROOT, 'cudaintro_b200')}", f"-Wl,-rpath,{os.path.join(ROOT, 'oracle')}",
           f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"]
    subprocess.run(cmd, check=True)
    return str(exe)


@pytest.mark.parametrize("width,mode", [(1024, 0), (1024, 1), (1024, 2), (250, 0)])
def test_reference_style_check_passes(tile_check, device, width, mode):
    res = subprocess.run([tile_check, str(width), str(mode)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "Matrix multiplication successful!" in res.stdout


@pytest.fixture(scope="module")
def wrappers_check(cb, oracle, tmp_path_factory):
    """tests/cxx/tensor_wrappers_check.cpp: the reference's thrustensor / thrustTensorBfloat16 /
    thrustcudacore demos (TileProgramming/matmulTensor.cu:140-228) on the shims of
    include/tile_programming.h."""
    exe = tmp_path_factory.mktemp("cxx") / "tensor_wrappers_check"
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O2", os.path.join(ROOT, "tests", "cxx", "tensor_wrappers_check.cpp"), "-o", str(exe),
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           "-L", os.path.join(ROOT, "cudaintro_b200"), "-lb200gemm", "-L", os.path.join(ROOT, "oracle"), "-loracle",
           "-L", os.path.join(cuda, "lib64"), "-lcudart",
           f"-Wl,-rpath,{os.path.join(ROOT, 'cudaintro_b200')}", f"-Wl,-rpath,{os.path.join(ROOT, 'oracle')}",
           f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"]
    subprocess.run(cmd, check=True)
    return str(exe)


@pytest.mark.parametrize("kind,width", [("half", 1024), ("bf16", 1024), ("f32", 1024), ("half", 264)])
def test_reference_launch_wrappers_on_this_library(wrappers_check, device, kind, width):
    res = subprocess.run([wrappers_check, kind, str(width)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "Matrix multiplication successful!" in res.stdout
