"""Builds and runs the C++ tests of the mirrored BatchLAS API (include/batchlas_b200.hh).
On CPU only the build and overload resolution are checked; the GPU run executes every group."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
EXE = os.path.join(ROOT, "tests", "cpp", "gemm_api_tests.bin")


def build_exe(lib):
    src = os.path.join(ROOT, "tests", "cpp", "gemm_api_tests.cc")
    hdr = os.path.join(ROOT, "include", "batchlas_b200.hh")
    libdir = os.path.join(ROOT, "batchlas_b200")
    if (not os.path.exists(EXE)) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        gxx = shutil.which("g++") or "/opt/gcc/bin/g++"
        subprocess.check_call([gxx, "-std=c++20", "-O1", "-I", os.path.join(ROOT, "include"), "-I",
                               os.path.join(CUDA, "include"), src, "-o", EXE, "-L", libdir, "-lbatchlas_b200",
                               "-L", os.path.join(CUDA, "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}",
                               f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"])
    return EXE


def test_cpp_api_compiles_and_overloads_resolve(lib):
    exe = build_exe(lib)
    out = subprocess.run([exe, "--compile-only-check"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0 and "overload set resolves" in out.stdout


@pytest.mark.gpu
def test_cpp_api_on_gpu(lib):
    exe = build_exe(lib)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    assert " 0 failed" in out.stdout
