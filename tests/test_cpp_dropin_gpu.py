"""Compiles and runs the C++ drop-in test: the reference's generator templates
(same names, same functor signatures) over the C ABI, with host vectors and
with device pointers, compared element for element with the oracle."""
import os
import subprocess

import pytest

from fbgemm_b200 import build
from oracle import checker

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def compile_dropin(out_dir):
    build.build()
    checker.build(("oracle",))
    exe = os.path.join(out_dir, "dropin_test")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "dropin_test.cc"), "-o", exe,
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           "-L", os.path.join(ROOT, "fbgemm_b200"), "-lfbgemm_b200", "-L", os.path.join(ROOT, "oracle"), "-loracle",
           "-L", os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "fbgemm_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle"),
           "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    subprocess.run(cmd, check=True)
    return exe


def test_cpp_caller_compiles_against_the_generator_header(tmp_path):
    """CPU part: a caller written against fbgemm's names builds and links."""
    assert os.path.exists(compile_dropin(str(tmp_path)))


@pytest.mark.gpu
def test_cpp_dropin_matches_oracle(tmp_path):
    exe = compile_dropin(str(tmp_path))
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "DROPIN_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
