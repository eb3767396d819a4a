"""The C++ shim that implements the reference's Gemma4BatchModelRunner over the C ABI
(carat_b200/shim/batch_model_runner_shim.cpp) must compile against the reference's own headers.
The headers exist only where the reference tree is mounted; elsewhere the test is skipped."""
import os
import shutil
import subprocess

import pytest

from conftest import reference_root

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(reference_root() is None, reason="no checkout of the reference found")
@pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")
def test_shim_compiles_against_the_reference_headers():
    cuda_home = os.environ.get("CUDA_HOME", os.path.dirname(os.path.dirname(shutil.which("nvcc"))))
    command = ["g++", "-std=c++20", "-fsyntax-only", "-Wall", "-Wextra", "-Werror",
               "-I", os.path.join(reference_root(), "include"), "-I", os.path.join(ROOT, "include"),
               "-I", os.path.join(cuda_home, "include"),
               os.path.join(ROOT, "carat_b200", "shim", "batch_model_runner_shim.cpp")]
    done = subprocess.run(command, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]


def test_shim_uses_only_declared_entry_points():
    """Every carat_b200_* name the shim calls is declared in the public header."""
    import re
    header = open(os.path.join(ROOT, "include", "carat_b200.h")).read()
    shim = open(os.path.join(ROOT, "carat_b200", "shim", "batch_model_runner_shim.cpp")).read()
    declared = set(re.findall(r"\b(carat_b200_[a-z0-9_]+)\s*\(", header))
    structs = set(re.findall(r"\b(carat_b200_[a-z0-9_]+)\b", header))
    for name in set(re.findall(r"\b(carat_b200_[a-z0-9_]+)\s*\(", shim)):
        assert name in declared, name
    for name in set(re.findall(r"\b(carat_b200_[a-z0-9_]+)\b", shim)):
        assert name in structs, name
