"""The header-only C++ host layer (include/b200const.hpp): tests/cpp/mirror_check.cpp is compiled with
g++ against the in-tree library; its host-only part (insertion order, type inference, error mapping)
runs everywhere, the folding part on the GPU box."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "npu_plugin_b200", "csrc")
BUILD = os.path.join(ROOT, "tests", "cpp", "_build")
EXE = os.path.join(BUILD, "mirror_check")


@pytest.fixture(scope="module")
def mirror_exe():
    if not os.path.exists(os.path.join(LIBDIR, "libb200const.so")):
        pytest.fail("libb200const.so is missing: run __graft_entry__.build() first")
    os.makedirs(BUILD, exist_ok=True)
    src = os.path.join(ROOT, "tests", "cpp", "mirror_check.cpp")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), src, "-o", EXE,
                           "-L" + LIBDIR, "-lb200const", "-Wl,-rpath," + LIBDIR])
    return EXE


def test_cpp_layer_host_part(mirror_exe):
    env = dict(os.environ, B200C_MIRROR_HOST_ONLY="1")
    r = subprocess.run([mirror_exe], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_layer_folds_on_the_device(mirror_exe):
    r = subprocess.run([mirror_exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
