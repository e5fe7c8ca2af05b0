"""Builds and runs the C++ host-layer test program (tests/cpp/test_builder.cpp): the graph
recogniser on CPU, and one training step through `bullet::Trainer` on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    from bullet_b200 import _lib

    _lib.load()
    exe = str(tmp_path_factory.mktemp("cpp") / "test_builder")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    libdir = os.path.join(ROOT, "bullet_b200")
    subprocess.check_call([cxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "test_builder.cpp"), "-o", exe,
                           "-L", libdir, "-lbullet_b200", f"-Wl,-rpath,{libdir}"])
    return exe


def test_recogniser_accepts_the_examples_and_refuses_the_rest(program):
    out = subprocess.run([program], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr


@pytest.mark.gpu
def test_cpp_trainer_runs_a_step(program):
    out = subprocess.run([program, "gpu"], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr
    losses = [ln for ln in out.stdout.splitlines() if ln.startswith("loss")][0].split()
    assert 0 < float(losses[2]) < float(losses[1]) < 1
