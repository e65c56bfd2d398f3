"""The C++ host mirror (welvet_b200/host/welvet.hpp) through its own test program
(tests/cpp/host_mirror_test.cpp): compiled here with g++ against libwelvet_cuda.so and the
oracle library, run once without a device (names, wire codec, argument and no-device errors)
and once on cuda:0 (Pack / Unpack / MatVec / dense.Forward parity with the oracle)."""
import os
import subprocess

import pytest

import oracle
from welvet_b200 import build as wvbuild

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")
OUT = os.path.join(ROOT, "tests", "cpp", "_build", "host_mirror_test")


def _binary() -> str:
    lib = wvbuild.build()
    osolib = oracle.build()
    deps = [SRC, os.path.join(ROOT, "welvet_b200", "host", "welvet.hpp"), os.path.join(ROOT, "include", "welvet_cuda.h"), lib, osolib]
    if not os.path.exists(OUT) or os.path.getmtime(OUT) < max(os.path.getmtime(d) for d in deps):
        os.makedirs(os.path.dirname(OUT), exist_ok=True)
        cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "welvet_b200", "host"),
               SRC, "-o", OUT, "-L", os.path.dirname(lib), "-lwelvet_cuda", "-L", os.path.dirname(osolib), "-lwelvet_oracle",
               f"-Wl,-rpath,{os.path.dirname(lib)}", f"-Wl,-rpath,{os.path.dirname(osolib)}"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
    return OUT


def _run(mode: str) -> None:
    res = subprocess.run([_binary(), mode], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert f"{mode}: 0 failure(s)" in res.stdout


def test_cpp_host_mirror_without_device():
    _run("host")


@pytest.mark.gpu
def test_cpp_host_mirror_on_device():
    _run("gpu")
