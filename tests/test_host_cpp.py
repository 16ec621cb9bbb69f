"""The C++ host mirror of the operator interface: it must compile everywhere (CPU check) and,
on a GPU, drive the fused op through the C ABI and match the oracle."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "_build", "host_mirror_test")


def build_binary():
    from deers_b200 import _lib
    from oracle import ref
    ref.build()
    _lib.lib()
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    ora_dir = os.path.join(ROOT, "oracle", "_build")
    cmd = ["g++", "-std=c++17", "-O2", os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"), "-o", BIN,
           f"-L{lib_dir}", "-ldeers_b200", f"-L{ora_dir}", "-lattn_ref",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{ora_dir}"]
    subprocess.run(cmd, check=True)
    return BIN


def test_host_mirror_compiles_and_links():
    assert os.path.exists(build_binary())


@pytest.mark.gpu
def test_host_mirror_matches_oracle_on_gpu():
    out = subprocess.run([build_binary()], capture_output=True, text=True, timeout=300)
    print(out.stdout, out.stderr)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count("PASS") == 9 and "FAIL" not in out.stdout
