"""The C++ host mirror (hipml_b200/host) and its `hipml parity`-style runner.

CPU: the runner builds against the C ABI and the oracle, and reports "no device" instead of
passing when there is no GPU (the reference's rule: a case that cannot run on the device is
skipped, never passed). GPU: every case of the table passes, including the 100,000-token
deep case.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "tests", "host", "_build")
EXE = os.path.join(BUILD, "hipml_parity")


def build_runner():
    import __graft_entry__ as entry
    entry.build()
    os.makedirs(BUILD, exist_ok=True)
    srcs = [os.path.join(ROOT, "tests", "host", "parity_main.cpp"),
            os.path.join(ROOT, "hipml_b200", "host", "hipml_host.cpp")]
    lib_dir = os.path.join(ROOT, "hipml_b200", "lib")
    ora_dir = os.path.join(ROOT, "oracle", "_build")
    if not os.path.exists(EXE) or any(os.path.getmtime(s) > os.path.getmtime(EXE) for s in srcs):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-Wall", *srcs, "-o", EXE,
                               f"-L{lib_dir}", "-lhipml_cuda", f"-L{ora_dir}", "-lhipml_oracle",
                               f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{ora_dir}"])
    return EXE


def test_runner_builds_and_never_passes_without_a_device():
    import torch
    exe = build_runner()
    if torch.cuda.is_available():
        pytest.skip("a device is present; the GPU test runs the table")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "SKIP no device" in r.stdout
    assert "PASS" not in r.stdout


@pytest.mark.gpu
def test_parity_table_passes_on_the_device():
    exe = build_runner()
    r = subprocess.run([exe, "--deep"], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and "31 cases, 0 failed" in r.stdout
