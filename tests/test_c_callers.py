"""The drop-in boundary seen from C: programs written against the reference's public header build
against include/aspen.h + libaspen_b200.so without a source change, and give the same results as the
Python binding.

CPU part: compile and link only (no compute): the reference's own callers where its tree is mounted
(main.c and the example programs, reference main.c:4, examples/*/aspen_*.c), and a caller of the same
style that is part of this repository.  GPU part: that caller runs a small network end to end.
"""
import glob
import os
import subprocess

import numpy as np
import pytest

import harness
from aspen_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFDIR = os.environ.get("ASPEN_REFERENCE", "/root/reference")
LIBDIR = os.path.join(ROOT, "aspen_b200")
OWN_CALLER = os.path.join(ROOT, "tests", "c_caller", "drop_in_caller.c")


def build_c(src: str, exe: str) -> subprocess.CompletedProcess:
    api.lib()    # makes sure the shared library exists
    return subprocess.run(["gcc", "-Wall", "-I", os.path.join(ROOT, "include"), src, "-o", exe, "-L", LIBDIR, "-laspen_b200", "-lm",
                           "-lpthread", f"-Wl,-rpath,{LIBDIR}"], capture_output=True, text=True)


def test_own_c_caller_compiles_and_links(workdir):
    r = build_c(OWN_CALLER, os.path.join(workdir, "drop_in_caller"))
    assert r.returncode == 0, r.stderr
    assert "error" not in r.stderr


REF_CALLERS = sorted(glob.glob(os.path.join(REFDIR, "main.c")) + glob.glob(os.path.join(REFDIR, "examples", "*", "aspen_*.c")))


@pytest.mark.skipif(not REF_CALLERS, reason="reference sources are not mounted")
@pytest.mark.parametrize("src", REF_CALLERS, ids=[os.path.relpath(p, REFDIR).replace(" ", "_") for p in REF_CALLERS])
def test_reference_c_callers_compile_and_link_unchanged(src, workdir):
    r = build_c(src, os.path.join(workdir, "ref_caller"))
    assert r.returncode == 0, r.stderr


@pytest.mark.gpu
def test_c_caller_runs_and_matches_the_python_binding(workdir):
    exe = os.path.join(workdir, "drop_in_caller_gpu")
    assert build_c(OWN_CALLER, exe).returncode == 0
    cfg, wf = harness.prepare("tiny_cnn", workdir)
    nchw = harness.make_input("tiny_cnn", (3, 3, 20, 20))
    inp = os.path.join(workdir, "c_in.tensor")
    nchw.tofile(inp)
    out = os.path.join(workdir, "c_out.bin")
    env = dict(os.environ, ASPEN_B200_PRECISION="1")
    r = subprocess.run([exe, cfg, wf, inp, "3", "2", os.path.join(workdir, "c.nasm"), out], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(out, np.float32)
    dev = harness.Device(cfg, wf, 3, 0, 8, precision=1, profile=0)
    assert dev.run(np.ascontiguousarray(nchw.transpose(0, 2, 3, 1)).reshape(-1, 3)) == 0
    want = dev.nasm.result([api.BATCH, api.OUT_C, api.OUT_H, api.OUT_W])
    dev.close()
    np.testing.assert_array_equal(got, want)
