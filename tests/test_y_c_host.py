"""The C ABI used from plain C: `tests/c_host/hb_c_host.c` includes only the public header,
is built as C99 and drives matmul (fp32 256^3 through the host-buffer call), causal
attention and the error path without Python or C++ in between."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c_host", "hb_c_host.c")
LIBDIR = os.path.join(ROOT, "habu_b200")
GCC = shutil.which("gcc") or "/usr/bin/gcc"


def build_host(out_dir):
    exe = os.path.join(str(out_dir), "hb_c_host")
    cmd = [GCC, "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", "-I", os.path.join(ROOT, "include"),
           SRC, "-o", exe, "-L", LIBDIR, "-lhabu_b200", "-lm", "-Wl,-rpath," + LIBDIR]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_public_header_is_valid_c99_and_the_host_links(tmp_path):
    # no compute here: compiling proves the header has no C++-isms, linking proves every
    # entry point the program names is exported
    assert os.path.exists(os.path.join(LIBDIR, "libhabu_b200.so")), "run `python -m habu_b200.build` first"
    exe = build_host(tmp_path)
    assert os.access(exe, os.X_OK)


@pytest.mark.gpu
def test_plain_c_host_runs_matmul_attention_and_error_path(tmp_path):
    exe = build_host(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("OK")
    assert "status 1" in r.stdout      # the mismatched matmul came back as HB_ERR_INVALID
