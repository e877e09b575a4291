"""The C17 surface compiled, not just bound: tests/c17_lifecycle.c includes <dl/decoder_c_api.h> (the reference's include
path, served by include/dl/), is compiled with `cc -std=c17 -pedantic -Werror`, linked with `-lctorch` (the reference
package's library name, a link beside libctorch_b200.so) and run - on the host here, on cuda:0 under the gpu marker.  The
program restates the decoder part of the reference's C ABI test (tests/c_api.c:28-42 of the reference)."""
import os
import shutil
import subprocess

import pytest

import ctorch_b200 as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.path.join(ROOT, "tests", "c17_lifecycle.c")
LIBDIR = os.path.join(ROOT, "ctorch_b200")


def build(tmp_path):
    compiler = shutil.which("cc") or shutil.which("gcc")
    if compiler is None:
        pytest.skip("no C compiler")
    B.lib()   # the library (and the links with the reference's names) must exist
    if not os.path.islink(os.path.join(LIBDIR, "libctorch.so")):
        from ctorch_b200 import build as builder
        builder.build()
    binary = str(tmp_path / "c17_lifecycle")
    cmd = [compiler, "-std=c17", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), SOURCE,
           "-L", LIBDIR, "-lctorch", "-Wl,-rpath," + LIBDIR, "-lm", "-o", binary]
    result = subprocess.run(cmd, capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
    return binary


def test_c17_program_compiles_links_and_runs_on_the_host(tmp_path):
    binary = build(tmp_path)
    result = subprocess.run([binary, "cpu"], capture_output=True, text=True, timeout=120)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "c17 lifecycle ok" in result.stdout


@pytest.mark.gpu
def test_c17_program_decodes_on_the_gpu(tmp_path):
    binary = build(tmp_path)
    result = subprocess.run([binary, "cuda"], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "c17 lifecycle ok" in result.stdout
