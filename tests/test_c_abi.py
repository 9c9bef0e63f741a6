"""The C ABI from plain C: tests/c_abi/abi_smoke.c is compiled with gcc (-std=c99 -pedantic -Werror) against include/hl_b200.h
and linked to the built library.  On the CPU it proves that the header is valid C and that every prototype a binding uses has
the documented argument types; on a GPU it commits a small matrix (64-bit rows and packed rows), opens it and compares."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    from intelligenceregulation_b200 import build

    build.build()
    exe = str(tmp_path / "abi_smoke")
    lib_dir = os.path.join(ROOT, "intelligenceregulation_b200")
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I" + os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "c_abi", "abi_smoke.c"), "-o", exe, "-L" + lib_dir, "-lhl_b200", "-Wl,-rpath," + lib_dir])
    return exe


def test_header_compiles_as_c_and_links(tmp_path):
    out = subprocess.run([_build(tmp_path)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "abi ok" in out.stdout, (out.returncode, out.stdout, out.stderr)


@pytest.mark.gpu
def test_a_commitment_from_plain_c(tmp_path):
    out = subprocess.run([_build(tmp_path), "gpu"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "two commitments" in out.stdout, (out.returncode, out.stdout, out.stderr)
