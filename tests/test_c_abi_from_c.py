"""The header is C: a C11 program that includes include/lfm25_b200.h is compiled with gcc (warnings are errors),
linked against the library and run.  It calls host-side entry points only, so no GPU is needed."""
import os
import shutil
import subprocess

import pytest

from lfm25_inference_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_compiles_as_c_and_host_entry_points_work(tmp_path):
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    library = _abi.LIBRARY_PATH
    assert os.path.exists(library), "build the library first (__graft_entry__.build())"
    binary = tmp_path / "host_abi"
    compile_command = ["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic",
                       "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "c", "host_abi.c"),
                       "-o", str(binary), library, f"-Wl,-rpath,{os.path.dirname(library)}"]
    compiled = subprocess.run(compile_command, capture_output=True, text=True)
    assert compiled.returncode == 0, compiled.stderr
    ran = subprocess.run([str(binary)], capture_output=True, text=True, timeout=120)
    assert ran.returncode == 0 and ran.stdout.strip() == "ok", ran.stdout + ran.stderr
