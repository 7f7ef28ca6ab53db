"""The C ABI driven from plain C (tests/c_abi_driver.c): the header compiles as C and the library runs the reference
server's call sequence (server/src/ffi.rs over src/capi.h) without Python or C++ in between."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(ROOT, "flint_mac_b200", "libflint_attn.so")


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("c_abi") / "c_abi_driver")
    src = os.path.join(HERE, "c_abi_driver.c")
    r = subprocess.run(["gcc", "-std=gnu11", "-Wall", "-Wextra", "-Werror", "-O1", "-o", exe, src, "-ldl", "-lm"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_valid_c_and_symbols_resolve(driver):
    import flint_mac_b200 as fa

    fa.load_library()  # built (there is no fallback)
    r = subprocess.run([driver, LIB, "symbols"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "symbols ok" in r.stdout


@pytest.mark.gpu
def test_reference_call_sequence_from_c(driver):
    r = subprocess.run([driver, LIB, "run"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "run ok" in r.stdout
