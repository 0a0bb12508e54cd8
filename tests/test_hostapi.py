"""Builds and runs the C++ programs that exercise the host-side mirror of the reference API."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "asc-devkit_clone_b200")


def _build(name, tmp_path, link_library=True):
    if shutil.which("g++") is None:
        pytest.skip("g++ not available")
    if link_library and not os.path.exists(os.path.join(PKG, "libascb200.so")):
        pytest.skip("libascb200.so not built (needs nvcc)")
    exe = os.path.join(str(tmp_path), name)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(PKG, "hostapi"),
           os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", exe]
    if link_library:
        cmd += ["-L" + PKG, "-lascb200", "-Wl,-rpath," + PKG]
    subprocess.check_call(cmd)
    return exe


def test_host_tiling_known_answers(tmp_path):
    # the tiling mirror asks the library for the SM count (PlatformAscendC::GetCoreNum): it links the C ABI like the operators
    out = subprocess.run([_build("test_tiling", tmp_path)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "tiling ok" in out.stdout


def test_hostapi_compiles_without_gpu(tmp_path):
    """The operator mirror must at least compile and link against the C ABI on a machine without a GPU."""
    _build("test_hostapi", tmp_path)


@pytest.mark.gpu
def test_hostapi_on_gpu(tmp_path):
    out = subprocess.run([_build("test_hostapi", tmp_path)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "hostapi ok" in out.stdout
