"""The C-ABI library must load without a GPU and export every function include/ascb200.h declares;
without a device, compute entry points report ASCB200_ENODEV instead of computing anything on the CPU."""
import ctypes as C
import os
import re

import ascb200 as ab

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ascb200.h")).read()
    return re.findall(r"ASCB200_API\s+(?:const\s+)?\w+\*?\s+(\w+)\s*\(", text)


def test_every_declared_symbol_is_exported():
    names = declared_functions()
    assert len(names) >= 30 and "ascb200_gemm" in names and "ascb200_softmax_quant" in names
    lib = ab.lib()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(set(ab.EXPORTS) - set(names)) == []   # the Python binding names nothing the header does not declare


def test_no_cpu_fallback_without_device():
    lib = ab.lib()
    rc = lib.ascb200_init(0)
    if rc == 0:   # running on a GPU box: nothing to check here
        return
    assert rc == -4
    assert lib.ascb200_softmax(None, None, None, None, 4, 64, ab.F16, 0, None) == -4
    d = ab.GemmDesc()
    assert lib.ascb200_gemm(C.byref(d), None) == -4
    assert lib.ascb200_dequant(None, None, 1, 8, 8, 8, ab.F32, None, ab.F32, C.c_float(1.0), None) == -4
    assert b"sm_100" in lib.ascb200_strerror(-4)


def test_binding_declares_argument_types_for_every_export():
    """ctypes passes an untyped Python int as a 32-bit C int: an entry point without argtypes would receive truncated
    device pointers.  Every export that takes arguments must have them declared."""
    lib = ab.lib()
    no_args = {"ascb200_last_cuda_error", "ascb200_sm_count"}
    untyped = [n for n in ab.EXPORTS if n not in no_args and getattr(lib, n).argtypes is None]
    assert not untyped, untyped
