"""Build recipe for the CPU oracle: oracle/asc_oracle.c -> oracle/liboracle.so (gcc, OpenMP).

There is no oracle/_ref here: the reference's own CPU path for these operators needs the closed
CANN CPU-twin libraries (tikicpulib, cpudebug, pem_davinci) and the bisheng compiler, none of which
are in the reference tree, so nothing of the reference can be compiled from its own sources.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))


def build_oracle(force=False):
    src = os.path.join(HERE, "asc_oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-Wall", "-o", out, src,
           "-lm"]
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build_oracle(force=True))
