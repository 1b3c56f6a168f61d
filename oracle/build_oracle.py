"""Compiles oracle/nnf_oracle.c (test infrastructure) into a serial and an OpenMP shared library.

Serial build = the deterministic checker; OpenMP build = the timed CPU baseline ("port").
No -ffast-math and -ffp-contract=off: signed zeros and the two roundings of x*mult+add must match
what the reference's plain backend produces when built the same way.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "nnf_oracle.c")
LIB = os.path.join(HERE, "libnnf_oracle.so")
LIB_OMP = os.path.join(HERE, "libnnf_oracle_omp.so")
FLAGS = ["-std=c99", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math"]


def build():
    for lib, extra in ((LIB, []), (LIB_OMP, ["-fopenmp"])):
        if os.path.exists(lib) and os.path.getmtime(lib) >= os.path.getmtime(SRC):
            continue
        subprocess.check_call(["gcc"] + FLAGS + extra + [SRC, "-o", lib, "-lm"])
    return True


if __name__ == "__main__":
    sys.exit(0 if build() else 1)
