"""Build the C restatement of the reference's CPU kernel (test infrastructure).

    python oracle/build.py

produces ``oracle/libhlq_cpu_oracle.so``.  The reference's own C++ sources are
ARM-NEON only and cannot be compiled for x86-64, so there is no ``oracle/_ref``
build; the restatement in ``cpu_lut_gemv.c`` stands in for it.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libhlq_cpu_oracle.so")
SRC = os.path.join(HERE, "cpu_lut_gemv.c")


def build(force: bool = False) -> str:
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    # -O2 as the reference's CMake uses; a fixed ISA level (AVX2 + F16C + FMA) instead
    # of -march=native so that the library built on one x86-64 host runs on another.
    cmd = ["gcc", "-O2", "-mavx2", "-mf16c", "-mfma", "-ffp-contract=off", "-fopenmp",
           "-shared", "-fPIC", "-o", LIB, SRC]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
