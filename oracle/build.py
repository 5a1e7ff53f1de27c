"""Build recipe for the CPU oracle (test infrastructure, not part of the product).

`build()` compiles norm_dist_oracle.c into liboracle.so next to this file with gcc.
Single IEEE fp32 operations are required for the bit-exact comparisons, hence
-ffp-contract=off and no fast-math.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "norm_dist_oracle.c")
LIB = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
           "-o", LIB, SRC, "-lm"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
