"""Build recipe for the CPU oracle (test infrastructure, never shipped).

`python oracle/build.py` compiles oracle/dg_oracle.c into
oracle/libdgoracle.so with gcc.  The reference crate is Rust and no Rust
toolchain exists in this environment, so there is no `oracle/_ref` build of
the reference's own sources; the C file restates its algorithm instead.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "dg_oracle.c")
OUT = os.path.join(HERE, "libdgoracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-shared", "-fPIC",
           "-fvisibility=hidden", "-o", OUT, SRC, "-lm"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
