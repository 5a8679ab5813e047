"""Compile the CPU checker (oracle/kvc_oracle.c) into oracle/libkvc_oracle.so.

Test infrastructure only: the product never imports or links this.  OpenMP is used
when the compiler has it (it only speeds up the timed CPU baseline); the results do
not depend on the thread count.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "kvc_oracle.c")
OUT = os.path.join(HERE, "libkvc_oracle.so")
BASE = ["-O2", "-fPIC", "-std=gnu11", "-Wall", "-Wno-unused-function", "-Wno-unknown-pragmas",
        "-ffp-contract=off", "-shared"]


def _compilers():
    seen = []
    for c in ("/usr/bin/gcc", os.environ.get("CC"), shutil.which("gcc"), shutil.which("cc")):
        if c and c not in seen and os.path.exists(c):
            seen.append(c)
    return seen


def build(force=False):
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    errors = []
    for cc in _compilers():
        for omp in (["-fopenmp"], []):
            cmd = [cc] + BASE + omp + ["-o", OUT, SRC, "-lm"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return OUT
            errors.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("could not compile the oracle:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
