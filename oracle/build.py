"""Build recipe for the CPU oracle (test infrastructure).

`build()` compiles oracle.c — the plain-C restatement of the reference's
arithmetic — into oracle/_build/liboracle.so with gcc.  The reference itself is
Rust + Metal; neither toolchain exists here, so there is nothing to compile
into oracle/_ref/ and the restatement is the only checker.
"""
from __future__ import annotations

import hashlib
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "oracle.c"
OUT = HERE / "_build"
LIB = OUT / "liboracle.so"
HASH = OUT / "liboracle.build_hash"
FLAGS = ["-O2", "-mf16c", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]


def build(force: bool = False) -> Path:
    h = hashlib.sha256(SRC.read_bytes() + " ".join(FLAGS).encode()).hexdigest()
    if not force and LIB.exists() and HASH.exists() and HASH.read_text().strip() == h:
        return LIB
    OUT.mkdir(exist_ok=True)
    subprocess.run(["gcc", *FLAGS, "-o", str(LIB), str(SRC), "-lm"], check=True)
    HASH.write_text(h + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force=True))
