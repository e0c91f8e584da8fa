"""Compiles the C restatement of the oracle (oracle/nvfp4_oracle.c) into oracle/_ref/.

    python oracle/build.py

The reference itself cannot be compiled here: its kernels are TIRx Python that needs the
external `tvm.tirx` compiler, so there is no `oracle/_ref` build of reference sources; the
directory only holds the shared object of this repository's own C restatement.
"""

from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
SOURCE = HERE / "nvfp4_oracle.c"
LIBRARY = OUT_DIR / "libnvfp4_oracle.so"


def build(force: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    if not force and LIBRARY.exists() and LIBRARY.stat().st_mtime >= SOURCE.stat().st_mtime:
        return LIBRARY
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
           "-o", str(LIBRARY), str(SOURCE), "-lm"]
    subprocess.run(cmd, check=True)
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True))
