"""Compile oracle/d2d_oracle.c into oracle/_build/libd2d_oracle.so (gcc).  Test infrastructure."""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "d2d_oracle.c"
OUT = HERE / "_build" / "libd2d_oracle.so"


def build(force: bool = False) -> Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-ffp-contract=off", str(SRC), "-o", str(OUT),
                    "-lm"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
