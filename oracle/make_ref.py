"""Brings the reference's own CPU forward next to the oracle, for the benchmark's reference arm.

    python oracle/make_ref.py [/path/to/reference]      (default: the BRASA_REFERENCE environment variable, else REFERENCE_DEFAULT)

The reference's CPU implementation of the token loop is three Python files (tools/qwen3_ref.py, tools/brasa_file.py,
tools/convert_brasa.py: torch and numpy only). They are copied, unmodified, from the checkout into oracle/_ref/, which
is ignored by git (nothing of the reference enters the history) but travels with a working copy to the machine that
runs the benchmark. `bench.py --impl reference` times Qwen3Ref from there when it is present and falls back to the C
port of this directory otherwise. Nothing else reads oracle/_ref/.
"""

from __future__ import annotations

import os
import pathlib
import shutil
import sys

HERE = pathlib.Path(__file__).resolve().parent
FILES = ("qwen3_ref.py", "brasa_file.py", "convert_brasa.py")
REFERENCE_DEFAULT = pathlib.Path(os.environ.get("BRASA_REFERENCE", str(HERE.parents[1] / "reference")))


def make(reference: str | pathlib.Path = REFERENCE_DEFAULT) -> bool:
    """Copies the tools when the checkout is there; returns whether oracle/_ref/ holds them afterwards."""
    src = pathlib.Path(reference) / "tools"
    dst = HERE / "_ref"
    if all((src / f).exists() for f in FILES):
        dst.mkdir(exist_ok=True)
        for f in FILES:
            shutil.copyfile(src / f, dst / f)
    return all((dst / f).exists() for f in FILES)


if __name__ == "__main__":
    ok = make(sys.argv[1] if len(sys.argv) > 1 else REFERENCE_DEFAULT)
    print("oracle/_ref ready" if ok else "reference checkout not found: oracle/_ref not made")
