"""Builds ``libgqa_b200.so`` (and the C++ harness) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")


def build(target: str = "all", jobs: int | None = None, quiet: bool = True) -> str:
    """Run ``make`` in ``csrc/``; returns the path of the shared library."""
    jobs = jobs or max(1, os.cpu_count() or 1)
    cmd = ["make", "-C", CSRC, f"-j{jobs}", target]
    out = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if out.returncode != 0:
        raise RuntimeError("building libgqa_b200.so failed:\n" + out.stdout[-4000:])
    if not quiet:
        print(out.stdout)
    return os.path.join(HERE, "libgqa_b200.so")


if __name__ == "__main__":
    print(build(quiet=False))
