"""Installs the reference's Triton package as a same-box comparator: baseline/_ref/flashlinear_triton_ref.

    python baseline/install_reference.py <path of the reference checkout>

The reference (flashlinear 0.2.1) is pure Python + Triton, so "installing" it is a copy of its
`flashlinear/` package directory. Two changes are made to the copy, nothing else:

1. The package is renamed to `flashlinear_triton_ref`, because this repository's drop-in package
   already owns the import name `flashlinear`. The reference only uses relative imports, so the
   rename needs no edit inside the files.
2. Eight lines of the four kernels build a one-element tuple and then call `.to(tl.int64)` on it
   (flashlinear/kernels/linear_attn_kernels.py:24-25,119-120 and
   flashlinear/kernels/linear_attn_kernels_smallv_hd.py:26-27,126-127):
       off_bs = (bh_pid // num_head,)   ->   off_bs = bh_pid // num_head
       off_h = (bh_pid % num_head,)     ->   off_h = bh_pid % num_head
   Triton 2.1/2.2 (what the reference's README pins) accepted that; Triton 3.6 refuses to compile
   it. Every number measured from this copy is labelled "reference (Triton 3.6, tuple fix)".

The copy is a comparator for tests and timing only (tests/test_triton_reference_gpu.py); nothing
in the product path imports it. baseline/_ref/ is not tracked by git.
"""
from __future__ import annotations

import os
import re
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "flashlinear_triton_ref")
TUPLE_LINE = re.compile(r"^(\s*off_(?:bs|h) = )\((bh_pid (?://|%) num_head),\)\s*$")


def install(reference_root: str) -> str:
    src = os.path.join(reference_root, "flashlinear")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"{src} not found")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    shutil.copytree(src, DEST, ignore=shutil.ignore_patterns("__pycache__", "test_*.py"))
    fixed = 0
    for name in ("linear_attn_kernels.py", "linear_attn_kernels_smallv_hd.py"):
        path = os.path.join(DEST, "kernels", name)
        with open(path) as f:
            lines = f.read().split("\n")
        for i, line in enumerate(lines):
            m = TUPLE_LINE.match(line)
            if m:
                lines[i] = m.group(1) + m.group(2)
                fixed += 1
        with open(path, "w") as f:
            f.write("\n".join(lines))
    if fixed != 8:
        raise RuntimeError(f"expected to fix 8 one-tuple lines, fixed {fixed}")
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(install(sys.argv[1]))
