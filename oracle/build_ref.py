"""Compile the reference's own CPU path into ``oracle/_ref/`` (test infrastructure).

The reference's translation unit ``src/scanscam_cpu.cpp`` (with ``src/scanscam_cpu.hpp``)
is compiled where it lies, unmodified, as a torch C++ extension named
``scanscam_ref_ext``; only the built module lands in ``oracle/_ref/``.  No reference
source is copied.  The module is used to validate the C restatement in
``scan_oracle.c`` and as the timed CPU baseline of the benchmark.

Usage:  python oracle/build_ref.py [path-to-reference-checkout]
"""
from __future__ import annotations

import os
import sys

# The reference checkout: SCANSCAM_REFERENCE_DIR if set, else a directory named `reference` beside
# this repository.
DEFAULT_REFERENCE = os.environ.get("SCANSCAM_REFERENCE_DIR") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def build_reference(ref_root: str = DEFAULT_REFERENCE, verbose: bool = False) -> str | None:
    """Returns the path of the built module, or None when the sources are absent."""
    here = os.path.dirname(os.path.abspath(__file__))
    out_dir = os.path.join(here, "_ref")
    src = os.path.join(ref_root, "src", "scanscam_cpu.cpp")
    existing = [f for f in (os.listdir(out_dir) if os.path.isdir(out_dir) else [])
                if f.startswith("scanscam_ref_ext") and f.endswith(".so")]
    if not os.path.exists(src):
        return os.path.join(out_dir, existing[0]) if existing else None
    if existing and os.path.getmtime(os.path.join(out_dir, existing[0])) >= os.path.getmtime(src):
        return os.path.join(out_dir, existing[0])
    os.makedirs(out_dir, exist_ok=True)
    from torch.utils.cpp_extension import load

    mod = load(name="scanscam_ref_ext", sources=[src], build_directory=out_dir,
               extra_cflags=["-O3"], verbose=verbose)
    return mod.__file__


if __name__ == "__main__":
    path = build_reference(*(sys.argv[1:2]), verbose=True)
    print(path if path else "reference sources not found; nothing built")
