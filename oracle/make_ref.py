"""Stage the unmodified reference package for the benchmark's CPU reference arm.  TEST INFRASTRUCTURE.

    python oracle/make_ref.py [--reference /path/to/Griffin]      (or set GRIFFIN_REFERENCE)

The reference is pure Python (griffin/__init__.py, griffin/griffin.py, griffin/triton_scan.py), so "building"
it for the CPU arm means placing those files, untouched, under ``oracle/_ref/griffin`` -- a directory that is
listed in .gitignore (reference sources never enter this repository's history) but travels with the working
tree to the machine the benchmark runs on.  ``bench.py --impl reference`` imports ``RG_LRU`` from there and
times ``scan_mode="sequential"`` (griffin/griffin.py:280-284); when the directory is absent it times the
oracle's restatement instead and says so (``cpu_baseline.kind``).
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = ("__init__.py", "griffin.py", "triton_scan.py")


def stage_reference(reference_root: str) -> str:
    """Copy the reference's package files into oracle/_ref/griffin and return that directory."""
    src = os.path.join(reference_root, "griffin")
    missing = [f for f in FILES if not os.path.isfile(os.path.join(src, f))]
    if missing:
        raise FileNotFoundError(f"{src} lacks {missing}: not a checkout of the reference project")
    dst = os.path.join(REF_DIR, "griffin")
    os.makedirs(dst, exist_ok=True)
    lines = []
    for name in FILES:
        shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
        with open(os.path.join(dst, name), "rb") as fh:
            lines.append(f"{hashlib.sha256(fh.read()).hexdigest()}  griffin/{name}")
    with open(os.path.join(REF_DIR, "SHA256SUMS"), "w") as fh:
        fh.write("\n".join(lines) + "\n")
    return dst


def import_reference():
    """The staged reference package as a module, or None when it has not been staged."""
    if not os.path.isfile(os.path.join(REF_DIR, "griffin", "griffin.py")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import griffin  # the unmodified reference

    return griffin


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("GRIFFIN_REFERENCE"))
    args = ap.parse_args()
    if not args.reference or not os.path.isdir(args.reference):
        ap.error("pass --reference <checkout of the reference project> (or set GRIFFIN_REFERENCE)")
    print(stage_reference(args.reference))


if __name__ == "__main__":
    main()
