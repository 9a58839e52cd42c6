"""Stage the reference's own PyTorch Kascade strategy for timing and cross-checks (TEST INFRASTRUCTURE ONLY).

    python oracle/make_ref.py --reference /path/to/kascade

The reference's ``KascadeStrategy`` and the classes it inherits from are plain-torch files
(strategies/KascadeStrategy.py and its parents: PostSoftmaxPooledPrefillTopkStrategy.py,
PostSoftmaxGQAPooledOracleTopKStrategy.py, OracleTopkLayer0GlobalStrategy.py, OracleTopkStrategy.py,
BaselineStrategy.py, Strategy.py, attention_utils.py).  This recipe copies exactly those files,
unmodified, from a checkout of the reference into ``oracle/_ref/kascade_ref/strategies/`` — a folder
that version control ignores, so no reference source ever enters this repository — and writes an
empty package marker beside them (the reference's own ``strategies/__init__.py`` is NOT staged: it
imports the TileLang kernels of the efficient strategy, which cannot run on this hardware).

``load_reference_strategy()`` imports the staged class; it is used by the CPU-baseline leg and the
``--impl reference`` arm of ``bench.py`` and by tests, never by the product path.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")
PKG = os.path.join(REF_ROOT, "kascade_ref")

FILES = [
    "Strategy.py", "BaselineStrategy.py", "attention_utils.py", "OracleTopkStrategy.py",
    "OracleTopkLayer0GlobalStrategy.py", "PostSoftmaxGQAPooledOracleTopKStrategy.py",
    "PostSoftmaxPooledPrefillTopkStrategy.py", "KascadeStrategy.py",
]


def stage(reference: str) -> str:
    """Copy the files listed in FILES from `reference`/src/strategies; returns the staged folder."""
    src = os.path.join(reference, "src", "strategies")
    dst = os.path.join(PKG, "strategies")
    os.makedirs(dst, exist_ok=True)
    lines = []
    for name in FILES:
        path = os.path.join(src, name)
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: not a checkout of the reference")
        shutil.copyfile(path, os.path.join(dst, name))
        with open(path, "rb") as f:
            lines.append(f"{hashlib.sha256(f.read()).hexdigest()}  strategies/{name}")
    for marker in (os.path.join(PKG, "__init__.py"), os.path.join(dst, "__init__.py")):
        with open(marker, "w") as f:
            f.write("# package marker written by oracle/make_ref.py (not a reference file)\n")
    with open(os.path.join(REF_ROOT, "MANIFEST.sha256"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return dst


def available() -> bool:
    return all(os.path.exists(os.path.join(PKG, "strategies", n)) for n in FILES)


def load_reference_strategy():
    """The reference's unmodified ``KascadeStrategy`` class from the staged files."""
    if not available():
        raise RuntimeError("oracle/_ref is not staged: run `python oracle/make_ref.py --reference <checkout>`")
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    return importlib.import_module("kascade_ref.strategies.KascadeStrategy").KascadeStrategy


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of microsoft/kascade (read only)")
    a = ap.parse_args()
    print(stage(a.reference))
