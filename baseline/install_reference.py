"""Install the unmodified reference into baseline/_ref (git-ignored; it travels to the GPU box).

Step 1 is the plain offline pip install of the reference's source tree.  The reference's
setup.py collects its packages with setuptools.find_packages(), which skips directories
without an __init__.py; zipage/engine, zipage/kernel, zipage/layers, zipage/utils and the
nanovllm sub-packages are such directories, so the wheel pip builds holds only the top-level
modules and `import zipage` fails on it.  (The reference's README installs it in editable
mode, where the source tree itself is imported and the omission does not show.)  Step 2
therefore completes the install: every .py file of the two package trees that pip left
out is copied verbatim next to the installed ones.  Nothing is edited.

Only the GPU tests that compare this library with the reference's own Triton kernels and
engine read baseline/_ref, and only when it is present.

usage: python baseline/install_reference.py <reference source tree>
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def install(src: Path) -> None:
    with tempfile.TemporaryDirectory() as tmp:
        # pip builds inside the tree it is given; the source tree may be read-only
        work = Path(tmp) / "reference"
        shutil.copytree(src, work)
        if DEST.exists():
            shutil.rmtree(DEST)
        subprocess.run(
            [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation",
             "--find-links", "/opt/wheelhouse", "--no-deps", "--target", str(DEST), str(work)],
            check=True)
    added = 0
    for pkg, root in (("zipage", src / "zipage"), ("nanovllm", src / "third_party" / "nanovllm")):
        for f in root.rglob("*.py"):
            out = DEST / pkg / f.relative_to(root)
            if not out.exists():
                out.parent.mkdir(parents=True, exist_ok=True)
                shutil.copyfile(f, out)
                added += 1
    print(f"reference installed in {DEST} ({added} module files completed after pip)")


if __name__ == "__main__":
    source = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ZIPAGE_REFERENCE_SRC")
    if not source:
        sys.exit("usage: python baseline/install_reference.py <reference source tree> (or set ZIPAGE_REFERENCE_SRC)")
    install(Path(source))
