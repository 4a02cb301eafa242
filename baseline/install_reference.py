"""Puts the unmodified reference package where `bench.py --impl reference` looks for it: `baseline/_ref`.

    python baseline/install_reference.py [SOURCE]

SOURCE is the reference's checkout (default: the environment variable
LITEINFER_REFERENCE_SRC, else a folder `reference` beside this repository).
First the offline pip install is tried.  The reference is a pure-Python
package whose wheel holds nothing but its `liteinfer/` folder, so where pip
cannot build it (its build backend is not in the offline wheelhouse) the
folder is copied as it is; nothing is compiled or changed either way.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def default_source() -> Path:
    given = os.environ.get("LITEINFER_REFERENCE_SRC")
    return Path(given) if given else HERE.parent.parent / "reference"


def install(source: Path | None = None, quiet: bool = False) -> str:
    """Returns how the package got there: "present", "pip", "copied" or "missing: <why>"."""
    if (TARGET / "liteinfer" / "__init__.py").is_file():
        return "present"
    source = source or default_source()
    if not (source / "liteinfer" / "__init__.py").is_file():
        return f"missing: no reference checkout at {source}"
    pip = subprocess.run(
        [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--find-links",
         "/opt/wheelhouse", "--target", str(TARGET), str(source)], capture_output=True, text=True)
    if pip.returncode == 0 and (TARGET / "liteinfer" / "__init__.py").is_file():
        return "pip"
    if not quiet:
        print("pip could not build the reference:", pip.stderr.strip().splitlines()[-1:] or pip.stdout[-200:])
    TARGET.mkdir(parents=True, exist_ok=True)
    shutil.copytree(source / "liteinfer", TARGET / "liteinfer", dirs_exist_ok=True,
                    ignore=shutil.ignore_patterns("__pycache__"))
    return "copied"


if __name__ == "__main__":
    print(install(Path(sys.argv[1]) if len(sys.argv) > 1 else None))
