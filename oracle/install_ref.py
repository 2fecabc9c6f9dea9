"""Recipe that puts the reference's own files for the key-cache path next to the oracle, untouched.

    python oracle/install_ref.py [/path/to/PolarQuant-checkout]      (default: $POLARQUANT_REFERENCE, else the checkout beside the home directory's repository)

Test infrastructure, like everything under ``oracle/``: the copies land in ``oracle/_ref/`` (listed in
``.gitignore``, so they never enter the history, and imported by nothing in the ``polarquant_b200`` package).  They
let the GPU tests and the benchmark's reference arm run the reference ITSELF where its checkout does not exist:

* ``models/modeling_llama_polar.py`` / ``models/modeling_qwen_polar.py`` - the attention patches whose decode
  branch (``:61-101`` / ``:60-100``) and quantizer method (``:135-157`` / ``:134-156``) define the path;
* ``models/kernel4group.py`` - the Triton kernel and its wrapper (``:14-109``), the same-GPU yardstick of the
  logits entry point;
* ``benchmark/benchmark_matmul.py`` - the reference's own micro-benchmark of that entry point (``:89-120``).

Files are copied byte for byte; a manifest with their SHA-256 is written beside them so a test can tell that what
it ran is what the checkout held.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = (
    "models/kernel4group.py",
    "models/modeling_llama_polar.py",
    "models/modeling_qwen_polar.py",
    "benchmark/benchmark_matmul.py",
)


def default_source() -> str:
    return os.environ.get("POLARQUANT_REFERENCE", os.path.join(os.sep, "root", "reference"))


def installed() -> bool:
    return all(os.path.isfile(os.path.join(DEST, f)) for f in FILES)


def install(source: str | None = None) -> str:
    """Copy the path's files from the checkout at ``source`` into ``oracle/_ref``; returns that directory."""
    source = source or default_source()
    missing = [f for f in FILES if not os.path.isfile(os.path.join(source, f))]
    if missing:
        raise FileNotFoundError(f"{source} is not a PolarQuant checkout (missing {missing})")
    manifest = {}
    for rel in FILES:
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(source, rel), dst)
        with open(dst, "rb") as f:
            manifest[rel] = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(DEST, "MANIFEST.json"), "w") as f:
        json.dump({"source": "ericshwu/PolarQuant", "files": manifest}, f, indent=1)
    return DEST


if __name__ == "__main__":
    print(install(sys.argv[1] if len(sys.argv) > 1 else None))
