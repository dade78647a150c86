"""Stage the files of a Self-Forcing checkout that the full-model harness imports.

    SF_REFERENCE_ROOT=/path/to/Self-Forcing python baseline/stage_reference.py

Copies, unmodified, the Python sources the causal rollout needs (the DiT, the wrapper, the scheduler,
the pipeline and the modules they import) into ``baseline/_ref/``, which version control ignores.
Nothing of the product imports that folder: ``baseline/reference_harness.py`` and ``bench.py --model``
do, and they skip when it is absent.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"

# directories are copied recursively (``*.py`` only), files as they are
WANTED = [
    "wan/modules",
    "utils/resolution.py",
    "utils/scheduler.py",
    "utils/wan_wrapper.py",
    "pipeline/causal_inference.py",
    "demo_utils/memory.py",
]


def stage(root: Path, dest: Path = DEST) -> int:
    n = 0
    for rel in WANTED:
        src = root / rel
        if src.is_dir():
            files = [p for p in src.rglob("*.py")]
        elif src.is_file():
            files = [src]
        else:
            raise FileNotFoundError(f"{src} not found: is SF_REFERENCE_ROOT a Self-Forcing checkout?")
        for f in files:
            out = dest / f.relative_to(root)
            out.parent.mkdir(parents=True, exist_ok=True)
            shutil.copyfile(f, out)
            n += 1
    return n


if __name__ == "__main__":
    root = os.environ.get("SF_REFERENCE_ROOT") or (sys.argv[1] if len(sys.argv) > 1 else None)
    if not root:
        sys.exit("set SF_REFERENCE_ROOT (or pass the checkout's path)")
    print(f"staged {stage(Path(root))} files into {DEST}")
