"""Places the reference's ``ops`` package under ``baseline/_ref/`` (git-ignored) for the GPU side arm of bench.py.

    python baseline/install_ref.py --ref <reference checkout>

The reference is a flat tree without packaging metadata (no setup.py; its pyproject.toml holds tool settings
only), so ``pip install --target baseline/_ref <checkout>`` stops at "Multiple top-level packages discovered in a
flat-layout".  What such an install would have produced for the part this repository times is the ``ops`` package
directory, unmodified; this script puts exactly that there.  Nothing under ``baseline/_ref`` is committed.
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
FILES = ("mini_vq.py", "attn_vq.py", "triton_fused_vq_attn.py", "triton_fused_local_attn_rerope.py")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference checkout")
    a = ap.parse_args()
    ref, dst = Path(a.ref), HERE / "_ref"
    r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                        "--target", str(dst), str(ref)], capture_output=True, text=True)
    if r.returncode == 0:
        print("pip install succeeded")
        return
    print("pip install failed (" + (r.stderr.strip().splitlines() or ["?"])[-1][:120] + "); copying the ops package files")
    (dst / "ops").mkdir(parents=True, exist_ok=True)
    for f in FILES:
        shutil.copyfile(ref / "ops" / f, dst / "ops" / f)
    print("installed", ", ".join(FILES), "->", dst / "ops")


if __name__ == "__main__":
    main()
