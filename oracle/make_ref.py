"""Stage the reference project's own, unmodified files under oracle/_ref/.

    python oracle/make_ref.py /path/to/monarch-muon-checkout

TEST INFRASTRUCTURE ONLY.  oracle/_ref/ is git-ignored: nothing of the
reference enters this repository's history.  The staged copy exists so that
machines which hold this repository's working tree but not the reference
checkout (a GPU box) can still run the reference itself as the arbiter:

  * its FP8 optimizer-state kernels (pretrain/src/models/monarch/
    coat_state_muon.py:22-114, pretrain/third_party/coat/optimizer/
    triton_kernels.py) JIT-compiled by Triton on the GPU, for the bit-exact
    codec tests;
  * its optimizer classes (pretrain/src/models/monarch/monarch_muon.py,
    membench/src/models/monarch/monarch_muon.py, finetune/sft_optimizer.py) on
    the GPU and on the host cores, for the reference arms of bench.py;
  * its training loop (pretrain/src/main.py, pretrain/src/optim/base.py) for the
    drop-in test that swaps in this library's optimizer.

Files are copied byte for byte; MANIFEST.json records a SHA-256 of each so a
test can verify that nothing was edited.  Only tests/, bench.py's reference
legs and __graft_entry__ may touch oracle/_ref/.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

# (path inside the reference project, kind)
TREES = (
    "pretrain/src",
    "pretrain/third_party",
    "membench/src/models",
    "membench/scripts/monarch_benchmark",
)
FILES = (
    "pretrain/train.py",
    "pretrain/tests/arm_build.py",
    "pretrain/tests/conftest.py",
    "pretrain/tests/test_coat_state_muon.py",
    "finetune/sft_optimizer.py",
)
SKIP_DIRS = {"__pycache__", ".git"}
KEEP_EXT = {".py", ".cpp", ".json", ".txt", ".md", ""}


def _sha(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _copy(src: str, rel: str, manifest: dict) -> None:
    dst = os.path.join(DEST, rel)
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    shutil.copyfile(src, dst)
    manifest[rel] = _sha(dst)


def stage(reference_root: str) -> str:
    reference_root = os.path.abspath(reference_root)
    if not os.path.isdir(os.path.join(reference_root, "pretrain", "src", "models", "monarch")):
        raise FileNotFoundError(f"{reference_root} does not look like the reference checkout")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    manifest: dict = {}
    for tree in TREES:
        top = os.path.join(reference_root, tree)
        for dirpath, dirnames, filenames in os.walk(top):
            dirnames[:] = sorted(d for d in dirnames if d not in SKIP_DIRS)
            for name in sorted(filenames):
                if os.path.splitext(name)[1] not in KEEP_EXT:
                    continue
                src = os.path.join(dirpath, name)
                _copy(src, os.path.relpath(src, reference_root), manifest)
    for rel in FILES:
        _copy(os.path.join(reference_root, rel), rel, manifest)
    with open(os.path.join(DEST, "MANIFEST.json"), "w") as f:
        json.dump({"files": manifest}, f, indent=1, sort_keys=True)
    return DEST


def verify() -> bool:
    """True if oracle/_ref/ exists and every staged file still has the recorded hash."""
    path = os.path.join(DEST, "MANIFEST.json")
    if not os.path.exists(path):
        return False
    with open(path) as f:
        manifest = json.load(f)["files"]
    return all(os.path.exists(os.path.join(DEST, rel)) and _sha(os.path.join(DEST, rel)) == digest
               for rel, digest in manifest.items())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(stage(sys.argv[1]), "staged;", "verified" if verify() else "VERIFY FAILED")
