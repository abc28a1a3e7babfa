"""Identity of the CUDA sources: what libfpkv.so was built from must be what
the tree holds.  The build script passes this value to the compiler, the
library returns it from ``fpkv_build_id()``, and the loader compares the two."""

from __future__ import annotations

import hashlib
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
HEADER = os.path.join(_PKG, "..", "include", "fpkv.h")


def source_files():
    names = sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h")))
    return [os.path.join(CSRC, f) for f in names] + [HEADER]


def source_hash() -> str | None:
    """First 16 hex digits of the sha256 over the kernel sources and the C
    header (file names and contents, sorted by name); None when the sources are
    not there (a deployment that ships the built library only)."""
    if not os.path.isdir(CSRC) or not os.path.exists(HEADER):
        return None
    h = hashlib.sha256()
    for path in source_files():
        h.update(os.path.basename(path).encode() + b"\0")
        with open(path, "rb") as f:
            h.update(f.read())
        h.update(b"\0")
    return h.hexdigest()[:16]
