"""Build libfpkv.so in-tree with nvcc for sm_100a.

    python falcon-perception_b200/build.py [--force] [--verbose]

The shared library lands beside the Python package (fpkv/libfpkv.so) so that
it is found without installation.  Nothing is built at import time: the
package refuses to load without the library, or with one built from other
sources than the tree holds.  A hash of the sources is compiled in
(``fpkv_build_id()``); a build is skipped only when the existing library
reports the hash of the present sources.
"""

import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)
from fpkv._srchash import CSRC, source_hash  # noqa: E402  (does not load the library)

OUT = os.path.join(HERE, "fpkv", "libfpkv.so")
SOURCES = ["api.cu", "append.cu", "pre_append.cu", "decode_portable.cu", "decode_tma.cu", "decode_static.cu",
           "prefill_tc.cu", "tables.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--use_fast_math", "-Xcompiler", "-fPIC,-O3,-fvisibility=hidden", "-shared"]


def built_id(path=OUT):
    """Source hash the library at ``path`` was compiled from, or None.  Read from the marker string in
    the file, not through dlopen: a process that loaded an older build would be handed that one again."""
    if not os.path.exists(path):
        return None
    with open(path, "rb") as f:
        m = re.search(rb"fpkv-build-id:([0-9a-f]{16})", f.read())
    return m.group(1).decode() if m else None


def build(force=False, verbose=False):
    want = source_hash()
    if not force and built_id() == want:
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    tmp = OUT + ".tmp"
    cmd = [nvcc] + NVCC_FLAGS + [f'-DFPKV_SRC_HASH="{want}"'] + (["-Xptxas", "-v"] if verbose else []) + \
          [os.path.join(CSRC, s) for s in SOURCES] + ["-o", tmp]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfpkv.so")
    os.replace(tmp, OUT)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(OUT, built_id())
