"""CPU: a plain C program (no Python, no torch types) can use the library through
include/fpkv.h: it compiles against the header, loads libfpkv.so, finds every
entry point and gets the documented error codes from argument validation."""

import os
import subprocess
import sys

import pytest

from fpkv import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C_SOURCE = r"""
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>
#include "fpkv.h"

typedef int (*version_fn)(void);
typedef const char* (*strerror_fn)(int);
typedef int (*append_fn)(const fpkv_pool*, int32_t, const int64_t*, const void*, int32_t, const void*, int64_t, int64_t,
                         const void*, int64_t, int64_t, int32_t, int32_t*, void*);
typedef int (*ws_fn)(const fpkv_pool*, int32_t, int32_t, int32_t, size_t*);

int main(int argc, char** argv) {
    void* h = dlopen(argv[1], RTLD_NOW);
    if (!h) { printf("dlopen failed: %s\n", dlerror()); return 1; }
    const char* names[] = {"fpkv_version", "fpkv_build_id", "fpkv_strerror", "fpkv_alloc_step", "fpkv_append_decode",
                           "fpkv_append_packed", "fpkv_pre_append", "fpkv_gather", "fpkv_decode_workspace_bytes",
                           "fpkv_decode_attn", "fpkv_prefill_attn", "fpkv_decode_attn_static"};
    for (unsigned i = 0; i < sizeof(names) / sizeof(names[0]); ++i)
        if (!dlsym(h, names[i])) { printf("missing %s\n", names[i]); return 2; }
    version_fn version = (version_fn)dlsym(h, "fpkv_version");
    strerror_fn err = (strerror_fn)dlsym(h, "fpkv_strerror");
    append_fn append = (append_fn)dlsym(h, "fpkv_append_decode");
    ws_fn ws = (ws_fn)dlsym(h, "fpkv_decode_workspace_bytes");
    if (version() < 100 || strcmp(err(FPKV_OK), "ok") != 0) return 3;
    static long long buf[64];                                 /* aligned host memory, never dereferenced */
    fpkv_pool pool = {buf, (const int64_t*)buf, (const int64_t*)buf, 1, 8, 64, 128, 128, 9, FPKV_BF16, 0};
    if (append(NULL, 0, (const int64_t*)buf, buf, FPKV_I32, buf, 1024, 128, buf, 1024, 128, 4, NULL, NULL) != FPKV_EINVAL) return 4;
    pool.head_dim = 80;
    if (append(&pool, 0, (const int64_t*)buf, buf, FPKV_I32, buf, 1024, 128, buf, 1024, 128, 4, NULL, NULL) != FPKV_ESHAPE) return 5;
    pool.head_dim = 128;
    if (append(&pool, 0, (const int64_t*)buf, buf, FPKV_I32, (char*)buf + 4, 1024, 128, buf, 1024, 128, 4, NULL, NULL) != FPKV_EALIGN) return 6;
    if (append(&pool, 0, (const int64_t*)buf, buf, FPKV_I32, buf, 1024, 128, buf, 1024, 128, 0, NULL, NULL) != FPKV_OK) return 7;
    size_t need = 0;
    if (ws(&pool, 64, 16, FPKV_DECODE_AUTO, &need) != FPKV_OK || need == 0) return 8;
    if (ws(&pool, 64, 12, FPKV_DECODE_AUTO, &need) != FPKV_ESHAPE) return 9;
    printf("c client ok: version %d, decode workspace %zu bytes\n", version(), need);
    return 0;
}
"""


def test_c_program_uses_the_library(tmp_path):
    src = tmp_path / "client.c"
    src.write_text(C_SOURCE)
    exe = tmp_path / "client"
    cc = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o",
                         str(exe), "-ldl"], capture_output=True, text=True)
    assert cc.returncode == 0, cc.stderr
    run = subprocess.run([str(exe), _lib.LIB_PATH], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    assert "c client ok" in run.stdout
