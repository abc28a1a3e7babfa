"""ctypes binding of libfpkv.so (the C ABI declared in include/fpkv.h).

There is no fallback: if the shared library has not been built the import
fails with instructions, and every compute entry point needs CUDA tensors.
"""

from __future__ import annotations

import ctypes
import os

from ._srchash import source_hash

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfpkv.so")

FPKV_F32, FPKV_BF16, FPKV_F16 = 0, 1, 2
FPKV_I32, FPKV_I64 = 0, 1
DECODE_AUTO, DECODE_PORTABLE, DECODE_TMA = 0, 1, 2
DECODE_AFTER_APPEND = 4
PREFILL_AUTO, PREFILL_PORTABLE, PREFILL_TC = 0, 1, 2
STATIC_SCRATCH_BYTES = 4 << 20
ESTATIC = -8
STATUS_BAD_SLOT, STATUS_BAD_POS, STATUS_BAD_PAGE, STATUS_TIMEOUT, STATUS_OPEN_SPAN = 1, 2, 4, 8, 16

# every symbol include/fpkv.h declares
EXPORTS = ("fpkv_version", "fpkv_build_id", "fpkv_strerror", "fpkv_alloc_step", "fpkv_append_decode", "fpkv_append_packed",
           "fpkv_pre_append", "fpkv_gather", "fpkv_decode_workspace_bytes", "fpkv_decode_attn", "fpkv_decode_attn_static",
           "fpkv_prefill_attn")
OP_ALLOCATE, OP_RESERVE, OP_ERASE, OP_MAP, OP_CLEAR = 0, 1, 2, 3, 4


class FpkvPool(ctypes.Structure):
    """struct fpkv_pool"""
    _fields_ = [("data", ctypes.c_void_p), ("page_table", ctypes.c_void_p),
                ("physical_to_logical", ctypes.c_void_p),
                ("num_layers", ctypes.c_int32), ("n_heads", ctypes.c_int32), ("n_pages", ctypes.c_int32),
                ("page_size", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("max_batch_size", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("split_q_heads", ctypes.c_int32)]


class FpkvAllocState(ctypes.Structure):
    """struct fpkv_alloc_state"""
    _fields_ = [("free_pages", ctypes.c_void_p), ("free_slots", ctypes.c_void_p), ("counts", ctypes.c_void_p)]


class FpkvEpilogue(ctypes.Structure):
    """struct fpkv_epilogue"""
    _fields_ = [("sinks", ctypes.c_void_p), ("sinks_dtype", ctypes.c_int32), ("token_major", ctypes.c_int32)]


class FpkvError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        super().__init__(f"{where}: {strerror(code)} (fpkv code {code})")


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python falcon-perception_b200/build.py` "
            "(nvcc, sm_100a). fpkv has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    try:
        lib.fpkv_build_id.restype = ctypes.c_char_p
        lib.fpkv_build_id.argtypes = []
        built = lib.fpkv_build_id().decode()
    except AttributeError:
        built = "(a build without an id)"
    want = source_hash()
    if want is not None and built != want:           # a stale binary must not pass for the sources in the tree
        raise ImportError(
            f"{LIB_PATH} was built from other sources than the tree holds (library {built}, tree {want}): "
            "rebuild it with `python falcon-perception_b200/build.py`.")
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float
    pool = ctypes.POINTER(FpkvPool)
    lib.fpkv_version.restype = ctypes.c_int
    lib.fpkv_version.argtypes = []
    lib.fpkv_strerror.restype = ctypes.c_char_p
    lib.fpkv_strerror.argtypes = [ctypes.c_int]
    lib.fpkv_append_decode.restype = ctypes.c_int
    lib.fpkv_append_decode.argtypes = [pool, i32, vp, vp, i32, vp, i64, i64, vp, i64, i64, i32, vp, vp]
    lib.fpkv_append_packed.restype = ctypes.c_int
    lib.fpkv_append_packed.argtypes = [pool, i32, vp, vp, i32, vp, i64, i64, vp, i64, i64, i32, vp, vp]
    lib.fpkv_pre_append.restype = ctypes.c_int
    lib.fpkv_pre_append.argtypes = [pool, i32, vp, i64, i32, i32, vp, vp, vp, vp, i32, i32, i32, vp, i64, i64,
                                    ctypes.c_float, vp, vp]
    lib.fpkv_gather.restype = ctypes.c_int
    lib.fpkv_gather.argtypes = [pool, i32, i32, i32, vp, vp, vp, vp]
    lib.fpkv_decode_workspace_bytes.restype = ctypes.c_int
    lib.fpkv_decode_workspace_bytes.argtypes = [pool, i32, i32, i32, ctypes.POINTER(ctypes.c_size_t)]
    lib.fpkv_decode_attn.restype = ctypes.c_int
    epi = ctypes.POINTER(FpkvEpilogue)
    lib.fpkv_decode_attn.argtypes = [pool, i32, vp, vp, vp, i64, i64, vp, vp, i32, i32, i32, f32, vp,
                                     ctypes.c_size_t, i32, epi, vp, vp]
    lib.fpkv_alloc_step.restype = ctypes.c_int
    lib.fpkv_alloc_step.argtypes = [pool, ctypes.POINTER(FpkvAllocState), vp, i32, vp, vp]
    lib.fpkv_prefill_attn.restype = ctypes.c_int
    lib.fpkv_prefill_attn.argtypes = [pool, i32, vp, vp, vp, i64, i64, vp, vp, i32, i32, f32, i32, epi, vp, vp]
    lib.fpkv_decode_attn_static.restype = ctypes.c_int
    lib.fpkv_decode_attn_static.argtypes = [pool, i32, vp, vp, vp, i64, i64, vp, vp, i32, i32, i32, f32, vp, vp]
    return lib


lib = _load()


def build_id() -> str:
    """Hash of the sources the loaded library was compiled from."""
    return lib.fpkv_build_id().decode()


def strerror(code: int) -> str:
    return lib.fpkv_strerror(int(code)).decode()


def check(code: int, where: str) -> None:
    if code != 0:
        raise FpkvError(code, where)
