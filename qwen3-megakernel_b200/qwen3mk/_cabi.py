"""ctypes binding of libq3mk.so (include/q3mk.h).  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libq3mk.so"

OK, ERR_INVALID, ERR_CUDA, ERR_NOT_RESIDENT, ERR_DEVICE_WAIT, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5
F_APPEND_KV, F_PATH_AUTO, F_PATH_LAYERED, F_PATH_PERSIST, F_PATH_FUSED, F_GRAPH = 0x1, 0x0, 0x10, 0x20, 0x30, 0x100

# every symbol include/q3mk.h declares
SYMBOLS = ("q3_create", "q3_destroy", "q3_set_weights", "q3_invalidate_weights", "q3_set_rope", "q3_tp_export", "q3_tp_attach", "q3_decode", "q3_decode_noalloc", "q3_noalloc_status", "q3_linear_tc", "q3_prefill", "q3_sample", "q3_status",
           "q3_set_trace", "q3_launch_count", "q3_grid_info", "q3_scratch", "q3_last_error", "q3_version")

WEIGHT_FIELDS = ("ln1", "wq", "wk", "wv", "qn", "kn", "wo", "ln2", "wg", "wu", "wd", "fnorm", "embed")


class Config(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("vocab", C.c_int32), ("max_batch", C.c_int32), ("max_tokens", C.c_int32),
                ("grid_limit", C.c_int32), ("wait_limit_us", C.c_int32)]


class Weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in WEIGHT_FIELDS]


class DecodeArgs(C.Structure):
    _fields_ = [("batch", C.c_int32), ("max_len", C.c_int32), ("flags", C.c_uint32), ("reserved", C.c_uint32),
                ("token", C.c_void_p), ("seq_k", C.c_void_p), ("seq_v", C.c_void_p), ("seq_layer_stride", C.c_void_p),
                ("seq_len", C.c_void_p), ("logits", C.c_void_p), ("next_token", C.c_void_p),
                ("k_write", C.c_void_p), ("v_write", C.c_void_p)]


class PrefillArgs(C.Structure):
    _fields_ = [("n_tokens", C.c_int32), ("cache_capacity", C.c_int32), ("ids", C.c_void_p), ("kcache", C.c_void_p),
                ("vcache", C.c_void_p), ("last_logits", C.c_void_p), ("next_token", C.c_void_p)]


_lib = None


def load() -> C.CDLL:
    """Load the library once.  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python qwen3-megakernel_b200/build.py` "
                           "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(str(LIB_PATH))
    lib.q3_create.argtypes = [C.c_int, C.POINTER(Config), C.POINTER(C.c_void_p)]
    lib.q3_create.restype = C.c_int
    lib.q3_destroy.argtypes = [C.c_void_p]
    lib.q3_destroy.restype = None
    lib.q3_set_weights.argtypes = [C.c_void_p, C.POINTER(Weights)]
    lib.q3_set_weights.restype = C.c_int
    lib.q3_invalidate_weights.argtypes = [C.c_void_p]
    lib.q3_invalidate_weights.restype = C.c_int
    lib.q3_set_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_int32]
    lib.q3_set_rope.restype = C.c_int
    lib.q3_tp_export.argtypes = [C.c_void_p, C.c_void_p]
    lib.q3_tp_export.restype = C.c_int
    lib.q3_tp_attach.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.q3_tp_attach.restype = C.c_int
    lib.q3_decode.argtypes = [C.c_void_p, C.POINTER(DecodeArgs), C.c_void_p]
    lib.q3_decode.restype = C.c_int
    lib.q3_decode_noalloc.argtypes = [C.POINTER(Weights), C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.POINTER(DecodeArgs), C.c_void_p]
    lib.q3_decode_noalloc.restype = C.c_int
    lib.q3_noalloc_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_int32]
    lib.q3_noalloc_status.restype = C.c_int
    lib.q3_linear_tc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                 C.c_void_p, C.c_int64, C.c_void_p]
    lib.q3_linear_tc.restype = C.c_int
    lib.q3_prefill.argtypes = [C.c_void_p, C.POINTER(PrefillArgs), C.c_void_p]
    lib.q3_prefill.restype = C.c_int
    lib.q3_sample.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.q3_sample.restype = C.c_int
    lib.q3_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32), C.c_int32]
    lib.q3_status.restype = C.c_int
    lib.q3_set_trace.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
    lib.q3_set_trace.restype = C.c_int
    lib.q3_launch_count.argtypes = [C.c_void_p]
    lib.q3_launch_count.restype = C.c_int64
    lib.q3_grid_info.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.q3_grid_info.restype = C.c_int
    lib.q3_scratch.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int64)]
    lib.q3_scratch.restype = C.c_int
    lib.q3_last_error.argtypes = [C.c_void_p]
    lib.q3_last_error.restype = C.c_char_p
    lib.q3_version.argtypes = []
    lib.q3_version.restype = C.c_char_p
    _lib = lib
    return lib


def check(lib, handle, rc: int, what: str) -> None:
    """Turn a negative return code into the exception type the reference's API raises."""
    if rc == OK:
        return
    msg = lib.q3_last_error(handle).decode(errors="replace")
    if rc == ERR_INVALID:
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg} (code {rc})")
