"""Tokenizer boundary: the gt_init / gt_encode / gt_free surface bunker's driver binds (prototypes/decode.ts:76-87,
shim/gigatoken_wrapper/src/lib.rs:19-93) over libbunker_tok.so, plus decode (ids -> text), which the reference lacks."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbunker_tok.so")
_lib = None


def load_library() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m bunker_b200.build`")
        lib = C.CDLL(LIB_PATH)
        lib.gt_init.restype, lib.gt_init.argtypes = C.c_void_p, [C.c_char_p]
        for name in ("gt_encode", "gt_encode_mt"):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_uint32), C.c_size_t]
        lib.gt_decode.restype, lib.gt_decode.argtypes = C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t, C.c_char_p, C.c_size_t]
        lib.gt_vocab_size.restype, lib.gt_vocab_size.argtypes = C.c_int, [C.c_void_p]
        lib.gt_free.restype, lib.gt_free.argtypes = None, [C.c_void_p]
        _lib = lib
    return _lib


class Tokenizer:
    def __init__(self, tokenizer_json: str):
        self.h = load_library().gt_init(tokenizer_json.encode())
        if not self.h:
            raise RuntimeError(f"gt_init failed for {tokenizer_json}")

    def encode(self, text: str, threads: bool = False) -> np.ndarray:
        """The reference's tokenize() (prototypes/decode.ts:79-87): out buffer of len(bytes) + 64 ids."""
        raw = text.encode("utf-8")
        out = (C.c_uint32 * (len(raw) + 64))()
        fn = load_library().gt_encode_mt if threads else load_library().gt_encode
        n = fn(self.h, raw, len(raw), out, len(out))
        if n < 0:
            raise RuntimeError("gt_encode failed")
        return np.frombuffer(out, np.uint32, count=min(n, len(out))).astype(np.int32)

    def decode(self, ids) -> str:
        ids = np.ascontiguousarray(ids, np.uint32)
        p = ids.ctypes.data_as(C.POINTER(C.c_uint32))
        n = load_library().gt_decode(self.h, p, len(ids), None, 0)
        if n < 0:
            raise RuntimeError("gt_decode failed")
        buf = C.create_string_buffer(max(n, 1))
        load_library().gt_decode(self.h, p, len(ids), buf, n)
        return buf.raw[:n].decode("utf-8", "replace")

    @property
    def vocab_size(self) -> int:
        return load_library().gt_vocab_size(self.h)

    def close(self) -> None:
        if self.h:
            load_library().gt_free(self.h)
            self.h = None
