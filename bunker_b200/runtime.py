"""Host-side mirror of bunker's runtime surface (src/ttir.ts:223-417) over libbunker_cuda.so.

bunker's callers (src/runner.ts, prototypes/decode.ts, prototypes/decode_graph.ts) use
``cuAlloc / cuHtoD / cuDtoH / cuFree / cuSync / cuLaunch`` and a ``LoadedKernel`` handle.
The same names are kept here; they bind the C ABI declared in include/bunker_cuda.h through
ctypes exactly the way bun:ffi would (device pointers as 64-bit integers, host buffers
borrowed for the call).  There is no CPU fallback: if the shared library is missing or the
process has no sm_100 GPU, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbunker_cuda.so")

# error codes of include/bunker_cuda.h
BK_OK = 0
BK_ERR_ARG = 10001
BK_ERR_STATE = 10002
BK_ERR_TIMEOUT = 10003
BK_ERR_UNSUPPORTED = 10004
BK_ERR_COMM = 10005

BK_PRO_Q8, BK_PRO_BF16, BK_PRO_RMSNORM, BK_PRO_STAGED = 0, 1, 2, 3
BK_Q8_BLOCKS, BK_Q8_STAGED = 0, 1
BK_EPI_F32, BK_EPI_BF16, BK_EPI_ADD_BF16, BK_EPI_SWIGLU = 0, 1, 2, 3
BK_DTYPE_F32, BK_DTYPE_BF16 = 0, 1
BK_GEMV_ORDER_AUTO, BK_GEMV_ORDER_LANES, BK_GEMV_ORDER_TILE = 0, 1, 2

BK_OP_EMBED, BK_OP_RMSNORM, BK_OP_GEMV, BK_OP_SWIGLU, BK_OP_CONV1D, BK_OP_ARGMAX, BK_OP_QUANT_Q8_1 = range(1, 8)
BK_OP_HEADNORM_ROPE, BK_OP_GDN, BK_OP_ATTN, BK_OP_QUANT_Q8_1_BF16 = 8, 9, 10, 11


class BunkerCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[bunker_cuda rc={code}] {message}")
        self.code = code


class bkGemvSeg(C.Structure):
    _fields_ = [("W", C.c_uint64), ("W2", C.c_uint64), ("out", C.c_uint64), ("residual", C.c_uint64),
                ("n_rows", C.c_int32), ("epilogue", C.c_int32), ("ld_out", C.c_int32), ("col_off", C.c_int32)]


class bkGemvArgs(C.Structure):
    _fields_ = [("K", C.c_int32), ("B", C.c_int32), ("n_segs", C.c_int32), ("prologue", C.c_int32),
                ("x", C.c_uint64), ("norm_w", C.c_uint64), ("eps", C.c_float), ("order", C.c_int32),
                ("segs", bkGemvSeg * 4)]


class bkGdnArgs(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("qkv", "z", "a", "b", "conv_w", "conv_state_in", "conv_state_new", "A_log",
                                           "dt_bias", "norm_w", "S_in", "S_new", "out", "o_raw", "conv_out")] + \
               [(n, C.c_int32) for n in ("B", "Hk", "Hv", "apply_conv", "state_is_settled", "out_q8_layout")] + \
               [("out_q8", C.c_uint64), ("n_tokens", C.c_int32), ("reserved", C.c_int32)]


class bkAttnArgs(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("qg", "k", "v", "q_norm_w", "k_norm_w", "cos_t", "sin_t", "k_cache",
                                           "v_cache", "pos", "out", "scratch")] + \
               [(n, C.c_int32) for n in ("B", "Hq", "Hkv", "HD", "rot_half", "max_len", "split_len", "max_pos")] + \
               [("scale", C.c_float), ("fused_norm_rope", C.c_int32), ("gate", C.c_uint64),
                ("cache_is_settled", C.c_int32), ("out_q8_layout", C.c_int32), ("out_q8", C.c_uint64)]


class bkModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "n_layers", "full_attn_interval", "vocab", "gdn_k_heads",
                                          "gdn_v_heads", "attn_q_heads", "attn_kv_heads", "head_dim", "rot_dim",
                                          "intermediate", "max_len", "batch", "tp_rank", "tp_size")] + \
               [("eps", C.c_float), ("rope_theta", C.c_double)]



# name -> (restype, argtypes); the list doubles as the export check used by the CPU tests
_U64, _I32, _F32, _VP = C.c_uint64, C.c_int32, C.c_float, C.c_void_p
_PU64 = C.POINTER(C.c_uint64)
SIGNATURES = {
    "bkInit": (_I32, [_I32]),
    "bkShutdown": (_I32, []),
    "bkLastError": (C.c_char_p, []),
    "bkDeviceInfo": (_I32, [C.POINTER(_I32), C.POINTER(_I32), C.POINTER(_I32), _PU64]),
    "bkAlloc": (_I32, [_U64, _PU64]),
    "bkFree": (_I32, [_U64]),
    "bkHtoD": (_I32, [_U64, _VP, _U64]),
    "bkDtoH": (_I32, [_VP, _U64, _U64]),
    "bkHtoDAsync": (_I32, [_U64, _VP, _U64]),
    "bkDtoHAsync": (_I32, [_VP, _U64, _U64]),
    "bkDtoD": (_I32, [_U64, _U64, _U64]),
    "bkMemset": (_I32, [_U64, _I32, _U64]),
    "bkHostAlloc": (_I32, [_U64, C.POINTER(_VP)]),
    "bkHostFree": (_I32, [_VP]),
    "bkSync": (_I32, []),
    "bkEventCreate": (_I32, [_PU64]),
    "bkEventRecord": (_I32, [_U64]),
    "bkEventSync": (_I32, [_U64]),
    "bkEventElapsedMs": (_I32, [_U64, _U64, C.POINTER(_F32)]),
    "bkEventDestroy": (_I32, [_U64]),
    "bkLaunchCount": (_I32, [_PU64]),
    "bkTraceEnable": (_I32, [_U64, _I32]),
    "bkTraceCtas": (_I32, [_U64, _I32]),
    "bkTraceDisable": (_I32, []),
    "bkStepTraceEnable": (_I32, [_U64, _I32]),
    "bkStepBarrierMode": (_I32, [_I32]),
    "bkSetSpinLimit": (_I32, [_I32]),
    "bkGemvQ4K": (_I32, [C.POINTER(bkGemvArgs)]),
    "bkGemvQ4KSimple": (_I32, [_U64, _I32, _I32, _U64, _I32, _U64]),
    "bkDequantQ4K": (_I32, [_U64, _I32, _I32, _U64]),
    "bkBlockDotsQ4K": (_I32, [_U64, _I32, _I32, _U64, _U64, _U64]),
    "bkQuantizeQ4K": (_I32, [_U64, _I32, C.c_int64, _I32, _U64]),
    "bkQuantQ8_1": (_I32, [_U64, _I32, _I32, _U64]),
    "bkQuantQ8_1Bf16": (_I32, [_U64, _I32, _I32, _U64]),
    "bkEmbedQ4K": (_I32, [_U64, _I32, _U64, _I32, _U64]),
    "bkRmsNorm": (_I32, [_U64, _U64, _I32, _I32, _F32, _U64]),
    "bkRmsNormQuantQ8_1": (_I32, [_U64, _U64, _I32, _I32, _F32, _U64, _I32]),
    "bkStagedBytes": (_U64, [_I32, _I32]),
    "bkReduceRmsNormQuantQ8_1": (_I32, [_U64, _I32, _U64, _U64, C.c_uint32, _U64, _U64, _U64, _I32, _I32, _F32, _U64, _I32]),
    "bkTuneGemvRing": (_I32, [_I32, _I32, _I32]),
    "bkTuneTileMinRows": (_I32, [_I32]),
    "bkSwiglu": (_I32, [_U64, _U64, _I32, _U64]),
    "bkConv1dStep": (_I32, [_U64, _U64, _U64, _I32, _I32, _U64, _U64]),
    "bkGdnStep": (_I32, [C.POINTER(bkGdnArgs)]),
    "bkRopeTables": (_I32, [_I32, _I32, C.c_double, C.POINTER(_F32), C.POINTER(_F32)]),
    "bkHeadNormRope": (_I32, [_U64, _I32, _U64, _U64, _U64, _I32, _U64, _I32, _I32, _I32, _U64]),
    "bkAttnDecode": (_I32, [C.POINTER(bkAttnArgs)]),
    "bkAttnPlan": (_I32, [_I32, _I32, _I32, C.POINTER(_I32), C.POINTER(_I32)]),
    "bkAttnScratchBytes": (_U64, [_I32, _I32, _I32, _I32, _I32]),
    "bkArgmax": (_I32, [_U64, _I32, _I32, _U64, _U64, _U64]),
    "bkArgmaxScratchBytes": (_U64, [_I32]),
    "bkArgmaxStatic": (_I32, [_U64, _I32, _I32, _U64, _U64]),
    "bkSample": (_I32, [_U64, _I32, _I32, _F32, _I32, _F32, _U64, _U64, C.c_uint32, _U64, _U64]),
    "bkLaunch": (_I32, [_I32, _PU64, _I32]),
    "bkCommCreate": (_I32, [_I32, _I32, _U64, _PU64]),
    "bkCommExportHandle": (_I32, [_U64, C.POINTER(C.c_uint8)]),
    "bkCommImportPeers": (_I32, [_U64, C.POINTER(C.c_uint8)]),
    "bkCommDestroy": (_I32, [_U64]),
    "bkCommAllReduceResidual": (_I32, [_U64, _I32, _U64, _I32, _U64, _U64]),
}

_MODEL_SIGS = {
    "bkModelCreate": (C.c_int32, [C.POINTER(bkModelConfig), C.POINTER(C.c_uint64)]),
    "bkModelSetTensor": (C.c_int32, [C.c_uint64, C.c_char_p, C.c_uint64, C.c_uint64]),
    "bkModelSetComm": (C.c_int32, [C.c_uint64, C.c_uint64]),
    "bkModelSetStepMode": (C.c_int32, [C.c_uint64, C.c_int32]),
    "bkModelFinalize": (C.c_int32, [C.c_uint64]),
    "bkDecodeStepEager": (C.c_int32, [C.c_uint64]),
    "bkModelReset": (C.c_int32, [C.c_uint64]),
    "bkDecodeStep": (C.c_int32, [C.c_uint64, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    "bkDecodeRun": (C.c_int32, [C.c_uint64, C.c_int32]),
    "bkModelPrefill": (C.c_int32, [C.c_uint64, C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    "bkDecodeStepProfiled": (C.c_int32, [C.c_uint64, C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_int32]),
    "bkModelTokens": (C.c_int32, [C.c_uint64, C.c_int32, C.c_int32, C.POINTER(C.c_int32)]),
    "bkModelInfo": (C.c_int32, [C.c_uint64, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                C.POINTER(C.c_int64)]),
    "bkModelBuffer": (C.c_int32, [C.c_uint64, C.c_char_p, C.POINTER(C.c_uint64)]),
    "bkModelDestroy": (C.c_int32, [C.c_uint64]),
}
SIGNATURES.update(_MODEL_SIGS)

_lib = None


def load_library() -> C.CDLL:
    """dlopen libbunker_cuda.so and bind every declared symbol.  Raises if the file is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BunkerCudaError(BK_ERR_STATE, f"{LIB_PATH} is missing: build it with `python -m bunker_b200.build` "
                                            "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = an export declared in the header is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(rc: int) -> None:
    if rc != 0:
        msg = load_library().bkLastError()
        raise BunkerCudaError(rc, msg.decode("utf-8", "replace") if msg else "unknown error")


_initialised_device = None


def cu(device: int | None = None) -> C.CDLL:
    """Open the library and create the context (src/ttir.ts:223-261 ``cu()``).  The first call picks the device
    (0 unless given); later calls return the same context and reject a different device."""
    global _initialised_device
    lib = load_library()
    if _initialised_device is None:
        dev = 0 if device is None else int(device)
        _check(lib.bkInit(dev))
        _initialised_device = dev
    elif device is not None and _initialised_device != device:
        raise BunkerCudaError(BK_ERR_STATE, f"context already on device {_initialised_device}")
    return lib


def cuAlloc(nbytes: int) -> int:
    """src/ttir.ts:266 -- returns a device pointer as an int; raises on failure."""
    out = C.c_uint64(0)
    _check(cu().bkAlloc(int(nbytes), C.byref(out)))
    return out.value


def cuFree(dev: int) -> None:
    _check(cu().bkFree(dev))


def _host_ptr(host) -> tuple[int, int]:
    if isinstance(host, np.ndarray):
        if not host.flags["C_CONTIGUOUS"]:
            raise ValueError("host array must be C-contiguous")
        return host.ctypes.data, host.nbytes
    mv = memoryview(host)
    arr = np.frombuffer(mv, dtype=np.uint8)
    return arr.ctypes.data, arr.nbytes


def cuHtoD(dev: int, host, nbytes: int | None = None) -> None:
    """src/ttir.ts:273"""
    p, n = _host_ptr(host)
    _check(cu().bkHtoD(dev, p, n if nbytes is None else int(nbytes)))


def cuDtoH(host, dev: int, nbytes: int | None = None) -> None:
    """src/ttir.ts:278 -- synchronous; the decode loop uses it as its per-token barrier."""
    p, n = _host_ptr(host)
    _check(cu().bkDtoH(p, dev, n if nbytes is None else int(nbytes)))


def cuHtoDAsync(dev: int, host, nbytes: int | None = None) -> None:
    p, n = _host_ptr(host)
    _check(cu().bkHtoDAsync(dev, p, n if nbytes is None else int(nbytes)))


def cuDtoHAsync(host, dev: int, nbytes: int | None = None) -> None:
    p, n = _host_ptr(host)
    _check(cu().bkDtoHAsync(p, dev, n if nbytes is None else int(nbytes)))


def cuMemset(dev: int, value: int, nbytes: int) -> None:
    _check(cu().bkMemset(dev, value, nbytes))


def cuSync() -> int:
    """src/ttir.ts:285 -- returns the rc instead of raising, like the reference."""
    return cu().bkSync()


def host_pinned(nbytes: int, dtype=np.uint8) -> np.ndarray:
    """Pinned host array (for the async copies); freed at process exit."""
    p = C.c_void_p()
    _check(cu().bkHostAlloc(int(nbytes), C.byref(p)))
    buf = (C.c_uint8 * int(nbytes)).from_address(p.value)
    return np.frombuffer(buf, dtype=np.uint8).view(dtype)


@dataclass(frozen=True)
class LoadedKernel:
    """src/ttir.ts:350.  ``fn`` is the library's op id; module/shmem are kept for shape parity."""
    module: int
    fn: int
    shmem: int = 0
    name: str = ""


_OPS = {"embed": BK_OP_EMBED, "rmsnorm": BK_OP_RMSNORM, "gemm": BK_OP_GEMV, "swiglu": BK_OP_SWIGLU,
        "conv1d_decode": BK_OP_CONV1D, "argmax": BK_OP_ARGMAX, "quant_q8_1": BK_OP_QUANT_Q8_1,
        # fused ops: q/k head norm + rope; conv1d + gdn_delta_rule + gated norm; norms + rope + KV append + fa2_attn
        "headnorm_rope": BK_OP_HEADNORM_ROPE, "gdn_delta_rule": BK_OP_GDN, "fa2_attn": BK_OP_ATTN,
        "quant_q8_1_bf16": BK_OP_QUANT_Q8_1_BF16}


def loadOp(name: str) -> LoadedKernel:
    """Stands where ``compileAndLoad(ttir, func, numWarps)`` stood (src/ttir.ts:488): kernels are
    precompiled in the library, so loading is a lookup by the graph's op name (src/model.ts)."""
    if name not in _OPS:
        raise BunkerCudaError(BK_ERR_ARG, f"unknown op {name!r}; known: {sorted(_OPS)}")
    cu()
    return LoadedKernel(module=0, fn=_OPS[name], shmem=0, name=name)


def cuLaunch(k: LoadedKernel, grid: Sequence[int], block: Sequence[int], args: Sequence[int | float]) -> int:
    """src/ttir.ts:321-348.  Each argument occupies one 8-byte slot (ints as i64, device pointers as
    u64, floats as their f32 bits); grid/block are accepted for signature parity and ignored, the
    library sizes its own launches.  Returns the rc and does not raise, like the reference."""
    slots = (C.c_uint64 * max(1, len(args)))()
    for i, a in enumerate(args):
        if isinstance(a, float):
            slots[i] = int(np.float32(a).view(np.uint32))
        else:
            slots[i] = int(a) & 0xFFFFFFFFFFFFFFFF
    return cu().bkLaunch(k.fn, slots, len(args))


def last_error() -> str:
    m = load_library().bkLastError()
    return m.decode("utf-8", "replace") if m else ""


class Event:
    """CUDA event on the library's stream (src/ttir.ts:352-417 profiler)."""

    def __init__(self):
        h = C.c_uint64(0)
        _check(cu().bkEventCreate(C.byref(h)))
        self.handle = h.value

    def record(self) -> "Event":
        _check(cu().bkEventRecord(self.handle))
        return self

    def synchronize(self) -> None:
        _check(cu().bkEventSync(self.handle))

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float(0)
        _check(cu().bkEventElapsedMs(self.handle, stop.handle, C.byref(ms)))
        return ms.value


def launch_count() -> int:
    n = C.c_uint64(0)
    _check(cu().bkLaunchCount(C.byref(n)))
    return n.value


def device_info() -> dict:
    sm, ma, mi, mem = C.c_int32(), C.c_int32(), C.c_int32(), C.c_uint64()
    _check(cu().bkDeviceInfo(C.byref(sm), C.byref(ma), C.byref(mi), C.byref(mem)))
    return {"sm_count": sm.value, "cc": (ma.value, mi.value), "total_mem": mem.value}


class DeviceBuffer:
    """Owning handle for a cuAlloc'd range, with numpy upload/download helpers."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self.ptr = cuAlloc(self.nbytes)

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(max(a.nbytes, 1))
        if a.nbytes:
            cuHtoD(buf.ptr, a)
        return buf

    @classmethod
    def zeros(cls, nbytes: int) -> "DeviceBuffer":
        buf = cls(nbytes)
        cuMemset(buf.ptr, 0, buf.nbytes)
        return buf

    def upload(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        cuHtoD(self.ptr, a)

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes, (out.nbytes, self.nbytes)
        cuDtoH(out, self.ptr)
        return out

    def free(self) -> None:
        if self.ptr:
            cuFree(self.ptr)
            self.ptr = 0
