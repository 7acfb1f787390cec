"""ctypes/numpy front end of the CPU oracle (liboracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped package never imports this module.

bf16 and f16 values travel as numpy uint16 arrays (bit patterns).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile liboracle.so with gcc if it is missing or older than its source."""
    src = os.path.join(_HERE, "bunker_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_q8half_to_f32.restype = C.c_float
        _lib.orc_q8half_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16_trunc.restype = C.c_uint16
        _lib.orc_f32_to_f16_trunc.argtypes = [C.c_float]
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        for name in ("orc_expf", "orc_logf", "orc_sigmoidf", "orc_softplusf"):
            getattr(_lib, name).restype = C.c_float
            getattr(_lib, name).argtypes = [C.c_float]
    return _lib


def set_threads(n: int = 0) -> int:
    """Set the OpenMP thread count of the oracle's loops (n <= 0: leave it) and return the count in effect."""
    fn = lib().orc_set_threads
    fn.restype = C.c_int
    fn.argtypes = [C.c_int]
    return int(fn(int(n)))


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# -- formats -----------------------------------------------------------------

def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (vectorised twin of orc_f32_to_bf16)."""
    u = _c(x, np.float32).view(np.uint32)
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    r[(u & 0x7FFFFFFF) > 0x7F800000] = 0x7FFF
    return r


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (_c(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def expf(x: float) -> float:
    return lib().orc_expf(C.c_float(x))


def logf(x: float) -> float:
    return lib().orc_logf(C.c_float(x))


def sigmoidf(x: float) -> float:
    return lib().orc_sigmoidf(C.c_float(x))


def softplusf(x: float) -> float:
    return lib().orc_softplusf(C.c_float(x))


# -- Q4_K ----------------------------------------------------------------------

def q4k_row_bytes(K: int) -> int:
    assert K % 256 == 0
    return K // 256 * 144


def q4k_scales(sb: np.ndarray):
    sb = _c(sb, np.uint8)
    sc = np.zeros(8, np.uint8)
    mn = np.zeros(8, np.uint8)
    lib().orc_q4k_scales(_p(sb), _p(sc), _p(mn))
    return sc, mn


def q4k_dequant(W: np.ndarray, N: int, K: int) -> np.ndarray:
    W = _c(W, np.uint8).reshape(N, q4k_row_bytes(K))
    out = np.empty((N, K), np.float32)
    for n in range(N):
        lib().orc_q4k_dequant_row(_p(W[n]), K, _p(out[n]))
    return out


def q4k_quantize(x: np.ndarray) -> np.ndarray:
    """f32 [N, K] -> Q4_K rows uint8 [N, K/256*144] (the loader's quantiser; see orc_q4k_quantize_row)."""
    x = _c(x, np.float32)
    N, K = x.shape
    assert K % 256 == 0
    out = np.empty((N, q4k_row_bytes(K)), np.uint8)
    for n in range(N):
        lib().orc_q4k_quantize_row(_p(x[n]), K, _p(out[n]))
    return out


def embed_q4k(table: np.ndarray, H: int, ids) -> np.ndarray:
    ids = _c(ids, np.int32)
    x = np.empty((len(ids), H), np.uint16)
    lib().orc_embed_q4k(_p(_c(table, np.uint8)), H, _p(ids), len(ids), _p(x))
    return x


# -- Q8_1 ----------------------------------------------------------------------

def q8_1_quantize(x: np.ndarray) -> np.ndarray:
    """f32 [B, K] (or [K]) -> uint8 [B, K/32, 36]."""
    x = _c(x, np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    B, K = x2.shape
    assert K % 32 == 0
    out = np.empty((B, K // 32, 36), np.uint8)
    for b in range(B):
        lib().orc_q8_1_quantize(_p(x2[b]), K, _p(out[b]))
    return out


def q8_1_quantize_bf16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.uint16)
    x2 = x.reshape(-1, x.shape[-1])
    B, K = x2.shape
    out = np.empty((B, K // 32, 36), np.uint8)
    lib().orc_q8_1_quantize_bf16(_p(x2), K, B, _p(out))
    return out


def q8_1_dequant(xq: np.ndarray) -> np.ndarray:
    """uint8 [B, nb, 36] -> f32 [B, nb*32] (flush-denormal half decode)."""
    xq = _c(xq, np.uint8)
    B, nb, _ = xq.shape
    q = xq[:, :, :32].view(np.int8).astype(np.float32)
    dh = xq[:, :, 32].astype(np.uint16) | (xq[:, :, 33].astype(np.uint16) << 8)
    d = np.array([lib().orc_q8half_to_f32(int(v)) for v in dh.ravel()], np.float32).reshape(B, nb, 1)
    return (q * d).reshape(B, nb * 32)


def q8_1_scales(xq: np.ndarray) -> np.ndarray:
    """uint8 [B, nb, 36] -> the block scales f32 [B, nb] as the GEMV reads them (flush-denormal half decode)."""
    xq = _c(xq, np.uint8)
    B, nb, _ = xq.shape
    dh = xq[:, :, 32].astype(np.uint16) | (xq[:, :, 33].astype(np.uint16) << 8)
    return np.array([lib().orc_q8half_to_f32(int(v)) for v in dh.ravel()], np.float32).reshape(B, nb)


def block_dots(wrow: np.ndarray, xq: np.ndarray, K: int):
    isum = np.empty(K // 32, np.int32)
    qsum = np.empty(K // 32, np.int32)
    lib().orc_block_dots(_p(_c(wrow, np.uint8)), _p(_c(xq, np.uint8)), K, _p(isum), _p(qsum))
    return isum, qsum


# -- GEMV ------------------------------------------------------------------------

def gemv_q4k_q8(W: np.ndarray, N: int, K: int, xq: np.ndarray) -> np.ndarray:
    """Canonical-order f32 [B, N]."""
    xq = _c(xq, np.uint8).reshape(-1, K // 32, 36)
    B = xq.shape[0]
    y = np.empty((B, N), np.float32)
    lib().orc_gemv_q4k_q8(_p(_c(W, np.uint8)), N, K, _p(xq), B, _p(y))
    return y


def gemv_q4k_q8_tile(W: np.ndarray, N: int, K: int, xq: np.ndarray) -> np.ndarray:
    """f32 [B, N] in the order of the dense tile path (batch >= 16): one chain per (row, column), sub-blocks then
    superblocks ascending."""
    xq = _c(xq, np.uint8).reshape(-1, K // 32, 36)
    B = xq.shape[0]
    y = np.empty((B, N), np.float32)
    lib().orc_gemv_q4k_q8_tile(_p(_c(W, np.uint8)), N, K, _p(xq), B, _p(y))
    return y


def gemv_q4k_q8_plain(W: np.ndarray, N: int, K: int, xq: np.ndarray) -> np.ndarray:
    xq = _c(xq, np.uint8).reshape(-1, K // 32, 36)
    B = xq.shape[0]
    y = np.empty((B, N), np.float64)
    lib().orc_gemv_q4k_q8_plain(_p(_c(W, np.uint8)), N, K, _p(xq), B, _p(y))
    return y


def sum_ranks(parts: np.ndarray) -> np.ndarray:
    parts = _c(parts, np.float32)
    R = parts.shape[0]
    n = parts[0].size
    out = np.empty(parts.shape[1:], np.float32)
    lib().orc_sum_ranks(_p(parts), R, n, _p(out))
    return out


def epilogue_cast(y: np.ndarray) -> np.ndarray:
    y = _c(y, np.float32)
    out = np.empty(y.shape, np.uint16)
    lib().orc_epilogue_cast(_p(y), y.size, _p(out))
    return out


def epilogue_add(y: np.ndarray, res: np.ndarray) -> np.ndarray:
    y = _c(y, np.float32)
    res = _c(res, np.uint16)
    assert res.shape == y.shape
    out = np.empty(y.shape, np.uint16)
    lib().orc_epilogue_add(_p(y), _p(res), y.size, _p(out))
    return out


def swiglu(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    g = _c(g, np.float32)
    u = _c(u, np.float32)
    out = np.empty(g.shape, np.uint16)
    lib().orc_swiglu(_p(g), _p(u), g.size, _p(out))
    return out


# -- norms / conv / gdn / rope / attention / argmax -------------------------------

def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    x = _c(x, np.uint16)
    B, H = x.reshape(-1, x.shape[-1]).shape
    y = np.empty((B, H), np.uint16)
    lib().orc_rmsnorm(_p(x), _p(_c(w, np.uint16)), H, B, C.c_float(eps), _p(y))
    return y


def rmsnorm_plain(x: np.ndarray, w: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    x = _c(x, np.uint16)
    B, H = x.reshape(-1, x.shape[-1]).shape
    y = np.empty((B, H), np.float64)
    lib().orc_rmsnorm_plain(_p(x), _p(_c(w, np.uint16)), H, B, C.c_double(eps), _p(y))
    return y


def conv1d_step(x: np.ndarray, state: np.ndarray, w: np.ndarray):
    """x [B,C] bf16, state [B,3,C] bf16, w [C,4] bf16 -> (out [B,C], new state)."""
    x = _c(x, np.uint16)
    B, Cc = x.shape
    state = _c(state, np.uint16).reshape(B, 3, Cc)
    out = np.empty((B, Cc), np.uint16)
    sn = np.empty((B, 3, Cc), np.uint16)
    lib().orc_conv1d_step(_p(x), _p(state), _p(_c(w, np.uint16)), Cc, B, _p(out), _p(sn))
    return out, sn


def gdn_step(conv_out, a, b, A_log, dt_bias, S, Hk: int, Hv: int):
    """-> (S_new f32 [B,Hv,128,128], o_raw f32 [B,Hv,128])."""
    conv_out = _c(conv_out, np.uint16)
    B = conv_out.shape[0]
    S = _c(S, np.float32).reshape(B, Hv, 128, 128)
    Sn = np.empty_like(S)
    o = np.empty((B, Hv, 128), np.float32)
    lib().orc_gdn_step(_p(conv_out), _p(_c(a, np.float32)), _p(_c(b, np.float32)), _p(_c(A_log, np.float32)),
                       _p(_c(dt_bias, np.uint16)), _p(S), B, Hk, Hv, _p(Sn), _p(o))
    return Sn, o


def gdn_gate_norm(o_raw, z, norm_w, Hv: int) -> np.ndarray:
    o_raw = _c(o_raw, np.float32)
    B = o_raw.reshape(-1, Hv * 128).shape[0]
    out = np.empty((B, Hv * 128), np.uint16)
    lib().orc_gdn_gate_norm(_p(o_raw), _p(_c(z, np.uint16)), _p(_c(norm_w, np.float32)), B, Hv, _p(out))
    return out


def gdn_step_plain(q, k, v, decay: float, beta: float, S):
    S = _c(S, np.float32)
    Sn = np.empty((128, 128), np.float64)
    o = np.empty(128, np.float64)
    lib().orc_gdn_step_plain(_p(_c(q, np.float32)), _p(_c(k, np.float32)), _p(_c(v, np.float32)),
                             C.c_double(decay), C.c_double(beta), _p(S), _p(Sn), _p(o))
    return Sn, o


def rope_tables(max_len: int, rot_dim: int = 64, theta: float = 1e7):
    half = rot_dim // 2
    c = np.empty((max_len, half), np.float32)
    s = np.empty((max_len, half), np.float32)
    lib().orc_rope_tables(max_len, rot_dim, C.c_double(theta), _p(c), _p(s))
    return c, s


def headnorm_rope(x, in_stride: int, w, cos_t, sin_t, pos, nheads: int, HD: int) -> np.ndarray:
    """x bf16 [B, nheads*in_stride] -> bf16 [B, nheads*HD] normed + rotated."""
    x = _c(x, np.uint16)
    B = x.shape[0]
    pos = _c(pos, np.int32)
    cos_t = _c(cos_t, np.float32)
    out = np.empty((B, nheads * HD), np.uint16)
    lib().orc_headnorm_rope(_p(x), in_stride, _p(_c(w, np.uint16)), _p(cos_t), _p(_c(sin_t, np.float32)),
                            cos_t.shape[1], _p(pos), B, nheads, HD, _p(out))
    return out


def attn_decode(q, gate, gate_stride: int, Kc, Vc, pos, Hq: int, Hkv: int, HD: int, split_len: int, W: int,
                scale: float) -> np.ndarray:
    """q bf16 [B,Hq*HD]; gate bf16 view with per-head stride; caches bf16 [B,Hkv,max_len,HD]."""
    q = _c(q, np.uint16)
    B = q.shape[0]
    Kc = _c(Kc, np.uint16)
    Vc = _c(Vc, np.uint16)
    max_len = Kc.shape[2]
    out = np.empty((B, Hq * HD), np.uint16)
    lib().orc_attn_decode(_p(q), _p(_c(gate, np.uint16)), gate_stride, _p(Kc), _p(Vc), _p(_c(pos, np.int32)), B, Hq,
                          Hkv, HD, max_len, split_len, W, C.c_float(scale), _p(out))
    return out


def attn_decode_plain(q, Kc, Vc, n: int, HD: int, scale: float) -> np.ndarray:
    out = np.empty(HD, np.float64)
    lib().orc_attn_decode_plain(_p(_c(q, np.uint16)), _p(_c(Kc, np.uint16)), _p(_c(Vc, np.uint16)), n, HD,
                                C.c_double(scale), _p(out))
    return out


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, step=None, step_add: int = 0):
    """-> (idx int32 [B], val f32 [B]); step: int32 [B] per-sequence counters or None."""
    logits = _c(logits, np.float32)
    B, V = logits.reshape(-1, logits.shape[-1]).shape
    idx, val = np.empty(B, np.int32), np.empty(B, np.float32)
    st = None if step is None else _c(step, np.int32)
    lib().orc_sample(_p(logits), V, B, C.c_float(temperature), top_k, C.c_float(top_p), C.c_uint64(seed),
                     None if st is None else _p(st), C.c_uint32(step_add), _p(idx), _p(val))
    return idx, val


def argmax(logits: np.ndarray):
    logits = _c(logits, np.float32)
    B, V = logits.reshape(-1, logits.shape[-1]).shape
    idx = np.empty(B, np.int32)
    val = np.empty(B, np.float32)
    lib().orc_argmax(_p(logits), V, B, _p(idx), _p(val))
    return idx, val
