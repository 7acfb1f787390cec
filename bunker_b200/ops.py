"""The decode-op interface of bunker's graph (src/model.ts op kinds: embed, rmsnorm, gemm, conv1d_decode,
gdn_delta_rule, qnorm/rope/knorm/ropek, fa2_attn, swiglu, argmax) bound to the C ABI.

Every function takes device pointers (ints, as returned by ``cuAlloc``) and enqueues on the library
stream without waiting, like the reference's ``cuLaunch``.  Failures raise ``BunkerCudaError``.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import runtime as R
from .runtime import (BK_EPI_ADD_BF16, BK_EPI_BF16, BK_EPI_F32, BK_EPI_SWIGLU, BK_PRO_BF16, BK_PRO_Q8,  # noqa: F401
                      BK_PRO_RMSNORM, _check, cu)


def gemv_seg(W: int, n_rows: int, out: int, epilogue: int = BK_EPI_F32, *, ld_out: int | None = None,
             col_off: int = 0, residual: int = 0, W2: int = 0) -> R.bkGemvSeg:
    return R.bkGemvSeg(W=W, W2=W2, out=out, residual=residual, n_rows=n_rows, epilogue=epilogue,
                       ld_out=n_rows + col_off if ld_out is None else ld_out, col_off=col_off)


def gemv(x: int, K: int, B: int, segs: Sequence[R.bkGemvSeg], prologue: int = BK_PRO_Q8, norm_w: int = 0,
         eps: float = 1e-6, order: int = 0) -> None:
    """Q4_K x Q8_1 GEMV with fused prologue/epilogues (buildMM / buildGateSwiglu, prototypes/decode.ts:101-186).
    order: BK_GEMV_ORDER_AUTO (0; the dense tcgen05 tile kernel from 16 columns of Q8_1 blocks and 4096 launch rows on),
    BK_GEMV_ORDER_LANES (1; always the batch <= 8 kernels' accumulation order) or BK_GEMV_ORDER_TILE (2; the tile kernel
    from 16 columns on whatever the row count)."""
    a = R.bkGemvArgs()
    a.K, a.B, a.n_segs, a.prologue, a.order = K, B, len(segs), prologue, order
    a.x, a.norm_w, a.eps = x, norm_w, eps
    for i, s in enumerate(segs):
        a.segs[i] = s
    _check(cu().bkGemvQ4K(C.byref(a)))


def gemv_simple(W: int, N: int, K: int, xq: int, B: int, y: int) -> None:
    _check(cu().bkGemvQ4KSimple(W, N, K, xq, B, y))


def dequant_q4k(W: int, N: int, K: int, out: int) -> None:
    _check(cu().bkDequantQ4K(W, N, K, out))


def block_dots(W: int, N: int, K: int, xq: int, isum: int, qsum: int) -> None:
    _check(cu().bkBlockDotsQ4K(W, N, K, xq, isum, qsum))


def quantize_q4k(x: int, n_rows: int, K: int, out: int, bf16: bool = False) -> None:
    """Weight rows f32 / bf16 [n_rows][K] -> Q4_K rows (the loader's quantiser)."""
    _check(cu().bkQuantizeQ4K(x, R.BK_DTYPE_BF16 if bf16 else R.BK_DTYPE_F32, n_rows, K, out))


def quant_q8_1(x: int, K: int, B: int, out: int, bf16: bool = False) -> None:
    _check((cu().bkQuantQ8_1Bf16 if bf16 else cu().bkQuantQ8_1)(x, K, B, out))


def embed(table: int, H: int, ids: int, B: int, x_out: int) -> None:
    _check(cu().bkEmbedQ4K(table, H, ids, B, x_out))


def rmsnorm(x: int, w: int, H: int, B: int, y: int, eps: float = 1e-6) -> None:
    _check(cu().bkRmsNorm(x, w, H, B, eps, y))


def rmsnorm_quant_q8_1(x: int, w: int, K: int, B: int, out: int, eps: float = 1e-6, layout: int = R.BK_Q8_BLOCKS) -> None:
    """RMSNorm (w != 0) and Q8_1 quantisation of bf16 rows in one launch; w = 0 quantises the rows as they are.
    layout BK_Q8_STAGED writes the staged image of the batch-3..8 GEMV (staged_bytes(K, B) bytes)."""
    _check(cu().bkRmsNormQuantQ8_1(x, w, K, B, eps, out, layout))


def staged_bytes(K: int, B: int) -> int:
    return int(R.load_library().bkStagedBytes(K, B))


def staged_to_blocks(img: np.ndarray, K: int, B: int):
    """Unpack a staged image (uint8) into (quants int8 [B][K], d8 f32 [B][K/32] with the 1/16 of odd blocks undone,
    s8 f32 [B][K/32]) -- the three things the GEMV reads from Q8_1 blocks."""
    rw = K // 4 + 8
    words = img[:B * rw * 4].view(np.uint32).reshape(B, rw)[:, :K // 4].reshape(B, K // 32, 8)
    pos = np.array([(w & 3) * 2 + (w >> 2) for w in range(8)])
    q = np.ascontiguousarray(words[:, :, pos]).view(np.int8).reshape(B, K)
    sc = img[B * rw * 4:B * rw * 4 + (K // 64) * 8 * 16].view(np.float32).reshape(K // 64, 8, 4)[:, :B]
    d8 = np.stack([sc[:, :, 0], sc[:, :, 1] * np.float32(16.0)], axis=-1)    # [u][b][2]
    s8 = np.stack([sc[:, :, 2], sc[:, :, 3]], axis=-1)
    return q, d8.transpose(1, 0, 2).reshape(B, K // 32), s8.transpose(1, 0, 2).reshape(B, K // 32)


def swiglu(g: int, u: int, n: int, out: int) -> None:
    _check(cu().bkSwiglu(g, u, n, out))


def conv1d_step(x: int, state_in: int, w: int, Cc: int, B: int, out: int, state_new: int) -> None:
    _check(cu().bkConv1dStep(x, state_in, w, Cc, B, out, state_new))


def gdn_step(**kw) -> None:
    """Fused conv1d + gated DeltaNet step; keyword names are the fields of bkGdnArgs."""
    a = R.bkGdnArgs()
    for k, v in kw.items():
        setattr(a, k, v)
    _check(cu().bkGdnStep(C.byref(a)))


def rope_tables(max_len: int, rot_dim: int = 64, theta: float = 1e7):
    half = rot_dim // 2
    c = np.empty((max_len, half), np.float32)
    s = np.empty((max_len, half), np.float32)
    _check(R.load_library().bkRopeTables(max_len, rot_dim, theta, c.ctypes.data_as(C.POINTER(C.c_float)),
                                         s.ctypes.data_as(C.POINTER(C.c_float))))
    return c, s


def headnorm_rope(x: int, in_stride: int, w: int, cos_t: int, sin_t: int, rot_half: int, pos: int, B: int,
                  nheads: int, HD: int, out: int) -> None:
    _check(cu().bkHeadNormRope(x, in_stride, w, cos_t, sin_t, rot_half, pos, B, nheads, HD, out))


def attn_plan(n_rows: int, B: int, Hkv: int) -> tuple[int, int]:
    sl, w = C.c_int32(), C.c_int32()
    _check(cu().bkAttnPlan(n_rows, B, Hkv, C.byref(sl), C.byref(w)))
    return sl.value, w.value


def attn_scratch_bytes(B: int, Hq: int, HD: int, max_len: int, split_len: int) -> int:
    return int(R.load_library().bkAttnScratchBytes(B, Hq, HD, max_len, split_len))


def attn_decode(**kw) -> None:
    """Split-KV decode attention; keyword names are the fields of bkAttnArgs."""
    a = R.bkAttnArgs()
    for k, v in kw.items():
        setattr(a, k, v)
    _check(cu().bkAttnDecode(C.byref(a)))


def argmax_scratch_bytes(B: int) -> int:
    return int(R.load_library().bkArgmaxScratchBytes(B))


def argmax(logits: int, V: int, B: int, idx: int, val: int, scratch: int) -> None:
    """scratch must have been zeroed once before its first use."""
    _check(cu().bkArgmax(logits, V, B, idx, val, scratch))


def argmax_static(logits: int, V: int, B: int, idx: int, val: int) -> None:
    """bkArgmax for callers that cannot allocate: the scratch is built into the library (B <= 64).
    Calls share that scratch, so do not let two of them overlap on the GPU."""
    _check(cu().bkArgmaxStatic(logits, V, B, idx, val))


def sample(logits: int, V: int, B: int, idx: int, val: int = 0, temperature: float = 1.0, top_k: int = 40, top_p: float = 1.0,
           seed: int = 0, step_dev: int = 0, step_add: int = 0) -> None:
    """Temperature / top-k / top-p sampling over f32 logits [B][V] (deterministic; see bkSample)."""
    _check(cu().bkSample(logits, V, B, temperature, top_k, top_p, seed, step_dev, step_add, idx, val))
