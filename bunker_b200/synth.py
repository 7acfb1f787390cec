"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

All arrays are numpy; bf16 and f16 values are uint16 bit patterns.  There is no dataset behind any
of this: weights are random-init in the Q4_K layout, activations are Gaussian.
"""
from __future__ import annotations

import numpy as np

SEED_BASE = 0xB0B0


def rng_for(config_id: int, tensor_index: int) -> np.random.Generator:
    return np.random.default_rng(SEED_BASE + config_id * 1000 + tensor_index)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def q4k_weights(rng: np.random.Generator, N: int, K: int, d_std: float = 1e-3) -> np.ndarray:
    """uint8 [N, K/256*144]: f16 d and dmin = |N(0, d_std)|, 6-bit scales/mins uniform 0..63 (every bit
    pattern of the 12 packed bytes is a valid pair set, so the bytes are drawn uniformly), nibbles uniform 0..15."""
    assert K % 256 == 0
    nsb = K // 256
    W = rng.integers(0, 256, size=(N, nsb, 144), dtype=np.uint8)
    dd = np.abs(rng.normal(0.0, d_std, size=(N, nsb, 2))).astype(np.float16)
    W[:, :, 0:4] = dd.view(np.uint8).reshape(N, nsb, 4)
    return W.reshape(N, nsb * 144)


def normal_bf16(rng: np.random.Generator, shape, std: float = 1.0, mean: float = 0.0) -> np.ndarray:
    return f32_to_bf16(rng.normal(mean, std, size=shape).astype(np.float32))


def gemv_case(N: int = 4096, K: int = 4096, B: int = 1, config_id: int = 0):
    """configs[0]: W Q4_K [N,K], x f32 N(0,1) [B,K]."""
    W = q4k_weights(rng_for(config_id, 0), N, K)
    x = rng_for(config_id, 1).normal(0.0, 1.0, size=(B, K)).astype(np.float32)
    return W, x


def gdn_case(B: int, Hk: int = 16, Hv: int = 32, config_id: int = 1):
    """configs[1]: state f32 N(0,0.02); pre-conv qkv bf16 N(0,1); conv state bf16 N(0,1); taps bf16 N(0,0.3);
    a+dt_bias ~ N(0,1), A_log ~ U(-2,0), b ~ N(0,1); z bf16 N(0,1); norm_w f32 1+N(0,0.02)."""
    D = 128
    Cw = 2 * Hk * D + Hv * D
    r = lambda i: rng_for(config_id, i)  # noqa: E731
    return {
        "S": r(0).normal(0, 0.02, size=(B, Hv, D, D)).astype(np.float32),
        "qkv": normal_bf16(r(1), (B, Cw)),
        "conv_state": normal_bf16(r(2), (B, 3, Cw)),
        "conv_w": normal_bf16(r(3), (Cw, 4), 0.3),
        "a": r(4).normal(0, 1, size=(B, Hv)).astype(np.float32),
        "b": r(5).normal(0, 1, size=(B, Hv)).astype(np.float32),
        "A_log": r(6).uniform(-2, 0, size=(Hv,)).astype(np.float32),
        "dt_bias": normal_bf16(r(7), (Hv,), 0.5),
        "z": normal_bf16(r(8), (B, Hv * D)),
        "norm_w": (1.0 + r(9).normal(0, 0.02, size=(D,))).astype(np.float32),
        "Hk": Hk, "Hv": Hv, "B": B,
    }


def attn_case(B: int, L: int, Hq: int = 16, Hkv: int = 2, HD: int = 256, max_len: int | None = None,
              config_id: int = 2):
    """configs[2]: q_proj output (q|gate per head), k, v projections bf16 N(0,1); cache rows 0..L-2 hold bf16
    N(0,1) keys/values; pos = L-1 for every sequence; norm weights bf16 N(0,0.02)."""
    max_len = max_len or L
    r = lambda i: rng_for(config_id, i)  # noqa: E731
    Kc = np.zeros((B, Hkv, max_len, HD), np.uint16)
    Vc = np.zeros((B, Hkv, max_len, HD), np.uint16)
    Kc[:, :, : L - 1] = normal_bf16(r(0), (B, Hkv, L - 1, HD))
    Vc[:, :, : L - 1] = normal_bf16(r(1), (B, Hkv, L - 1, HD))
    return {
        "qg": normal_bf16(r(2), (B, Hq * 2 * HD)),
        "k": normal_bf16(r(3), (B, Hkv * HD)),
        "v": normal_bf16(r(4), (B, Hkv * HD)),
        "q_norm_w": normal_bf16(r(5), (HD,), 0.02),
        "k_norm_w": normal_bf16(r(6), (HD,), 0.02),
        "k_cache": Kc, "v_cache": Vc,
        "pos": np.full((B,), L - 1, np.int32),
        "B": B, "Hq": Hq, "Hkv": Hkv, "HD": HD, "max_len": max_len,
    }
