"""CPU-only: the oracle against the known-answer vectors of tests/golden/kat.npz (derived without the oracle),
and the canonical-order functions against the plain restatements of the reference loops."""
import math
import os

import numpy as np
import pytest

from bunker_b200 import synth
from oracle import oracle as O

KAT = np.load(os.path.join(os.path.dirname(__file__), "golden", "kat.npz"))


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(f"u{a.dtype.itemsize}")


def test_scale_min_unpack():
    for i in range(16):
        sb = np.zeros(144, np.uint8)
        sb[4:16] = KAT["scales_packed"][i]
        sc, mn = O.q4k_scales(sb)
        assert np.array_equal(sc, KAT["scales_sc"][i]) and np.array_equal(mn, KAT["scales_mn"][i])


def test_dequant_known_answer():
    got = O.q4k_dequant(KAT["dequant_row"], 1, 768)
    assert np.array_equal(bits(got.reshape(-1)), bits(KAT["dequant_want"]))


def test_f16_trunc_and_bf16_rounding():
    lib = O.lib()
    got = np.array([lib.orc_f32_to_f16_trunc(float(v)) for v in KAT["f16_trunc_in"]], np.uint16)
    assert np.array_equal(got, KAT["f16_trunc_want"])
    assert np.array_equal(O.f32_to_bf16(KAT["bf16_in"]), KAT["bf16_want"])
    assert np.array_equal(np.array([lib.orc_f32_to_bf16(float(v)) for v in KAT["bf16_in"]], np.uint16), KAT["bf16_want"])
    assert np.array_equal(synth.f32_to_bf16(KAT["bf16_in"]), KAT["bf16_want"])
    assert lib.orc_q8half_to_f32(0x0001) == 0.0 and lib.orc_f16_to_f32(0x0001) == 2.0 ** -24  # flush vs IEEE decode


def test_q8_1_known_answer():
    got = O.q8_1_quantize(KAT["q8_in"].reshape(1, -1))[0]
    assert np.array_equal(got, KAT["q8_want"])


def test_gemv_closed_forms():
    K = 512
    y = O.gemv_q4k_q8(KAT["gemv_a_row"], 1, K, KAT["gemv_a_xq"])
    assert y[0, 0] == KAT["gemv_a_want"]
    y = O.gemv_q4k_q8(KAT["gemv_b_row"], 1, K, KAT["gemv_a_xq"])
    assert y[0, 0] == KAT["gemv_b_want"]
    isum, qsum = O.block_dots(KAT["gemv_a_row"], KAT["gemv_a_xq"], K)
    q8 = KAT["gemv_a_xq"].reshape(-1, 36)[:, :32].view(np.int8).astype(np.int64)
    assert np.array_equal(isum, q8.sum(1)) and np.array_equal(qsum, q8.sum(1))   # all nibbles are 1


def test_gemv_canonical_vs_plain_and_linearity():
    N, K, B = 48, 4096, 3
    W, x = synth.gemv_case(N, K, B)
    xq = O.q8_1_quantize(x)
    y, yp = O.gemv_q4k_q8(W, N, K, xq), O.gemv_q4k_q8_plain(W, N, K, xq)
    assert np.abs(y - yp).max() / np.abs(yp).max() < 1e-5
    # against unquantised activations the Q8_1 error stays at the percent level
    yf = x.astype(np.float64) @ O.q4k_dequant(W, N, K).astype(np.float64).T
    assert np.abs(yp - yf).max() / np.abs(yf).max() < 2e-2
    # tensor-parallel emulation: K cut in 4 slices, partials summed in rank order
    parts = []
    W3 = W.reshape(N, K // 256, 144)
    for r in range(4):
        Wr = np.ascontiguousarray(W3[:, 4 * r:4 * r + 4]).reshape(N, -1)
        parts.append(O.gemv_q4k_q8(Wr, N, 1024, np.ascontiguousarray(xq[:, 32 * r:32 * r + 32])))
    ys = O.sum_ranks(np.stack(parts))
    assert np.abs(ys - yp).max() / np.abs(yp).max() < 1e-5


def test_gemv_tile_order_is_a_chain_of_four_superblock_chunks():
    """The dense tile path's order: per (row, column) y = ((0 + c0) + c1) + ... over chunks of four superblocks, each
    chunk a chain from zero -- so a chunk computed on its own K slice is exactly that chunk's term (what lets a launch
    be cut along K), and a ragged last chunk (K = 2304: 4 + 4 + 1 superblocks) is a term like any other."""
    N, B = 40, 5
    for K in (1024, 2048, 2304):
        W, x = synth.gemv_case(N, K, B)
        xq = O.q8_1_quantize(x)
        y = O.gemv_q4k_q8_tile(W, N, K, xq)
        yp = O.gemv_q4k_q8_plain(W, N, K, xq)
        assert np.abs(y - yp).max() / np.abs(yp).max() < 1e-5
        W3 = W.reshape(N, K // 256, 144)
        acc = np.zeros((B, N), np.float32)
        for s0 in range(0, K // 256, 4):
            n = min(4, K // 256 - s0)
            Wc = np.ascontiguousarray(W3[:, s0:s0 + n]).reshape(N, -1)
            acc = acc + O.gemv_q4k_q8_tile(Wc, N, n * 256, np.ascontiguousarray(xq[:, 8 * s0:8 * (s0 + n)]))
        assert np.array_equal(bits(acc), bits(y)), K


def test_transcendentals_close_to_libm():
    for x in np.linspace(-80, 80, 4001).astype(np.float32):
        x = float(x)
        assert abs(O.expf(x) - math.exp(x)) <= 3e-7 * math.exp(x)
    for x in np.exp(np.linspace(0, 60, 2001)).astype(np.float32):
        x = float(x)
        assert abs(O.logf(x) - math.log(x)) <= 3e-7 * max(1.0, abs(math.log(x)))
    assert O.expf(0.0) == 1.0 and O.sigmoidf(0.0) == 0.5
    assert O.sigmoidf(-200.0) < 1e-37 and O.sigmoidf(200.0) == 1.0
    assert abs(O.softplusf(30.0) - 30.0) < 1e-5


def test_argmax_ties():
    idx, val = O.argmax(KAT["argmax_in"])
    assert np.array_equal(idx, KAT["argmax_idx"]) and np.array_equal(val, KAT["argmax_val"])


def test_rmsnorm_vs_plain():
    rng = np.random.default_rng(2)
    for H in (256, 2048, 5120):
        x, w = synth.normal_bf16(rng, (2, H), 2.0), synth.normal_bf16(rng, (H,), 0.02)
        y = synth.bf16_to_f32(O.rmsnorm(x, w)).astype(np.float64)
        yp = O.rmsnorm_plain(x, w)
        assert np.abs(y - yp).max() / np.abs(yp).max() < 5e-3   # one bf16 ulp


def test_conv1d_state_shift_and_silu():
    C = 8
    x = O.f32_to_bf16(np.arange(C, dtype=np.float32).reshape(1, C))
    st = O.f32_to_bf16(np.stack([np.full(C, 1.0), np.full(C, 2.0), np.full(C, 3.0)]).astype(np.float32).reshape(1, 3, C))
    w = O.f32_to_bf16(np.tile(np.array([0.5, -1.0, 0.25, 2.0], np.float32), (C, 1)))
    out, sn = O.conv1d_step(x, st, w)
    raw = 0.5 * 1 - 1.0 * 2 + 0.25 * 3 + 2.0 * np.arange(C)
    want = raw / (1 + np.exp(-raw))
    assert np.abs(O.bf16_to_f32(out)[0] - want).max() < 4e-3 * np.abs(want).max()
    assert np.array_equal(sn[0, 0], st[0, 1]) and np.array_equal(sn[0, 1], st[0, 2]) and np.array_equal(sn[0, 2], x[0])


def test_gdn_zero_state_closed_form_and_plain():
    Hk = Hv = 1
    co = np.concatenate([KAT["gdn_q"], KAT["gdn_k"], KAT["gdn_v"]]).reshape(1, -1)
    S0 = np.zeros((1, 1, 128, 128), np.float32)
    Sn, o = O.gdn_step(O.f32_to_bf16(co), np.array([[KAT["gdn_a"]]], np.float32), np.array([[KAT["gdn_beta_logit"]]], np.float32),
                       np.zeros(1, np.float32), O.f32_to_bf16(np.zeros(1, np.float32)), S0, Hk, Hv)
    assert np.abs(o[0, 0] - KAT["gdn_o_want"]).max() < 1e-5 * np.abs(KAT["gdn_o_want"]).max() + 1e-7
    assert np.abs(Sn[0, 0, 3] - KAT["gdn_S33_want"]).max() < 1e-6 * np.abs(KAT["gdn_S33_want"]).max() + 1e-7
    assert np.count_nonzero(np.delete(Sn[0, 0], 3, axis=0)) == 0
    # random case against the double recurrence of prototypes/gdn_gated.ts:67-88
    c = synth.gdn_case(1, Hk=1, Hv=2, config_id=55)
    Sn, o = O.gdn_step(c["qkv"], c["a"], c["b"], c["A_log"], c["dt_bias"], c["S"], 1, 2)
    f = synth.bf16_to_f32(c["qkv"][0])
    for hv in range(2):
        sp = math.log1p(math.exp(float(c["a"][0, hv]) + float(synth.bf16_to_f32(c["dt_bias"])[hv])))
        decay = math.exp(-math.exp(float(c["A_log"][hv])) * sp)
        beta = 1 / (1 + math.exp(-float(c["b"][0, hv])))
        Sp, op = O.gdn_step_plain(f[0:128], f[128:256], f[256 + 128 * hv:384 + 128 * hv], decay, beta, c["S"][0, hv])
        assert np.abs(Sn[0, hv] - Sp).max() / np.abs(Sp).max() < 1e-3
        assert np.abs(o[0, hv] - op).max() / np.abs(op).max() < 1e-3


def test_attention_uniform_keys_and_split_invariance():
    n, HD = 40, 256
    Kc = np.zeros((1, 1, 64, HD), np.uint16)
    Vc = np.zeros((1, 1, 64, HD), np.uint16)
    Kc[0, 0, :n] = O.f32_to_bf16(KAT["attn_k"])
    Vc[0, 0, :n] = O.f32_to_bf16(KAT["attn_V"])
    q = O.f32_to_bf16(KAT["attn_q"].reshape(1, HD))
    gate = O.f32_to_bf16(np.full((1, HD), 30.0, np.float32))      # sigmoid(30) == 1 in f32
    pos = np.array([n - 1], np.int32)
    want = O.bf16_to_f32(Vc[0, 0, :n]).astype(np.float64).mean(0)
    outs = []
    for split_len, W in ((64, 8), (8, 8), (16, 3)):
        out = O.bf16_to_f32(O.attn_decode(q, gate, HD, Kc, Vc, pos, 1, 1, HD, split_len, W, 1 / 16))[0]
        assert np.abs(out - want).max() < 5e-3 * np.abs(want).max()
        outs.append(out)
    plain = O.attn_decode_plain(q[0], Kc[0, 0], Vc[0, 0], n, HD, 1 / 16)
    assert np.abs(plain - want).max() < 1e-6


def test_rope_tables_and_rotation():
    c, s = O.rope_tables(8, 64, float(KAT["rope_theta"]))
    assert np.array_equal(c[0], np.ones(32, np.float32)) and np.array_equal(s[0], np.zeros(32, np.float32))
    assert np.array_equal(c[5], KAT["rope_cos_p5"]) and np.array_equal(s[5], KAT["rope_sin_p5"])
    HD = 256
    x = O.f32_to_bf16(np.random.default_rng(4).normal(0, 1, (2, HD)).astype(np.float32))
    w = np.zeros(HD, np.uint16)
    y0 = O.headnorm_rope(x, HD, w, c, s, np.array([0, 0], np.int32), 1, HD)
    y5 = O.headnorm_rope(x, HD, w, c, s, np.array([5, 5], np.int32), 1, HD)
    f0, f5 = O.bf16_to_f32(y0), O.bf16_to_f32(y5)
    assert np.array_equal(y0[:, 64:], y5[:, 64:])                 # dims beyond the rotary part pass through
    a = f0[:, :32] * c[5] - f0[:, 32:64] * s[5]
    assert np.abs(f5[:, :32] - a).max() < 2e-2
    rms = np.sqrt((f0.astype(np.float64) ** 2).mean(1))
    assert np.abs(rms - 1).max() < 1e-2                            # normalised, weight 1+0
