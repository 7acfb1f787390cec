"""GPU parity of the non-GEMV decode ops (embed, rmsnorm, swiglu, conv1d, GDN step, head norm + rope,
attention, argmax) against the CPU oracle: bit-exact against the canonical-order functions, 1e-3
relative against the plain restatements of the reference's host loops."""
import numpy as np
import pytest

from bunker_b200 import ops, synth
from bunker_b200 import runtime as R
from oracle import oracle as O
from tests.util import assert_same_bits, dev, rel_err

pytestmark = pytest.mark.gpu


def test_embed(bk):
    V, H, B = 300, 2048, 5
    table = synth.q4k_weights(np.random.default_rng(5), V, H)
    ids = np.array([0, 299, 17, 17, 123], np.int32)
    dt, di, out = dev(table), dev(ids), R.DeviceBuffer(B * H * 2)
    ops.embed(dt.ptr, H, di.ptr, B, out.ptr)
    assert_same_bits(out.download(np.uint16, (B, H)), O.embed_q4k(table, H, ids), "embed")


@pytest.mark.parametrize("H", [2048, 5120, 256])
def test_rmsnorm(bk, H):
    B = 3
    rng = np.random.default_rng(6)
    x, w = synth.normal_bf16(rng, (B, H), 3.0), synth.normal_bf16(rng, (H,), 0.02)
    dx, dw, dy = dev(x), dev(w), R.DeviceBuffer(B * H * 2)
    ops.rmsnorm(dx.ptr, dw.ptr, H, B, dy.ptr)
    y = dy.download(np.uint16, (B, H))
    assert_same_bits(y, O.rmsnorm(x, w), "rmsnorm")
    assert rel_err(synth.bf16_to_f32(y), O.rmsnorm_plain(x, w)) < 5e-3  # bf16 output rounding


@pytest.mark.parametrize("K", [256, 2048, 5120, 17408])
def test_rmsnorm_quant_q8_1(bk, K):
    """The stand-alone (RMSNorm ->) Q8_1 launch used between ops at batch >= 2, with and without the norm."""
    B = 5
    rng = np.random.default_rng(60)
    x, w = synth.normal_bf16(rng, (B, K), 2.0), synth.normal_bf16(rng, (K,), 0.02)
    x[1, :32] = 0  # an all-zero block: d = 0
    dx, dw, dq = dev(x), dev(w), R.DeviceBuffer(B * K // 32 * 36)
    ops.rmsnorm_quant_q8_1(dx.ptr, dw.ptr, K, B, dq.ptr)
    assert_same_bits(dq.download(np.uint8, (B, K // 32, 36)), O.q8_1_quantize_bf16(O.rmsnorm(x, w)), "norm + Q8_1")
    ops.rmsnorm_quant_q8_1(dx.ptr, 0, K, B, dq.ptr)
    assert_same_bits(dq.download(np.uint8, (B, K // 32, 36)), O.q8_1_quantize_bf16(x), "plain Q8_1")
    # the staged image carries the same quants, block scales (after their f16 round trip) and d8 * sum(q)
    img = R.DeviceBuffer.zeros(ops.staged_bytes(K, B))
    for w_ptr, ref in ((dw.ptr, O.rmsnorm(x, w)), (0, x)):
        ops.rmsnorm_quant_q8_1(dx.ptr, w_ptr, K, B, img.ptr, layout=R.BK_Q8_STAGED)
        _check_staged(img.download(np.uint8, (ops.staged_bytes(K, B),)), O.q8_1_quantize_bf16(ref), K, B)


def _check_staged(img, blocks, K, B):
    q, d8, s8 = ops.staged_to_blocks(img, K, B)
    assert_same_bits(q.reshape(B, K // 32, 32), blocks[:, :, :32].view(np.int8), "staged quants")
    want_d8 = O.q8_1_scales(blocks)
    assert_same_bits(d8, want_d8, "staged block scales")
    want_s8 = want_d8 * blocks[:, :, :32].view(np.int8).astype(np.int32).sum(-1).astype(np.float32)
    assert_same_bits(s8, want_s8.astype(np.float32), "staged d8 * sum(q)")


def test_swiglu(bk):
    n = 6144
    rng = np.random.default_rng(7)
    g, u = rng.normal(0, 4, n).astype(np.float32), rng.normal(0, 4, n).astype(np.float32)
    g[:4] = [0.0, -100.0, 100.0, -1e-8]
    dg, du, out = dev(g), dev(u), R.DeviceBuffer(n * 2)
    ops.swiglu(dg.ptr, du.ptr, n, out.ptr)
    assert_same_bits(out.download(np.uint16, (n,)), O.swiglu(g, u), "swiglu")


def test_conv1d_step(bk):
    B, Cw = 2, 8192
    rng = np.random.default_rng(8)
    x, st, w = synth.normal_bf16(rng, (B, Cw)), synth.normal_bf16(rng, (B, 3, Cw)), synth.normal_bf16(rng, (Cw, 4), 0.3)
    dx, ds, dw = dev(x), dev(st), dev(w)
    out, sn = R.DeviceBuffer(B * Cw * 2), R.DeviceBuffer(B * 3 * Cw * 2)
    ops.conv1d_step(dx.ptr, ds.ptr, dw.ptr, Cw, B, out.ptr, sn.ptr)
    wo, ws = O.conv1d_step(x, st, w)
    assert_same_bits(out.download(np.uint16, (B, Cw)), wo, "conv out")
    assert_same_bits(sn.download(np.uint16, (B, 3, Cw)), ws, "conv state")


def _gdn_oracle(c):
    conv_out, cs_new = O.conv1d_step(c["qkv"], c["conv_state"], c["conv_w"])
    S_new, o_raw = O.gdn_step(conv_out, c["a"], c["b"], c["A_log"], c["dt_bias"], c["S"], c["Hk"], c["Hv"])
    out = O.gdn_gate_norm(o_raw, c["z"], c["norm_w"], c["Hv"])
    return conv_out, cs_new, S_new, o_raw, out


@pytest.mark.parametrize("B", [1, 8])
def test_gdn_step_config1(bk, B):
    """configs[1]: 16 key heads, 32 value heads, d=128, fused causal conv over width 8192."""
    c = synth.gdn_case(B)
    Hk, Hv = c["Hk"], c["Hv"]
    Cw = 2 * Hk * 128 + Hv * 128
    d = {k: dev(v) for k, v in c.items() if isinstance(v, np.ndarray)}
    cs_new, S_new = R.DeviceBuffer(B * 3 * Cw * 2), R.DeviceBuffer(B * Hv * 128 * 128 * 4)
    out, o_raw, conv_out = R.DeviceBuffer(B * Hv * 128 * 2), R.DeviceBuffer(B * Hv * 128 * 4), R.DeviceBuffer(B * Cw * 2)
    out_q8 = R.DeviceBuffer(B * Hv * 4 * 36)
    ops.gdn_step(out_q8=out_q8.ptr, qkv=d["qkv"].ptr, z=d["z"].ptr, a=d["a"].ptr, b=d["b"].ptr, conv_w=d["conv_w"].ptr,
                 conv_state_in=d["conv_state"].ptr, conv_state_new=cs_new.ptr, A_log=d["A_log"].ptr,
                 dt_bias=d["dt_bias"].ptr, norm_w=d["norm_w"].ptr, S_in=d["S"].ptr, S_new=S_new.ptr, out=out.ptr,
                 o_raw=o_raw.ptr, conv_out=conv_out.ptr, B=B, Hk=Hk, Hv=Hv, apply_conv=1)
    w_conv, w_cs, w_S, w_o, w_out = _gdn_oracle(c)
    assert_same_bits(conv_out.download(np.uint16, (B, Cw)), w_conv, "conv_out")
    assert_same_bits(cs_new.download(np.uint16, (B, 3, Cw)), w_cs, "conv state")
    assert_same_bits(o_raw.download(np.float32, (B, Hv, 128)), w_o, "o_raw")
    assert_same_bits(S_new.download(np.float32, (B, Hv, 128, 128)), w_S, "S_new")
    assert_same_bits(out.download(np.uint16, (B, Hv * 128)), w_out, "gated out")
    assert_same_bits(out_q8.download(np.uint8, (B, Hv * 4, 36)), O.q8_1_quantize_bf16(w_out).reshape(B, Hv * 4, 36),
                     "gated out as Q8_1 blocks")
    img = R.DeviceBuffer.zeros(ops.staged_bytes(Hv * 128, B))
    d2 = dev(c["S"])
    ops.gdn_step(out_q8=img.ptr, out_q8_layout=R.BK_Q8_STAGED, qkv=d["qkv"].ptr, z=d["z"].ptr, a=d["a"].ptr, b=d["b"].ptr,
                 conv_w=d["conv_w"].ptr, conv_state_in=d["conv_state"].ptr, conv_state_new=cs_new.ptr,
                 A_log=d["A_log"].ptr, dt_bias=d["dt_bias"].ptr, norm_w=d["norm_w"].ptr, S_in=d2.ptr, S_new=S_new.ptr,
                 out=out.ptr, B=B, Hk=Hk, Hv=Hv, apply_conv=1)
    _check_staged(img.download(np.uint8, (ops.staged_bytes(Hv * 128, B),)), O.q8_1_quantize_bf16(w_out), Hv * 128, B)
    # plain recurrence (prototypes/gdn_gated.ts:67-88) on head (0, 5), double math
    import math
    hv, hk = 5, 5 // (Hv // Hk)
    co = synth.bf16_to_f32(w_conv[0])
    q, k = co[hk * 128:(hk + 1) * 128], co[Hk * 128 + hk * 128: Hk * 128 + (hk + 1) * 128]
    v = co[2 * Hk * 128 + hv * 128: 2 * Hk * 128 + (hv + 1) * 128]
    sp = math.log1p(math.exp(float(c["a"][0, hv]) + float(synth.bf16_to_f32(c["dt_bias"][hv:hv + 1])[0])))
    decay = math.exp(-math.exp(float(c["A_log"][hv])) * sp)
    beta = 1.0 / (1.0 + math.exp(-float(c["b"][0, hv])))
    Sp, op = O.gdn_step_plain(q, k, v, decay, beta, c["S"][0, hv])
    assert rel_err(w_S[0, hv], Sp) < 1e-3 and rel_err(w_o[0, hv], op) < 1e-3


def test_gdn_step_several_tokens_in_one_launch(bk):
    """n_tokens = 3: three consecutive tokens of two sequences in one launch (state and conv taps stay in registers)
    equal three single-token launches: outputs of every token, final state, final conv state; staged output too."""
    B, T = 2, 3
    cases = [synth.gdn_case(B, config_id=50 + t) for t in range(T)]
    c0 = cases[0]
    Hk, Hv = c0["Hk"], c0["Hv"]
    Cw = 2 * Hk * 128 + Hv * 128
    S, cs = c0["S"], c0["conv_state"]
    want_out = []
    for t in range(T):
        c = dict(cases[t], S=S, conv_state=cs, conv_w=c0["conv_w"], A_log=c0["A_log"], dt_bias=c0["dt_bias"], norm_w=c0["norm_w"])
        _, cs, S, _, out = _gdn_oracle(c)
        want_out.append(out)
    stack = lambda k: np.ascontiguousarray(np.concatenate([cases[t][k] for t in range(T)], axis=0))
    d = {k: dev(stack(k)) for k in ("qkv", "z", "a", "b")}
    d0 = {k: dev(c0[k]) for k in ("conv_w", "conv_state", "A_log", "dt_bias", "norm_w", "S")}
    cs_new, out = R.DeviceBuffer(B * 3 * Cw * 2), R.DeviceBuffer(T * B * Hv * 128 * 2)
    img = R.DeviceBuffer.zeros(ops.staged_bytes(Hv * 128, T * B))
    ops.gdn_step(qkv=d["qkv"].ptr, z=d["z"].ptr, a=d["a"].ptr, b=d["b"].ptr, conv_w=d0["conv_w"].ptr,
                 conv_state_in=d0["conv_state"].ptr, conv_state_new=cs_new.ptr, A_log=d0["A_log"].ptr,
                 dt_bias=d0["dt_bias"].ptr, norm_w=d0["norm_w"].ptr, S_in=d0["S"].ptr, S_new=d0["S"].ptr, out=out.ptr,
                 out_q8=img.ptr, out_q8_layout=R.BK_Q8_STAGED, B=B, Hk=Hk, Hv=Hv, apply_conv=1, n_tokens=T)
    got = out.download(np.uint16, (T, B, Hv * 128))
    for t in range(T):
        assert_same_bits(got[t], want_out[t], f"gated out of token {t}")
    assert_same_bits(d0["S"].download(np.float32, (B, Hv, 128, 128)), S, "state after the last token")
    assert_same_bits(cs_new.download(np.uint16, (B, 3, Cw)), cs, "conv state after the last token")
    _check_staged(img.download(np.uint8, (ops.staged_bytes(Hv * 128, T * B),)),
                  O.q8_1_quantize_bf16(np.concatenate(want_out, axis=0)), Hv * 128, T * B)


def test_gdn_step_without_conv(bk):
    c = synth.gdn_case(2, Hk=2, Hv=4, config_id=21)
    Hk, Hv, B = 2, 4, 2
    d = {k: dev(v) for k, v in c.items() if isinstance(v, np.ndarray)}
    S_new, out = R.DeviceBuffer(B * Hv * 128 * 128 * 4), R.DeviceBuffer(B * Hv * 128 * 2)
    ops.gdn_step(qkv=d["qkv"].ptr, z=d["z"].ptr, a=d["a"].ptr, b=d["b"].ptr, A_log=d["A_log"].ptr,
                 dt_bias=d["dt_bias"].ptr, norm_w=d["norm_w"].ptr, S_in=d["S"].ptr, S_new=S_new.ptr, out=out.ptr,
                 B=B, Hk=Hk, Hv=Hv, apply_conv=0)
    w_S, w_o = O.gdn_step(c["qkv"], c["a"], c["b"], c["A_log"], c["dt_bias"], c["S"], Hk, Hv)
    assert_same_bits(S_new.download(np.float32, (B, Hv, 128, 128)), w_S, "S_new")
    assert_same_bits(out.download(np.uint16, (B, Hv * 128)), O.gdn_gate_norm(w_o, c["z"], c["norm_w"], Hv), "out")


def test_headnorm_rope(bk):
    B, nh, HD = 3, 16, 256
    rng = np.random.default_rng(9)
    x, w = synth.normal_bf16(rng, (B, nh * 2 * HD)), synth.normal_bf16(rng, (HD,), 0.02)
    cos_t, sin_t = ops.rope_tables(4096)
    oc, os_ = O.rope_tables(4096)
    assert_same_bits(cos_t, oc, "cos table")
    assert_same_bits(sin_t, os_, "sin table")
    pos = np.array([0, 77, 4095], np.int32)
    dx, dw, dc, ds, dp = dev(x), dev(w), dev(cos_t), dev(sin_t), dev(pos)
    out = R.DeviceBuffer(B * nh * HD * 2)
    ops.headnorm_rope(dx.ptr, 2 * HD, dw.ptr, dc.ptr, ds.ptr, 32, dp.ptr, B, nh, HD, out.ptr)
    assert_same_bits(out.download(np.uint16, (B, nh * HD)), O.headnorm_rope(x, 2 * HD, w, cos_t, sin_t, pos, nh, HD),
                     "headnorm_rope")


def _attn_oracle(c, cos_t, sin_t, split_len, W):
    B, Hq, Hkv, HD = c["B"], c["Hq"], c["Hkv"], c["HD"]
    q = O.headnorm_rope(c["qg"], 2 * HD, c["q_norm_w"], cos_t, sin_t, c["pos"], Hq, HD)
    k = O.headnorm_rope(c["k"], HD, c["k_norm_w"], cos_t, sin_t, c["pos"], Hkv, HD)
    Kc, Vc = c["k_cache"].copy(), c["v_cache"].copy()
    for b in range(B):
        Kc[b, :, c["pos"][b]] = k[b].reshape(Hkv, HD)
        Vc[b, :, c["pos"][b]] = c["v"][b].reshape(Hkv, HD)
    gate = np.ascontiguousarray(c["qg"].reshape(B, Hq, 2, HD)[:, :, 1])
    out = O.attn_decode(q, gate, HD, Kc, Vc, c["pos"], Hq, Hkv, HD, split_len, W, 1.0 / 16.0)
    return q, Kc, Vc, out


def _run_attn(c, cos_t, sin_t, split_len=0):
    B, Hq, Hkv, HD, ml = c["B"], c["Hq"], c["Hkv"], c["HD"], c["max_len"]
    max_pos = int(c["pos"].max())
    plan_len, W = ops.attn_plan(max_pos + 1, B, Hkv)   # W: row classes (warps per split) of the library's kernel
    if split_len == 0:
        split_len = plan_len
    d = {k: dev(v) for k, v in c.items() if isinstance(v, np.ndarray)}
    dc, ds = dev(cos_t), dev(sin_t)
    scratch = R.DeviceBuffer.zeros(ops.attn_scratch_bytes(B, Hq, HD, ml, split_len))
    out, out_q8 = R.DeviceBuffer(B * Hq * HD * 2), R.DeviceBuffer(B * Hq * HD // 32 * 36)
    ops.attn_decode(out_q8=out_q8.ptr, qg=d["qg"].ptr, k=d["k"].ptr, v=d["v"].ptr, q_norm_w=d["q_norm_w"].ptr, k_norm_w=d["k_norm_w"].ptr,
                    cos_t=dc.ptr, sin_t=ds.ptr, k_cache=d["k_cache"].ptr, v_cache=d["v_cache"].ptr, pos=d["pos"].ptr,
                    out=out.ptr, scratch=scratch.ptr, B=B, Hq=Hq, Hkv=Hkv, HD=HD, rot_half=32, max_len=ml,
                    split_len=split_len, max_pos=max_pos, scale=1.0 / 16.0, fused_norm_rope=1)
    got = out.download(np.uint16, (B, Hq * HD))
    assert_same_bits(out_q8.download(np.uint8, (B, Hq * HD // 32, 36)),
                     O.q8_1_quantize_bf16(got).reshape(B, Hq * HD // 32, 36), "attention output as Q8_1 blocks")
    out_q8.free()
    if B <= 8:   # same call again (the cache row is rewritten with the same values) with the staged layout
        img = R.DeviceBuffer.zeros(ops.staged_bytes(Hq * HD, B))
        ops.attn_decode(out_q8=img.ptr, out_q8_layout=R.BK_Q8_STAGED, qg=d["qg"].ptr, k=d["k"].ptr, v=d["v"].ptr,
                        q_norm_w=d["q_norm_w"].ptr, k_norm_w=d["k_norm_w"].ptr, cos_t=dc.ptr, sin_t=ds.ptr,
                        k_cache=d["k_cache"].ptr, v_cache=d["v_cache"].ptr, pos=d["pos"].ptr, out=out.ptr,
                        scratch=scratch.ptr, B=B, Hq=Hq, Hkv=Hkv, HD=HD, rot_half=32, max_len=ml, split_len=split_len,
                        max_pos=max_pos, scale=1.0 / 16.0, fused_norm_rope=1)
        _check_staged(img.download(np.uint8, (ops.staged_bytes(Hq * HD, B),)), O.q8_1_quantize_bf16(got), Hq * HD, B)
        img.free()
    Kg = d["k_cache"].download(np.uint16, c["k_cache"].shape)
    Vg = d["v_cache"].download(np.uint16, c["v_cache"].shape)
    for b in d.values():
        b.free()
    scratch.free(), out.free(), dc.free(), ds.free()
    return got, Kg, Vg, split_len, W


@pytest.mark.parametrize("B,L", [(1, 1), (1, 7), (2, 64), (1, 65), (2, 300), (1, 1024), (8, 1024), (1, 4096)])
def test_attn_decode(bk, B, L):
    """configs[2] shapes: 16 q heads, 2 kv heads, head_dim 256, rotary 64 of 256, theta 1e7, sigmoid gate."""
    cos_t, sin_t = ops.rope_tables(max(L, 64))
    c = synth.attn_case(B, L)
    got, Kg, Vg, split_len, W = _run_attn(c, cos_t, sin_t)
    q, Kc, Vc, want = _attn_oracle(c, cos_t, sin_t, split_len, W)
    assert_same_bits(Kg, Kc, "k cache after append")
    assert_same_bits(Vg, Vc, "v cache after append")
    assert_same_bits(got, want, f"attention B={B} L={L} split_len={split_len}")


def test_attn_decode_ragged_positions_and_plain(bk):
    """Sequences of different lengths in one batch; one head also checked against the plain softmax."""
    B, L = 4, 700
    cos_t, sin_t = ops.rope_tables(1024)
    c = synth.attn_case(B, L, max_len=1024, config_id=31)
    c["pos"] = np.array([0, 63, 64, 699], np.int32)
    got, Kg, Vg, split_len, W = _run_attn(c, cos_t, sin_t, split_len=64)
    q, Kc, Vc, want = _attn_oracle(c, cos_t, sin_t, split_len, W)
    assert_same_bits(got, want, "ragged attention")
    b, h, HD = 3, 9, 256
    kvh = h // 8
    plain = O.attn_decode_plain(q[b, h * HD:(h + 1) * HD], Kc[b, kvh], Vc[b, kvh], 700, HD, 1.0 / 16.0)
    gate = synth.bf16_to_f32(c["qg"].reshape(B, 16, 2, HD)[b, h, 1]).astype(np.float64)
    plain = plain / (1.0 + np.exp(-gate))
    assert rel_err(synth.bf16_to_f32(got[b, h * HD:(h + 1) * HD]), plain) < 5e-3  # bf16 output rounding


@pytest.mark.parametrize("B,L", [(1, 32768), (8, 4096), (8, 32768)])
def test_attn_decode_long_context(bk, B, L):
    """configs[2] long caches (4096 and 32768 rows) at batch 1 and 8, default plan; bit-exact against the oracle."""
    cos_t, sin_t = ops.rope_tables(L)
    c = synth.attn_case(B, L)
    got, Kg, Vg, split_len, W = _run_attn(c, cos_t, sin_t)
    q, Kc, Vc, want = _attn_oracle(c, cos_t, sin_t, split_len, W)
    assert_same_bits(got, want, f"attention B={B} L={L} split_len={split_len}")


def test_argmax(bk):
    B, V = 3, 151936
    rng = np.random.default_rng(11)
    logits = rng.normal(0, 3, (B, V)).astype(np.float32)
    logits[0, 5] = logits[0, 150000] = 50.0       # tie: lowest index wins
    logits[1, V - 1] = 60.0                       # maximum in the last, short chunk
    logits[2, :] = -7.0                           # all equal -> index 0
    dl, idx, val = dev(logits), R.DeviceBuffer(B * 4), R.DeviceBuffer(B * 4)
    scratch = R.DeviceBuffer.zeros(ops.argmax_scratch_bytes(B))
    for _ in range(2):  # second call checks that the kernel re-armed its counters
        ops.argmax(dl.ptr, V, B, idx.ptr, val.ptr, scratch.ptr)
    wi, wv = O.argmax(logits)
    assert np.array_equal(idx.download(np.int32, (B,)), wi) and list(wi) == [5, V - 1, 0]
    assert_same_bits(val.download(np.float32, (B,)), wv, "argmax value")


def test_culaunch_surface(bk):
    """The cuLaunch-shaped path (src/ttir.ts:321-348): op handle + 8-byte slots; rc returned, not raised."""
    H, B = 2048, 2
    rng = np.random.default_rng(12)
    x, w = synth.normal_bf16(rng, (B, H)), synth.normal_bf16(rng, (H,), 0.02)
    dx, dw, dy = R.cuAlloc(x.nbytes), R.cuAlloc(w.nbytes), R.cuAlloc(x.nbytes)
    R.cuHtoD(dx, x), R.cuHtoD(dw, w)
    k = R.loadOp("rmsnorm")
    assert R.cuLaunch(k, [1, 1, 1], [128, 1, 1], [dx, dw, dy, H, B, 1e-6]) == 0
    assert R.cuSync() == 0
    y = np.empty_like(x)
    R.cuDtoH(y, dy)
    assert_same_bits(y, O.rmsnorm(x, w), "rmsnorm via cuLaunch")
    assert R.cuLaunch(k, [1, 1, 1], [128, 1, 1], [dx, dw]) == R.BK_ERR_ARG  # wrong slot count -> rc, no raise
    for p in (dx, dw, dy):
        R.cuFree(p)


def test_culaunch_fused_ops(bk):
    """gdn_delta_rule, fa2_attn and headnorm_rope through cuLaunch slot lists give the results of the struct calls."""
    # GDN
    B = 2
    c = synth.gdn_case(B, Hk=2, Hv=4, config_id=61)
    Hk, Hv = 2, 4
    Cw = 2 * Hk * 128 + Hv * 128
    d = {k: dev(v) for k, v in c.items() if isinstance(v, np.ndarray)}
    cs_new, out = R.DeviceBuffer(B * 3 * Cw * 2), R.DeviceBuffer(B * Hv * 128 * 2)
    k = R.loadOp("gdn_delta_rule")
    rc = R.cuLaunch(k, [1, 1, 1], [1, 1, 1], [d["qkv"].ptr, d["z"].ptr, d["a"].ptr, d["b"].ptr, d["conv_w"].ptr,
                                              d["conv_state"].ptr, cs_new.ptr, d["A_log"].ptr, d["dt_bias"].ptr,
                                              d["norm_w"].ptr, d["S"].ptr, d["S"].ptr, out.ptr, B, Hk, Hv, 1, 0])
    assert rc == 0, R.last_error()
    _, w_cs, w_S, _, w_out = _gdn_oracle(c)
    assert_same_bits(out.download(np.uint16, (B, Hv * 128)), w_out, "gdn via cuLaunch")
    assert_same_bits(d["S"].download(np.float32, (B, Hv, 128, 128)), w_S, "state via cuLaunch")
    assert_same_bits(cs_new.download(np.uint16, (B, 3, Cw)), w_cs, "conv state via cuLaunch")
    # attention
    B, L = 2, 100
    cos_t, sin_t = ops.rope_tables(128)
    ca = synth.attn_case(B, L, max_len=128, config_id=62)
    Hq, Hkv, HD, ml = ca["Hq"], ca["Hkv"], ca["HD"], ca["max_len"]
    split_len, W = ops.attn_plan(L, B, Hkv)
    da = {kk: dev(v) for kk, v in ca.items() if isinstance(v, np.ndarray)}
    dc, ds = dev(cos_t), dev(sin_t)
    scratch = R.DeviceBuffer.zeros(ops.attn_scratch_bytes(B, Hq, HD, ml, split_len))
    o = R.DeviceBuffer(B * Hq * HD * 2)
    k = R.loadOp("fa2_attn")
    rc = R.cuLaunch(k, [1, 1, 1], [1, 1, 1], [da["qg"].ptr, da["k"].ptr, da["v"].ptr, da["q_norm_w"].ptr, da["k_norm_w"].ptr,
                                              dc.ptr, ds.ptr, da["k_cache"].ptr, da["v_cache"].ptr, da["pos"].ptr, o.ptr,
                                              scratch.ptr, B, Hq, Hkv, HD, 32, ml, split_len, int(ca["pos"].max()),
                                              1.0 / 16.0, 0])
    assert rc == 0, R.last_error()
    _, _, _, want = _attn_oracle(ca, cos_t, sin_t, split_len, W)
    assert_same_bits(o.download(np.uint16, (B, Hq * HD)), want, "attention via cuLaunch")
    assert R.cuLaunch(k, [1, 1, 1], [1, 1, 1], [1, 2, 3]) == R.BK_ERR_ARG
    # head norm + rope
    rng = np.random.default_rng(63)
    nh = 4
    x, w = synth.normal_bf16(rng, (B, nh * HD)), synth.normal_bf16(rng, (HD,), 0.02)
    pos = np.array([3, 77], np.int32)
    dx, dw, dp, y = dev(x), dev(w), dev(pos), R.DeviceBuffer(B * nh * HD * 2)
    rc = R.cuLaunch(R.loadOp("headnorm_rope"), [1, 1, 1], [1, 1, 1], [dx.ptr, HD, dw.ptr, dc.ptr, ds.ptr, 32, dp.ptr, B, nh, HD, y.ptr])
    assert rc == 0, R.last_error()
    assert_same_bits(y.download(np.uint16, (B, nh * HD)), O.headnorm_rope(x, HD, w, cos_t, sin_t, pos, nh, HD), "headnorm_rope via cuLaunch")


@pytest.mark.parametrize("n_ranks", [1, 2, 3, 4, 8])
def test_exchange_reduce_all_rank_counts_on_one_gpu(bk, n_ranks):
    """The consumer of the tensor-parallel exchange with the ranks' tagged words laid out by the host: sum in rank order +
    residual -> bf16 -> RMSNorm -> Q8_1, for every rank count (pairs of ranks per polling pass, odd tail included)."""
    B, K = 3, 2048
    rng = np.random.default_rng(300 + n_ranks)
    parts = rng.normal(0, 1, (n_ranks, B, K)).astype(np.float32)
    res, w = synth.normal_bf16(rng, (B, K)), synth.normal_bf16(rng, (K,), 0.02)
    epoch, tag_add = 7, 5
    tag = epoch * 256 + tag_add
    stride = B * K + 64          # words between ranks (padded)
    words = np.zeros((n_ranks, stride, 2), np.uint32)
    words[:, :B * K, 0] = parts.reshape(n_ranks, -1).view(np.uint32)
    words[:, :B * K, 1] = tag
    dw_, de, dres, dnw = dev(words), dev(np.array([epoch], np.uint32)), dev(res), dev(w)
    dsum, dq = R.DeviceBuffer.zeros(B * K * 2), R.DeviceBuffer(B * K // 32 * 36)
    R._check(R.cu().bkReduceRmsNormQuantQ8_1(dw_.ptr, n_ranks, stride, de.ptr, tag_add, dres.ptr, dsum.ptr, dnw.ptr, K, B, 1e-6,
                                             dq.ptr, R.BK_Q8_BLOCKS))
    want_sum = O.epilogue_add(O.sum_ranks(parts), res)
    assert_same_bits(dsum.download(np.uint16, (B, K)), want_sum, "sum of the ranks + residual")
    assert_same_bits(dq.download(np.uint8, (B, K // 32, 36)), O.q8_1_quantize_bf16(O.rmsnorm(want_sum, w)), "norm + Q8_1")


def test_exchange_wait_runs_out_and_reports_timeout(bk):
    """A bounded device-side wait that can never be satisfied: the consumer of the tensor-parallel exchange is given
    words whose tag never matches and a poll limit of a few hundred.  The launch must return by itself, bkSync must
    report BK_ERR_TIMEOUT once (and clear the status), and the same call with matching tags must then pass."""
    B, K, n_ranks = 1, 2048, 2
    rng = np.random.default_rng(77)
    parts = rng.normal(0, 1, (n_ranks, B, K)).astype(np.float32)
    res, w = synth.normal_bf16(rng, (B, K)), synth.normal_bf16(rng, (K,), 0.02)
    epoch, tag_add = 3, 9
    stride = B * K
    words = np.zeros((n_ranks, stride, 2), np.uint32)
    words[:, :, 0] = parts.reshape(n_ranks, -1).view(np.uint32)
    words[:, :, 1] = epoch * 256 + tag_add + 1          # a tag this exchange never waits for
    dw_, de, dres, dnw = dev(words), dev(np.array([epoch], np.uint32)), dev(res), dev(w)
    dsum, dq = R.DeviceBuffer.zeros(B * K * 2), R.DeviceBuffer(B * K // 32 * 36)
    lib = R.cu()
    assert R.cuSync() == 0
    R._check(lib.bkSetSpinLimit(200))
    try:
        R._check(lib.bkReduceRmsNormQuantQ8_1(dw_.ptr, n_ranks, stride, de.ptr, tag_add, dres.ptr, dsum.ptr, dnw.ptr, K, B,
                                              1e-6, dq.ptr, R.BK_Q8_BLOCKS))
        assert R.cuSync() == R.BK_ERR_TIMEOUT
        assert "bounded device-side wait" in R.last_error()
        assert R.cuSync() == 0                           # reported once, then cleared
    finally:
        R._check(lib.bkSetSpinLimit(0))
    words[:, :, 1] = epoch * 256 + tag_add
    R.cuHtoD(dw_.ptr, words)
    R._check(lib.bkReduceRmsNormQuantQ8_1(dw_.ptr, n_ranks, stride, de.ptr, tag_add, dres.ptr, dsum.ptr, dnw.ptr, K, B, 1e-6,
                                          dq.ptr, R.BK_Q8_BLOCKS))
    assert R.cuSync() == 0
    want_sum = O.epilogue_add(O.sum_ranks(parts), res)
    assert_same_bits(dsum.download(np.uint16, (B, K)), want_sum, "sum of the ranks + residual after a timed-out call")


def test_sampling_matches_oracle(bk):
    """Temperature / top-k / top-p sampling: the same token as the CPU checker for every (seed, step, sequence) tried,
    the argmax at temperature 0 and at top_k 1, ties resolved to the lower index, and a plausible spread of tokens."""
    B, V = 4, 151936
    rng = np.random.default_rng(70)
    logits = rng.normal(0, 2, (B, V)).astype(np.float32)
    logits[0, 7] = logits[0, 100000] = 9.5          # a tie among the candidates
    logits[1, :] = -3.0                             # all equal: candidates are indices 0..k-1
    logits[2, 5] = np.nan                           # NaN is never a candidate
    dl, idx, val = dev(logits), R.DeviceBuffer(B * 4), R.DeviceBuffer(B * 4)
    steps = np.array([0, 5, 9, 1000], np.int32)
    dsteps = dev(steps)
    seen = set()
    for seed in range(6):
        for (T, k, p) in ((1.0, 40, 1.0), (0.7, 64, 0.9), (1.5, 8, 0.5), (0.0, 40, 1.0), (1.0, 1, 1.0)):
            ops.sample(dl.ptr, V, B, idx.ptr, val.ptr, temperature=T, top_k=k, top_p=p, seed=seed, step_dev=dsteps.ptr, step_add=seed * 3)
            gi, gv = idx.download(np.int32, (B,)), val.download(np.float32, (B,))
            wi, wv = O.sample(logits, T, k, p, seed, steps, seed * 3)
            assert np.array_equal(gi, wi), (seed, T, k, p, gi, wi)
            assert_same_bits(gv, wv, "sampled logit")
            if T == 0.0 or k == 1:
                assert gi[0] == 7 and gi[1] == 0 and gi[3] == int(np.argmax(logits[3]))
            else:
                seen.add(int(gi[3]))
    assert len(seen) > 3
    with pytest.raises(R.BunkerCudaError):
        ops.sample(dl.ptr, V, B, idx.ptr, top_k=65)
