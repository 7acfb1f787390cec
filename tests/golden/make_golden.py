"""Writes tests/golden/kat.npz: known-answer vectors for the oracle, derived here WITHOUT the oracle.

Every expected value below comes from a closed form or from a few lines of numpy that restate the data
format (ggml Q4_K superblock description; bunker's packQ8_1 and encodeHalf, bench/bench.ts:41-72), never
from oracle/ code.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kat.npz")
f32 = np.float32
kat = {}

# ---- 1. 6-bit scale/min unpacking: choose sc, mn, pack by the format rule, expect them back ----
rng = np.random.default_rng(1234)
sc = rng.integers(0, 64, (16, 8)).astype(np.uint8)
mn = rng.integers(0, 64, (16, 8)).astype(np.uint8)
sc[0], mn[0] = 63, 63
sc[1], mn[1] = 0, 0
sc[2], mn[2] = np.arange(8) * 9, 63 - np.arange(8) * 9
packed = np.zeros((16, 12), np.uint8)
for j in range(4):
    packed[:, j] = sc[:, j] | ((sc[:, j + 4] >> 4) << 6)
    packed[:, j + 4] = mn[:, j] | ((mn[:, j + 4] >> 4) << 6)
    packed[:, j + 8] = (sc[:, j + 4] & 0xF) | ((mn[:, j + 4] & 0xF) << 4)
kat["scales_packed"], kat["scales_sc"], kat["scales_mn"] = packed, sc, mn

# ---- 2. dequant of hand-built superblocks ----
nsb = 3
sb = np.zeros((nsb, 144), np.uint8)
d = np.array([1.0, 0.5, 2.0 ** -20], np.float16)        # the last one is a subnormal half
dmin = np.array([0.25, 1.5, 2.0 ** -18], np.float16)
q = rng.integers(0, 16, (nsb, 256)).astype(np.uint8)
for s in range(nsb):
    sb[s, 0:2] = d[s:s + 1].view(np.uint8)
    sb[s, 2:4] = dmin[s:s + 1].view(np.uint8)
    sb[s, 4:16] = packed[s]
    for p in range(4):   # 32 bytes serve sub-blocks 2p (low nibbles) and 2p+1 (high nibbles)
        sb[s, 16 + 32 * p: 48 + 32 * p] = q[s, 64 * p: 64 * p + 32] | (q[s, 64 * p + 32: 64 * p + 64] << 4)
want = np.zeros((nsb, 256), f32)
for s in range(nsb):
    for j in range(8):
        dl = f32(d[s]) * f32(sc[s, j])
        ml = f32(dmin[s]) * f32(mn[s, j])
        want[s, 32 * j: 32 * j + 32] = dl * q[s, 32 * j: 32 * j + 32].astype(f32) - ml
kat["dequant_row"], kat["dequant_want"] = sb.reshape(-1), want.reshape(-1)

# ---- 3. f16 truncating encode (bench/bench.ts:41-51) and flush decode ----
vals = np.array([0.0, 1.0, -2.5, 0.1, 65504.0, 70000.0, 6e-5, 6.2e-5, -1e-7, 0.33333334, 1.0009765], f32)
enc = []
for v in vals:
    if v == 0:
        enc.append(0)
        continue
    bits = int(np.array([v], f32).view(np.uint32)[0])
    s_, e_, m_ = (bits >> 16) & 0x8000, (bits >> 23) & 0xFF, bits & 0x7FFFFF
    ne = e_ - 127 + 15
    enc.append(s_ | 0x7C00 if ne >= 31 else (s_ if ne <= 0 else s_ | (ne << 10) | (m_ >> 13)))
kat["f16_trunc_in"], kat["f16_trunc_want"] = vals, np.array(enc, np.uint16)

# ---- 4. bf16 round-to-nearest-even, including exact ties ----
bits_in = np.array([0x3F800000, 0x3F808000, 0x3F818000, 0x3F808001, 0x3F807FFF, 0xBF808000, 0x7F7FFFFF, 0x00008000,
                    0x477FE000], np.uint32)
bits_out = np.array([0x3F80, 0x3F80, 0x3F82, 0x3F81, 0x3F80, 0xBF80, 0x7F80, 0x0000, 0x4780], np.uint16)
kat["bf16_in"], kat["bf16_want"] = bits_in.view(f32), bits_out

# ---- 5. Q8_1 blocks (packQ8_1, bench/bench.ts:53-72 with the reciprocal form) ----
x = np.zeros(96, f32)
x[0:32] = np.arange(32, dtype=f32) - 16          # amax 16 -> d = 16/127
x[32:64] = 0.0                                    # zero block
x[64:96] = np.linspace(-1, 1, 32).astype(f32) * 127  # amax 127 -> d = 1
blocks = np.zeros((3, 36), np.uint8)
for b in range(3):
    xb = x[32 * b: 32 * b + 32]
    amax = f32(np.abs(xb).max())
    dd = f32(amax / f32(127))
    idd = f32(1) if dd == 0 else f32(f32(1) / dd)
    # fma(x, 1/d, 0.5) in one rounding == round of the exact value; float64 holds x*id exactly enough here
    qv = np.floor((xb.astype(np.float64) * np.float64(idd) + 0.5).astype(f32)).astype(np.int64)
    ssum = int(qv.sum())
    qv = np.clip(qv, -128, 127)
    blocks[b, :32] = qv.astype(np.int8).view(np.uint8)

    def enc_half(v):
        if v == 0:
            return 0
        bits = int(np.array([v], f32).view(np.uint32)[0])
        s_, e_, m_ = (bits >> 16) & 0x8000, (bits >> 23) & 0xFF, bits & 0x7FFFFF
        ne = e_ - 127 + 15
        return s_ | 0x7C00 if ne >= 31 else (s_ if ne <= 0 else s_ | (ne << 10) | (m_ >> 13))
    hd, hs = enc_half(dd), enc_half(f32(f32(ssum) * dd))
    blocks[b, 32:36] = [hd & 0xFF, hd >> 8, hs & 0xFF, hs >> 8]
kat["q8_in"], kat["q8_want"] = x, blocks

# ---- 6. GEMV closed forms ----
# (a) all nibbles 1, scales 1, mins 0, d=1, dmin=0, q8 = small ints with d8 = 1  ->  y = sum(q8) exactly
K = 512
row = np.zeros((K // 256, 144), np.uint8)
row[:, 0:2] = np.array([1.0], np.float16).view(np.uint8)
one_sc = np.ones(8, np.uint8)
zero_mn = np.zeros(8, np.uint8)
pk = np.zeros(12, np.uint8)
for j in range(4):
    pk[j] = one_sc[j] | ((one_sc[j + 4] >> 4) << 6)
    pk[j + 4] = zero_mn[j]
    pk[j + 8] = one_sc[j + 4] & 0xF
row[:, 4:16] = pk
row[:, 16:] = 0x11
xq = np.zeros((K // 32, 36), np.uint8)
q8 = rng.integers(-20, 21, (K // 32, 32)).astype(np.int8)
xq[:, :32] = q8.view(np.uint8)
xq[:, 32:34] = np.array([1.0], np.float16).view(np.uint8)
kat["gemv_a_row"], kat["gemv_a_xq"], kat["gemv_a_want"] = row.reshape(-1), xq.reshape(-1), f32(q8.astype(np.int64).sum())
# (b) same weights but dmin = 2, mins = 3  ->  y = sum(q8) - 2*3*sum(q8) = -5*sum(q8)
row_b = row.copy()
row_b[:, 2:4] = np.array([2.0], np.float16).view(np.uint8)
three = np.full(8, 3, np.uint8)
pk_b = pk.copy()
for j in range(4):
    pk_b[j + 4] = three[j] | ((three[j + 4] >> 4) << 6)
    pk_b[j + 8] = (one_sc[j + 4] & 0xF) | ((three[j + 4] & 0xF) << 4)
row_b[:, 4:16] = pk_b
kat["gemv_b_row"], kat["gemv_b_want"] = row_b.reshape(-1), f32(-5 * q8.astype(np.int64).sum())

# ---- 7. argmax ties ----
lg = np.full((2, 1000), -1.0, f32)
lg[0, [7, 400, 999]] = 3.0
lg[1, 999] = 0.5
kat["argmax_in"], kat["argmax_idx"], kat["argmax_val"] = lg, np.array([7, 999], np.int32), np.array([3.0, 0.5], f32)

# ---- 8. GDN with zero state: S' = k_n (outer) (v*beta), o = (q_n.k_n) * v*beta ----
D = 128
qv = np.zeros(D, f32); kv = np.zeros(D, f32)
qv[3] = 2.0                                    # q_n = e3 / sqrt(128) (up to the 1e-6 in the norm)
kv[3] = 4.0                                    # k_n = e3
vv = (np.arange(D, dtype=f32) - 64) / 8
kat["gdn_q"], kat["gdn_k"], kat["gdn_v"] = qv, kv, vv
kat["gdn_beta_logit"], kat["gdn_a"] = f32(0.0), f32(0.0)   # beta = 0.5; decay irrelevant for S = 0
kat["gdn_o_want"] = (vv * 0.5 / np.sqrt(128.0)).astype(f32)   # to ~1e-6 relative
kat["gdn_S33_want"] = (vv * 0.5).astype(f32)                  # row 3 of S'

# ---- 9. attention with identical keys: softmax is uniform, o = mean of V ----
n, HD = 40, 256
krow = rng.normal(0, 1, HD).astype(f32)
V = rng.normal(0, 1, (n, HD)).astype(f32)
kat["attn_k"], kat["attn_V"], kat["attn_q"] = krow, V, rng.normal(0, 1, HD).astype(f32)

# ---- 10. RoPE: pos 0 is the identity; at pos p pair (i, i+32) rotates by p*theta^(-2i/64) ----
kat["rope_theta"] = np.float64(1e7)
i = np.arange(32)
kat["rope_cos_p5"] = np.cos(5 * (1.0 / np.power(1e7, 2.0 * i / 64))).astype(f32)
kat["rope_sin_p5"] = np.sin(5 * (1.0 / np.power(1e7, 2.0 * i / 64))).astype(f32)

np.savez_compressed(OUT, **kat)
print("wrote", OUT, {k: getattr(v, "shape", ()) for k, v in kat.items()})
