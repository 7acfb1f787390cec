"""Stand-alone timings of the three hot kernels on the shapes they are specified on, against the HBM roofline.

Each function times one kernel with CUDA events on the library stream: `reps` timed regions of `n` back-to-back
launches after a warm-up, and reports median / min / max of the per-launch time.  Inputs that would fit the 126 MB
L2 are rotated over enough distinct copies (weights, recurrent state, KV cache) that every launch reads its bytes
from HBM.  `bytes` is the algorithmic traffic of one launch (what the op must move, not what it happens to move):

  GEMV       N*K*144/256 weight bytes + the Q8_1 activation + the f32 result        (4096 x 4096: 9,458,176 B)
  GDN step   per sequence: state read + write, conv state read + write, qkv, z, out  (4,325,376 B)
  attention  per sequence: K and V rows 0..L-1 (L * 2048 B) + q, gate, out

Used by bench.py; runnable by hand:  python -m bunker_b200.opbench
"""
from __future__ import annotations

import json

import numpy as np

from . import ops, synth
from . import runtime as R

L2_BYTES = 126 * 1024 * 1024


def _stats(us: list[float], nbytes: int, peak_gbs: float) -> dict:
    med = float(np.median(us))
    return {"us": med, "us_min": float(min(us)), "us_max": float(max(us)), "bytes": int(nbytes),
            "gbs": nbytes / (med * 1e-6) / 1e9, "frac": nbytes / (med * 1e-6) / 1e9 / peak_gbs, "regions": len(us)}


def _time(launch, n: int, reps: int, warm: int = 3) -> list[float]:
    """launch(i) enqueues launch number i.  Returns the per-launch time (us) of each of `reps` regions of n launches."""
    for i in range(warm * n):
        launch(i)
    assert R.cuSync() == 0, R.last_error()
    out = []
    for _ in range(reps):
        e0, e1 = R.Event(), R.Event()
        e0.record()
        for i in range(n):
            launch(i)
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_ms(e1) * 1e3 / n)
    assert R.cuSync() == 0, R.last_error()
    return out


def _copies(per_copy: int, cap: int = 96) -> int:
    """distinct copies needed for the rotation to exceed L2 with some margin"""
    return int(max(2, min(cap, -(-int(1.3 * L2_BYTES) // max(per_copy, 1)))))


def _replicate(host: np.ndarray, copies: int) -> list[R.DeviceBuffer]:
    first = R.DeviceBuffer.from_numpy(host)
    bufs = [first]
    for _ in range(copies - 1):
        b = R.DeviceBuffer(first.nbytes)
        R._check(R.cu().bkDtoD(b.ptr, first.ptr, first.nbytes))
        bufs.append(b)
    return bufs


def bench_gemv_q4k(peak_gbs: float, N: int = 4096, K: int = 4096, B: int = 1, reps: int = 5, n: int = 64) -> dict:
    """The single dequant-GEMV configuration: W [N][K] Q4_K, x Q8_1 (quantised by the library), y f32."""
    W, x = synth.gemv_case(N, K, B)
    wcopies = _replicate(W, _copies(W.nbytes))
    dx = R.DeviceBuffer.from_numpy(x)
    xq = R.DeviceBuffer(B * K // 32 * 36)
    ops.quant_q8_1(dx.ptr, K, B, xq.ptr)
    y = R.DeviceBuffer(B * N * 4)
    us = _time(lambda i: ops.gemv_simple(wcopies[i % len(wcopies)].ptr, N, K, xq.ptr, B, y.ptr), n, reps)
    nbytes = W.nbytes + B * K // 32 * 36 + B * N * 4
    for b in wcopies + [dx, xq, y]:
        b.free()
    r = _stats(us, nbytes, peak_gbs)
    r.update({"shape": f"W {N}x{K} Q4_K, batch {B}", "weight_copies": len(wcopies), "launches_per_region": n})
    return r


def bench_gdn(peak_gbs: float, B: int = 1, reps: int = 5, n: int = 64) -> dict:
    """One conv1d + gated-DeltaNet step: 16 key heads, 32 value heads, d = 128, conv width 8192."""
    c = synth.gdn_case(B)
    Hk, Hv = c["Hk"], c["Hv"]
    Cw = 2 * Hk * 128 + Hv * 128
    scopies = _replicate(c["S"], _copies(2 * c["S"].nbytes))
    cs_a = _replicate(c["conv_state"], len(scopies))
    cs_b = _replicate(c["conv_state"], len(scopies))
    d = {k: R.DeviceBuffer.from_numpy(v) for k, v in c.items() if isinstance(v, np.ndarray) and k not in ("S", "conv_state")}
    out = R.DeviceBuffer(B * Hv * 128 * 2)

    def launch(i):
        j = i % len(scopies)
        ops.gdn_step(qkv=d["qkv"].ptr, z=d["z"].ptr, a=d["a"].ptr, b=d["b"].ptr, conv_w=d["conv_w"].ptr,
                     conv_state_in=cs_a[j].ptr, conv_state_new=cs_b[j].ptr, A_log=d["A_log"].ptr, dt_bias=d["dt_bias"].ptr,
                     norm_w=d["norm_w"].ptr, S_in=scopies[j].ptr, S_new=scopies[j].ptr, out=out.ptr, B=B, Hk=Hk, Hv=Hv,
                     apply_conv=1, state_is_settled=1)

    us = _time(launch, n, reps)
    per_seq = 2 * Hv * 128 * 128 * 4 + 2 * 3 * Cw * 2 + Cw * 2 + 2 * Hv * 128 * 2
    nbytes = B * per_seq + Cw * 4 * 2
    for b in scopies + cs_a + cs_b + list(d.values()) + [out]:
        b.free()
    r = _stats(us, nbytes, peak_gbs)
    r.update({"shape": f"batch {B}, {Hk} key / {Hv} value heads, d 128", "state_copies": len(scopies), "launches_per_region": n})
    return r


def bench_attn(peak_gbs: float, B: int, L: int, reps: int = 5, n: int | None = None) -> dict:
    """Split-KV decode attention over a cache of L rows: 16 query heads, 2 KV heads, head_dim 256."""
    Hq, Hkv, HD = 16, 2, 256
    rng = synth.rng_for(2, 40)
    kv_bytes = B * Hkv * L * HD * 2
    copies = _copies(2 * kv_bytes, cap=64)
    # the cache content does not matter for the timing: one block of bf16 N(0,1) rows tiled over the cache
    tile_rows = min(L, 2048)
    tile = synth.normal_bf16(rng, (tile_rows, HD))
    dt = R.DeviceBuffer.from_numpy(tile)

    def make_cache():
        buf = R.DeviceBuffer(kv_bytes)
        off = 0
        while off < kv_bytes:
            nb = min(dt.nbytes, kv_bytes - off)
            R._check(R.cu().bkDtoD(buf.ptr + off, dt.ptr, nb))
            off += nb
        return buf

    kcs, vcs = [make_cache() for _ in range(copies)], [make_cache() for _ in range(copies)]
    qg = R.DeviceBuffer.from_numpy(synth.normal_bf16(rng, (B, Hq * 2 * HD)))
    k = R.DeviceBuffer.from_numpy(synth.normal_bf16(rng, (B, Hkv * HD)))
    v = R.DeviceBuffer.from_numpy(synth.normal_bf16(rng, (B, Hkv * HD)))
    qn = R.DeviceBuffer.from_numpy(synth.normal_bf16(rng, (HD,), 0.02))
    kn = R.DeviceBuffer.from_numpy(synth.normal_bf16(rng, (HD,), 0.02))
    cos_t, sin_t = ops.rope_tables(L)
    dc, ds = R.DeviceBuffer.from_numpy(cos_t), R.DeviceBuffer.from_numpy(sin_t)
    pos = R.DeviceBuffer.from_numpy(np.full((B,), L - 1, np.int32))
    split_len, _ = ops.attn_plan(L, B, Hkv)
    scratch = R.DeviceBuffer.zeros(ops.attn_scratch_bytes(B, Hq, HD, L, split_len))
    out = R.DeviceBuffer(B * Hq * HD * 2)
    if n is None:
        n = 64 if kv_bytes < (64 << 20) else 16

    def launch(i):
        j = i % copies
        ops.attn_decode(qg=qg.ptr, k=k.ptr, v=v.ptr, q_norm_w=qn.ptr, k_norm_w=kn.ptr, cos_t=dc.ptr, sin_t=ds.ptr,
                        k_cache=kcs[j].ptr, v_cache=vcs[j].ptr, pos=pos.ptr, out=out.ptr, scratch=scratch.ptr, B=B, Hq=Hq,
                        Hkv=Hkv, HD=HD, rot_half=32, max_len=L, split_len=split_len, max_pos=L - 1, scale=1.0 / 16.0,
                        fused_norm_rope=1, cache_is_settled=1)

    us = _time(launch, n, reps)
    nbytes = B * (2 * Hkv * L * HD * 2 + Hq * 2 * HD * 2 + Hq * HD * 2)
    for b in kcs + vcs + [qg, k, v, qn, kn, dc, ds, pos, scratch, out, dt]:
        b.free()
    r = _stats(us, nbytes, peak_gbs)
    r.update({"shape": f"batch {B}, cache {L} rows, 16 q / 2 kv heads, head_dim 256", "split_len": split_len,
              "cache_copies": copies, "launches_per_region": n})
    return r


def run_all(peak_gbs: float, reps: int = 5) -> dict:
    res = {"gemv_4096x4096_b1": bench_gemv_q4k(peak_gbs, reps=reps)}
    for B in (1, 8):
        res[f"gdn_step_b{B}"] = bench_gdn(peak_gbs, B, reps=reps)
    for L in (1024, 4096, 32768):
        for B in (1, 8):
            res[f"attn_L{L}_b{B}"] = bench_attn(peak_gbs, B, L, reps=reps)
    return res


if __name__ == "__main__":
    import argparse
    import os
    ap = argparse.ArgumentParser(description="stand-alone roofline timings of the GEMV, GDN-step and decode-attention kernels")
    ap.add_argument("--op", default="all", choices=["all", "gemv", "gdn", "attn"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--rows", type=int, default=32768, help="attention: cache rows")
    ap.add_argument("--reps", type=int, default=5, help="timed regions")
    ap.add_argument("--n", type=int, default=0, help="launches per region (0: the default of the op)")
    a = ap.parse_args()
    peak = 6650.0
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = float(json.load(open(p))["hbm_gbs"])
    R.cu(0)
    kw = {"reps": a.reps, **({"n": a.n} if a.n else {})}
    if a.op == "all":
        res = run_all(peak, reps=a.reps)
    elif a.op == "gemv":
        res = {f"gemv_4096x4096_b{a.batch}": bench_gemv_q4k(peak, B=a.batch, **kw)}
    elif a.op == "gdn":
        res = {f"gdn_step_b{a.batch}": bench_gdn(peak, a.batch, **kw)}
    else:
        res = {f"attn_L{a.rows}_b{a.batch}": bench_attn(peak, a.batch, a.rows, **kw)}
    for k, v in res.items():
        print(k, json.dumps(v))
