"""CPU-only: the Q4_K quantiser of the weight loader (oracle side), the checkpoint reader and the name map."""
import os

import numpy as np

from bunker_b200 import loader as L
from bunker_b200 import synth
from oracle import oracle as O


def _grid_block():
    """256 weights that lie exactly on a Q4_K grid: d = 2^-13 with 6-bit scales k_j, dmin = 2^-12 with mins m_j,
    every sub-block using both ends of its 4-bit range -- quantising them must reproduce them exactly."""
    rng = np.random.default_rng(5)
    k = rng.integers(1, 64, 8)
    m = rng.integers(0, 64, 8)
    k[3], m[6] = 63, 63                               # the superblock scales are exactly max/63
    d, dm = np.float32(2.0 ** -13), np.float32(2.0 ** -12)
    q = rng.integers(0, 16, (8, 32))
    q[:, 0], q[:, 1] = 0, 15
    for j in range(8):                                # a sub-block's minimum must be -dmin*m: needs q=0 present (it is)
        pass
    x = (d * k[:, None].astype(np.float32)) * q.astype(np.float32) - (dm * m[:, None].astype(np.float32))
    return x.astype(np.float32).reshape(1, 256), k, m, q


def test_quantiser_reproduces_weights_on_the_grid():
    x, k, m, q = _grid_block()
    blk = O.q4k_quantize(x)
    sc, mn = O.q4k_scales(blk[0])
    assert list(sc) == list(k) and list(mn) == list(m)
    assert blk[0, :2].view(np.float16)[0] == np.float16(2.0 ** -13) and blk[0, 2:4].view(np.float16)[0] == np.float16(2.0 ** -12)
    w = O.q4k_dequant(blk, 1, 256)
    assert np.array_equal(w.view(np.uint32), x.view(np.uint32))
    qs = blk[0, 16:].reshape(4, 32)
    got = np.stack([qs[p] & 15 if (j % 2 == 0) else qs[p] >> 4 for j in range(8) for p in [j // 2]])
    assert np.array_equal(got, q)


def test_quantiser_error_bound_and_edge_blocks():
    rng = np.random.default_rng(6)
    x = rng.normal(0, 0.02, (8, 1024)).astype(np.float32)
    x[0, :256] = 0.0                                  # all-zero superblock
    x[1, :32] = 0.5                                   # constant positive sub-block: lo clamps to 0
    x[2, 256:512] = np.abs(x[2, 256:512])             # all-positive superblock: every min is 0
    w = O.q4k_dequant(O.q4k_quantize(x), 8, 1024)
    xb, wb = x.reshape(8, 32, 32), w.reshape(8, 32, 32)
    rng_b = xb.max(-1) - np.minimum(xb.min(-1), 0)
    # half a quant step, plus the 6-bit rounding of scale and min against the superblock's largest ones
    sup = rng_b.reshape(8, 4, 8).max(-1).repeat(8, -1).reshape(8, 32)
    lo_sup = (-np.minimum(xb.min(-1), 0)).reshape(8, 4, 8).max(-1).repeat(8, -1).reshape(8, 32)
    bound = rng_b / 30 + sup / 15 / 63 * 8 + lo_sup / 63 + 1e-7
    assert (np.abs(wb - xb).max(-1) <= bound).all()
    assert np.array_equal(w[0, :256], np.zeros(256, np.float32))
    assert np.abs(w[1, :32] - 0.5).max() < 0.5 / 15


def test_half_rounding_is_nearest_even():
    import ctypes as C
    f = O.lib().orc_f32_to_f16_rne
    f.restype, f.argtypes = C.c_uint16, [C.c_float]
    vals = np.concatenate([np.random.default_rng(1).normal(0, 1e-3, 2000), [0.0, 6.1e-5, 5.9e-8, 3e-8, 65504.0, 1e-9]]).astype(np.float32)
    for v in vals:
        assert f(float(v)) == np.float16(v).view(np.uint16), v


def test_checkpoint_names_and_file_round_trip(tmp_path):
    present = {"model.language_model.embed_tokens.weight", "model.language_model.norm.weight",
               "model.language_model.layers.3.self_attn.q_proj.weight", "model.layers.0.extra"}
    assert L.safetensors_name("embed.weight", present) == "model.language_model.embed_tokens.weight"
    assert L.safetensors_name("lm_head.weight", present) == "model.language_model.embed_tokens.weight"
    assert L.safetensors_name("final.norm.weight", present) == "model.language_model.norm.weight"
    assert L.safetensors_name("model.layers.3.self_attn.q_proj.weight", present) == \
        "model.language_model.layers.3.self_attn.q_proj.weight"
    assert L.safetensors_name("model.layers.0.extra", present) == "model.layers.0.extra"
    assert L.safetensors_name("model.layers.9.missing", present) is None
    p = os.path.join(tmp_path, "t.safetensors")
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = synth.normal_bf16(np.random.default_rng(0), (5,))
    L.write_safetensors(p, {"a": a, "b": b}, bf16_names={"b"})
    hdr, data0 = L.read_header(p)
    assert hdr["a"] == {"dtype": "F32", "shape": [3, 4], "data_offsets": [0, 48]} and hdr["b"]["dtype"] == "BF16"
    raw = np.fromfile(p, np.uint8)[data0:]
    assert np.array_equal(raw[:48].view(np.float32).reshape(3, 4), a) and np.array_equal(raw[48:58].view(np.uint16), b)


def test_tensor_parallel_cut_commutes_with_quantising():
    """A rank that loads its shard cuts rows / a K range of whole superblocks out of the unquantised tensor and then
    quantises; the result must be the same bytes as cutting the quantised full tensor (model.shard_weights), for every
    linear weight of a small hybrid model, 2 and 4 ranks."""
    from bunker_b200 import model as M
    cfg = M.CONFIG_TINY.with_(n_layers=4, gdn_k_heads=4, gdn_v_heads=8)   # head counts divisible by 4 ranks
    rng = np.random.default_rng(11)
    raw, full_q = {}, {}
    for name, kind, shape in M.tensor_specs(cfg):
        if kind == "q4k" and name != "embed.weight":
            raw[name] = rng.normal(0, 0.05, shape).astype(np.float32)
            full_q[name] = O.q4k_quantize(raw[name])
        else:   # replicated or small tensors: any bytes do; quantised dict entries must exist for shard_weights
            raw[name] = rng.normal(0, 0.05, shape).astype(np.float32)
            full_q[name] = raw[name] if kind != "q4k" else O.q4k_quantize(raw[name])
    for n in (2, 4):
        for rank in range(n):
            want = M.shard_weights(cfg, full_q, rank, n)
            for name, kind, shape in M.tensor_specs(cfg):
                part = L.shard_source(cfg, name, raw[name], rank, n)
                got = O.q4k_quantize(part) if kind == "q4k" else part
                assert got.shape == want[name].shape, (name, n, rank)
                assert np.array_equal(got, want[name]), (name, n, rank)
