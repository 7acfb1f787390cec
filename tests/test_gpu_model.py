"""Whole-model parity: greedy token streams identical to the CPU oracle for 256 steps, logits bit-exact."""
import numpy as np
import pytest

from bunker_b200 import model as M
from bunker_b200 import runtime as R
from oracle.model_oracle import OracleModel
from tests.util import assert_same_bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B", [1, 3, 8])
def test_tiny_model_256_greedy_steps_match_oracle(bk, B):
    """32-token random prompt then 256 greedy steps (the configs[3] workload on a 4-layer model of the same
    architecture): every generated token and the logits of the first, a middle and the last step are identical."""
    cfg = M.CONFIG_TINY
    w = M.synth_weights(cfg)
    gm = M.DecodeModel(cfg, w, batch=B)
    info = gm.info()
    om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(100 + B).integers(0, cfg.vocab, (32, B)).astype(np.int32)
    checkpoints = {0, 31, 150, 32 + 256 - 2}
    step_no = [0]
    want_ids = []

    def run_oracle(tokens):
        ids, val = om.step(tokens)
        return ids, val

    ids_g = ids_o = None
    for t in range(32 + 256 - 1):
        tok = prompt[t] if t < 32 else ids_o
        ids_o, val_o = run_oracle(tok)
        ids_g, val_g = gm.step(prompt[t] if t < 32 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}: gpu {ids_g} oracle {ids_o}"
        assert_same_bits(val_g, val_o, f"step {t} max logit")
        if t in checkpoints:
            assert_same_bits(gm.logits(), om.logits, f"logits at step {t}")
        want_ids.append(ids_o)
    # the device-side history holds the same stream
    hist = gm.tokens(0, 32 + 256 - 1)
    assert np.array_equal(hist, np.stack(want_ids))
    gm.destroy()


def test_device_feedback_run_matches_host_loop(bk):
    """bkDecodeRun (no host traffic, argmax fed back on the device) produces the stream of the per-token API."""
    cfg = M.CONFIG_TINY
    w = M.synth_weights(cfg, seed=5)
    gm = M.DecodeModel(cfg, w, batch=2)
    prompt = np.random.default_rng(7).integers(0, cfg.vocab, (8, 2)).astype(np.int32)
    a = M.runGraphDecode(gm, prompt, 64)
    gm.reset()
    for t in range(8):
        gm.step(prompt[t], read=False)
    gm.run(63)
    assert R.cuSync() == 0
    b = gm.tokens(7, 64)
    assert np.array_equal(a, b)
    gm.destroy()


def test_model_rejects_missing_tensor(bk):
    import ctypes as C
    cfg = M.CONFIG_TINY
    c = M.bkModelConfig(hidden=cfg.hidden, n_layers=cfg.n_layers, full_attn_interval=4, vocab=cfg.vocab,
                        gdn_k_heads=2, gdn_v_heads=4, attn_q_heads=4, attn_kv_heads=1, head_dim=256, rot_dim=64,
                        intermediate=1024, max_len=64, batch=1, tp_rank=0, tp_size=1, eps=1e-6, rope_theta=1e7)
    h = C.c_uint64()
    lib = R.cu()
    assert lib.bkModelCreate(C.byref(c), C.byref(h)) == 0
    assert lib.bkModelFinalize(h.value) == R.BK_ERR_STATE
    assert "embed.weight" in R.last_error()
    assert lib.bkModelDestroy(h.value) == 0


@pytest.mark.parametrize("mode", [1, 2])
def test_full_size_model_first_steps_match_oracle(bk, mode):
    """configs[3] at full size (24 layers, hidden 2048, vocabulary 151936): 3 prompt tokens + 3 greedy steps
    against the oracle (about 1.1 GB of Q4_K weights per token on the CPU), logits bit-exact; once with one launch
    per op, once with the persistent step kernel."""
    cfg = M.CONFIG_HYBRID_24L.with_(max_len=64)
    w = M.synth_weights(cfg)
    gm = M.DecodeModel(cfg, w, batch=1, step_mode=mode)
    info = gm.info()
    om = OracleModel(cfg, w, batch=1, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, (3, 1)).astype(np.int32)
    ids_g = ids_o = None
    for t in range(6):
        ids_o, val_o = om.step(prompt[t] if t < 3 else ids_o)
        ids_g, val_g = gm.step(prompt[t] if t < 3 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}"
        assert_same_bits(gm.logits(), om.logits, f"logits at step {t}")
    assert np.isfinite(om.logits).all()
    gm.destroy()


def test_full_size_model_256_greedy_steps_match_oracle(bk):
    """The whole configs[3] workload at batch 1: 32-token random prompt, then 256 greedy steps, on the full 24-layer
    model.  Every token must equal the oracle's (the CPU takes about 0.15 s per token), the max logit bit for bit,
    and the full logits at the first generated step and at the end."""
    from oracle import oracle as O
    import os
    O.set_threads(os.cpu_count() or 1)
    P, G = 32, 256
    cfg = M.CONFIG_HYBRID_24L.with_(max_len=P + G + 32)
    w = M.synth_weights(cfg)
    gm = M.DecodeModel(cfg, w, batch=1)
    info = gm.info()
    om = OracleModel(cfg, w, batch=1, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(0xB0B0 + 3000).integers(0, cfg.vocab, (P, 1)).astype(np.int32)
    ids_g = ids_o = None
    min_gap = np.inf
    for t in range(P + G - 1):
        ids_o, val_o = om.step(prompt[t] if t < P else ids_o)
        ids_g, val_g = gm.step(prompt[t] if t < P else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}: gpu {ids_g} oracle {ids_o}"
        assert_same_bits(val_g, val_o, f"step {t} max logit")
        if t in (P - 1, P + G - 2):
            assert_same_bits(gm.logits(), om.logits, f"logits at step {t}")
        top2 = np.partition(om.logits[0], -2)[-2:]
        min_gap = min(min_gap, float(top2[1] - top2[0]))
    print(f"smallest top-1/top-2 logit gap over {P + G - 1} steps: {min_gap:.3e}")
    gm.destroy()


def test_persistent_step_barrier_gives_up_cleanly(bk):
    """The grid barrier of the persistent step kernel with a poll limit of 1: some CTA's first look at the arrival
    counter comes too early, its barrier gives up, sets the status word and the launch winds down by itself (every
    other wait ends as soon as it sees the status).  bkSync must report BK_ERR_TIMEOUT and clear it; afterwards, with
    the limit restored and the state reset, the same model must decode exactly like a fresh one."""
    cfg = M.CONFIG_TINY.with_(max_len=64)
    w = M.synth_weights(cfg, seed=9)
    prompt = np.random.default_rng(2).integers(0, cfg.vocab, (4, 1)).astype(np.int32)
    lib = R.cu()
    gm = M.DecodeModel(cfg, w, batch=1, step_mode=2)
    want = M.runGraphDecode(gm, prompt, 12)
    gm.reset()
    assert R.cuSync() == 0
    R._check(lib.bkSetSpinLimit(1))
    try:
        seen = 0
        for _ in range(20):                      # eager launches pick the limit up; a few steps make the race certain
            gm.step_eager()
            rc = R.cuSync()
            assert rc in (0, R.BK_ERR_TIMEOUT)
            seen += rc == R.BK_ERR_TIMEOUT
        assert seen > 0, "no barrier ran out with a poll limit of 1"
    finally:
        R._check(lib.bkSetSpinLimit(0))
    assert R.cuSync() == 0
    gm.reset()
    got = M.runGraphDecode(gm, prompt, 12)
    assert np.array_equal(got, want)
    gm.destroy()


@pytest.mark.parametrize("B", [9, 12, 32])
def test_tiny_model_more_than_eight_sequences(bk, B):
    """Batch above 8 (column groups of 8 in every projection): 6 prompt tokens + 10 greedy steps, tokens identical to
    the oracle and logits bit-identical at the end."""
    cfg = M.CONFIG_TINY.with_(max_len=32)
    w = M.synth_weights(cfg, seed=20 + B)
    gm = M.DecodeModel(cfg, w, batch=B)
    info = gm.info()
    om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(6).integers(0, cfg.vocab, (6, B)).astype(np.int32)
    ids_g = ids_o = None
    for t in range(16):
        ids_o, _ = om.step(prompt[t] if t < 6 else ids_o)
        ids_g, _ = gm.step(prompt[t] if t < 6 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}"
    assert_same_bits(gm.logits(), om.logits, "logits")
    gm.destroy()


@pytest.mark.parametrize("B", [16, 32, 40])
def test_tiny_model_every_projection_on_the_tile_kernel(bk, B):
    """From 16 sequences on the projections of many rows run on the dense tile kernel.  The small model's launches are
    all below the row threshold except the output projection, so the threshold is lowered to 1 for this model (and
    the oracle told the same): every GEMV of the step then takes the tcgen05 path, with each fused epilogue."""
    cfg = M.CONFIG_TINY.with_(max_len=32)
    w = M.synth_weights(cfg, seed=40 + B)
    assert R.cu().bkTuneTileMinRows(1) == 0
    try:
        gm = M.DecodeModel(cfg, w, batch=B)
        info = gm.info()
        om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"], tile_min_rows=1)
        prompt = np.random.default_rng(8).integers(0, cfg.vocab, (4, B)).astype(np.int32)
        ids_g = ids_o = None
        for t in range(10):
            ids_o, _ = om.step(prompt[t] if t < 4 else ids_o)
            ids_g, _ = gm.step(prompt[t] if t < 4 else ids_g)
            assert np.array_equal(ids_g, ids_o), f"step {t}"
        assert_same_bits(gm.logits(), om.logits, "logits")
        gm.destroy()
    finally:
        R.cu().bkTuneTileMinRows(0)


@pytest.mark.parametrize("B,T,chunk", [(1, 13, None), (1, 20, 9), (2, 11, None), (3, 7, 3), (8, 5, None)])
def test_prefill_equals_token_by_token(bk, B, T, chunk):
    """bkModelPrefill: T prompt tokens in multi-token passes leave the model in the state T single steps leave it in:
    same argmax after the prompt, then 6 greedy steps with identical tokens and bit-identical logits."""
    cfg = M.CONFIG_TINY.with_(max_len=64)
    w = M.synth_weights(cfg, seed=40 + B)
    gm = M.DecodeModel(cfg, w, batch=B)
    info = gm.info()
    om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(T).integers(0, cfg.vocab, (T, B)).astype(np.int32)
    for t in range(T):
        ids_o, val_o = om.step(prompt[t])
    ids_g, val_g = gm.prefill(prompt, chunk=chunk)
    assert np.array_equal(ids_g, ids_o)
    assert_same_bits(val_g, val_o, "max logit after the prompt")
    assert_same_bits(gm.logits(), om.logits, "logits after the prompt")
    for t in range(6):
        ids_o, _ = om.step(ids_o)
        ids_g, _ = gm.step(ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t} after the prompt"
    assert_same_bits(gm.logits(), om.logits, "logits after 6 more steps")
    gm.destroy()


@pytest.mark.parametrize("B,T", [(1, 200), (3, 70)])
def test_long_prefill_across_attention_splits(bk, B, T):
    """Prompt passes whose columns sit on both sides of attention split boundaries (the split length is well below
    the prompt length) and, at batch 3, interleave three sequences: the state after bkModelPrefill equals the state after
    T single decode steps -- same argmax, bit-identical logits, and six identical greedy steps afterwards."""
    cfg = M.CONFIG_TINY.with_(max_len=256)
    w = M.synth_weights(cfg, seed=70 + B)
    prompt = np.random.default_rng(T).integers(0, cfg.vocab, (T, B)).astype(np.int32)
    ga, gb = M.DecodeModel(cfg, w, batch=B), M.DecodeModel(cfg, w, batch=B)
    assert ga.info()["split_len"] < T
    ia, va = ga.prefill(prompt)
    for t in range(T):
        ib, vb = gb.step(prompt[t])
    assert np.array_equal(ia, ib)
    assert_same_bits(va, vb, "max logit after the prompt")
    assert_same_bits(ga.logits(), gb.logits(), "logits after the prompt")
    for t in range(6):
        ia, _ = ga.step(ia)
        ib, _ = gb.step(ib)
        assert np.array_equal(ia, ib), f"step {t} after the prompt"
    assert_same_bits(ga.logits(), gb.logits(), "logits after 6 more steps")
    ga.destroy()
    gb.destroy()


@pytest.mark.parametrize("B", [1, 2])
def test_per_op_runner_equals_step_graph(bk, B):
    """A host that schedules every op itself through cuLaunch (bunker's runner shape) gets the bits of the library's
    fused step graph and of the oracle: 4 prompt tokens + 6 greedy steps, tokens and final logits."""
    from bunker_b200.runner import OpRunner
    cfg = M.CONFIG_TINY.with_(max_len=32)
    w = M.synth_weights(cfg, seed=60 + B)
    gm = M.DecodeModel(cfg, w, batch=B)
    rn = OpRunner(cfg, w, batch=B)
    info = gm.info()
    assert rn.split_len == info["split_len"]
    om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(7).integers(0, cfg.vocab, (4, B)).astype(np.int32)
    ids_g = ids_r = ids_o = None
    for t in range(10):
        ids_o, val_o = om.step(prompt[t] if t < 4 else ids_o)
        ids_g, val_g = gm.step(prompt[t] if t < 4 else ids_g)
        ids_r, val_r = rn.step(prompt[t] if t < 4 else ids_r)
        assert np.array_equal(ids_r, ids_o) and np.array_equal(ids_g, ids_o), f"step {t}"
        assert_same_bits(val_r, val_o, f"max logit at step {t}")
    assert_same_bits(rn.logits_host(), om.logits, "per-op logits vs oracle")
    assert_same_bits(rn.logits_host(), gm.logits(), "per-op logits vs step graph")
    gm.destroy()


def test_scaled_model_shapes_first_steps_match_oracle(bk):
    """configs[4] shapes (hidden 5120, 16/48 GDN heads, 24/4 attention heads of 256, FFN 17408 = 68 superblocks) on a
    4-layer stack with a reduced vocabulary: exercises K = 5120, 6144 and 17408 and group size 6 in attention."""
    cfg = M.CONFIG_HYBRID_64L.with_(n_layers=4, vocab=8192, max_len=64)
    w = M.synth_weights(cfg, seed=11)
    gm = M.DecodeModel(cfg, w, batch=1)
    info = gm.info()
    om = OracleModel(cfg, w, batch=1, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, (3, 1)).astype(np.int32)
    ids_g = ids_o = None
    for t in range(5):
        ids_o, val_o = om.step(prompt[t] if t < 3 else ids_o)
        ids_g, val_g = gm.step(prompt[t] if t < 3 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}"
        assert_same_bits(gm.logits(), om.logits, f"logits at step {t}")
    gm.destroy()


def test_scaled_model_shapes_batch8_tensor_core_path(bk):
    """Same head shapes at batch 8: int8 tensor-core GEMV path for K = 5120 and 6144; the FFN down projection
    (K = 17408) does not fit that path's shared memory and runs as column pairs on the small-batch kernel."""
    cfg = M.CONFIG_HYBRID_64L.with_(n_layers=4, vocab=4096, max_len=32)
    w = M.synth_weights(cfg, seed=12)
    gm = M.DecodeModel(cfg, w, batch=8)
    info = gm.info()
    om = OracleModel(cfg, w, batch=8, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, (2, 8)).astype(np.int32)
    ids_g = ids_o = None
    for t in range(3):
        ids_o, _ = om.step(prompt[t] if t < 2 else ids_o)
        ids_g, _ = gm.step(prompt[t] if t < 2 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}"
    assert_same_bits(gm.logits(), om.logits, "logits")
    gm.destroy()


def test_scaled_model_shapes_batch32_tile_path(bk):
    """Same head shapes at batch 32: the projections of 1024+ rows run on the tcgen05 tile kernel -- K = 5120 (five chunks
    of four superblocks), the down projection with K = 17408 (17 chunks, cut along K over several thread blocks), the
    SwiGLU pair of 2 x 17408 rows with gate and up rows in separate tile halves, weights fed through tensor maps."""
    cfg = M.CONFIG_HYBRID_64L.with_(n_layers=4, vocab=8192, max_len=32)
    w = M.synth_weights(cfg, seed=13)
    B = 32
    gm = M.DecodeModel(cfg, w, batch=B)
    info = gm.info()
    om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"])
    prompt = np.random.default_rng(6).integers(0, cfg.vocab, (2, B)).astype(np.int32)
    ids_g = ids_o = None
    for t in range(4):
        ids_o, _ = om.step(prompt[t] if t < 2 else ids_o)
        ids_g, _ = gm.step(prompt[t] if t < 2 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"step {t}"
    assert_same_bits(gm.logits(), om.logits, "logits")
    gm.destroy()


@pytest.mark.parametrize("interval,n_layers", [(4, 4), (1, 2), (2, 3), (4, 3)])
def test_persistent_step_equals_per_op_step_and_oracle(bk, interval, n_layers):
    """Batch 1 on one GPU can run as a persistent kernel (phases + device-side barriers, step mode 2).  The same model
    stepped with one launch per op must give the same tokens and bit-identical logits, and both match the oracle --
    also when every layer is an attention layer (interval 1) or the model ends on GDN layers."""
    cfg = M.CONFIG_TINY.with_(full_attn_interval=interval, n_layers=n_layers, max_len=96)
    w = M.synth_weights(cfg, seed=40 + interval)
    prompt = np.random.default_rng(interval).integers(0, cfg.vocab, (5, 1)).astype(np.int32)
    outs = {}
    for mode in (1, 2):
        gm = M.DecodeModel(cfg, w, batch=1, step_mode=mode)
        info = gm.info()
        toks = M.runGraphDecode(gm, prompt, 40)
        # device-side feedback through the same graphs
        gm.run(20)
        assert R.cuSync() == 0
        outs[mode] = (toks, gm.tokens(0, 5 + 39 + 20), gm.logits(), info)
        gm.destroy()
    assert outs[2][3]["kernels_per_step"] < outs[1][3]["kernels_per_step"]
    assert np.array_equal(outs[1][0], outs[2][0])
    assert np.array_equal(outs[1][1], outs[2][1])
    assert_same_bits(outs[1][2], outs[2][2], "logits, per-op step vs persistent step")
    om = OracleModel(cfg, w, batch=1, split_len=outs[2][3]["split_len"], attn_warps=outs[2][3]["attn_warps"])
    want = om.generate(prompt, 40)
    assert np.array_equal(outs[2][0], want)


def test_graph_front_end_decodes_like_the_step_graph(bk):
    """A runner.ts-style caller: build the declarative graph, take the static partition, resolve weights and
    double-buffered state through callbacks, rotate the state after every token.  Tokens must equal DecodeModel's and
    the oracle's."""
    from bunker_b200 import graph as G
    cfg = M.CONFIG_TINY.with_(max_len=64)
    w = M.synth_weights(cfg, seed=12)
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, (5, 1)).astype(np.int32)
    g = G.buildModelGraph(cfg)
    comp = G.compileStep(g, G.choosePartition(g))
    store = G.StateStore(g, cfg, w)
    runner = G.GraphRunner(comp, cfg, store.resolve)
    got = G.runGraphDecode(runner, prompt, 20, store.onToken)
    gm = M.DecodeModel(cfg, w, batch=1)
    want = M.runGraphDecode(gm, prompt, 20)
    assert np.array_equal(got, want)
    om = OracleModel(cfg, w, batch=1, split_len=runner.split_len, attn_warps=runner.attn_warps)
    assert np.array_equal(got, om.generate(prompt, 20))
    gm.destroy()
