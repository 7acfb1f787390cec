"""CPU-only, two gloo ranks: the sharding rule and the rank-order sum of the tensor-parallel path.

Each rank cuts its shard with model.shard_weights, computes its partial of a row-parallel GEMV and its slice of a
column-parallel GEMV with the oracle, exchanges the results through bunker_b200.dist, and checks them against the
single-process oracle that emulates the ranks."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank: int, world: int, port: int, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port))
        sys.path.insert(0, ROOT)
        from bunker_b200 import dist
        from bunker_b200 import model as M
        from oracle import oracle as O
        from oracle.model_oracle import OracleModel
        dist.init("gloo")
        cfg = M.CONFIG_TINY
        w = M.synth_weights(cfg)
        sw = M.shard_weights(cfg, w, rank, world)
        d = M.local_dims(cfg, rank, world)
        H, B = cfg.hidden, 2
        rng = np.random.default_rng(9)
        act = O.f32_to_bf16(rng.normal(0, 1, (B, cfg.intermediate)).astype(np.float32))
        # row-parallel down_proj: partial over this rank's K slice
        name = "model.layers.0.mlp.down_proj.weight"
        xs = np.ascontiguousarray(act[:, d["inter_off"]:d["inter_off"] + d["inter"]])
        part = O.gemv_q4k_q8(sw[name], H, d["inter"], O.q8_1_quantize_bf16(xs))
        parts = np.stack([np.frombuffer(b, np.float32).reshape(B, H) for b in dist.all_gather_bytes(part.tobytes())])
        total = O.sum_ranks(parts)
        om = OracleModel(cfg, w, batch=B, split_len=64, tp=world)
        want = om._gemv_rowpar(name, H, cfg.intermediate, act)
        assert np.array_equal(total.view(np.uint32), want.view(np.uint32)), "row-parallel sum differs"
        # column-parallel gate_proj: this rank's rows are a slice of the full result
        x = O.f32_to_bf16(rng.normal(0, 1, (B, H)).astype(np.float32))
        xq = O.q8_1_quantize_bf16(x)
        g_full = O.gemv_q4k_q8(w["model.layers.0.mlp.gate_proj.weight"], cfg.intermediate, H, xq)
        g_mine = O.gemv_q4k_q8(sw["model.layers.0.mlp.gate_proj.weight"], d["inter"], H, xq)
        assert np.array_equal(g_mine, g_full[:, d["inter_off"]:d["inter_off"] + d["inter"]])
        # GDN shard: the rank's q|k|v rows are the rows of its heads
        qkv_full = O.gemv_q4k_q8(w["model.layers.0.linear_attn.in_proj_qkv.weight"], cfg.conv_width, H, xq)
        qkv_mine = O.gemv_q4k_q8(sw["model.layers.0.linear_attn.in_proj_qkv.weight"], 2 * d["Hk"] * 128 + d["Hv"] * 128, H, xq)
        kd = cfg.gdn_k_heads * 128
        sel = np.concatenate([np.arange(rank * d["Hk"] * 128, (rank + 1) * d["Hk"] * 128),
                              kd + np.arange(rank * d["Hk"] * 128, (rank + 1) * d["Hk"] * 128),
                              2 * kd + np.arange(rank * d["Hv"] * 128, (rank + 1) * d["Hv"] * 128)])
        assert np.array_equal(qkv_mine, qkv_full[:, sel])
        assert dist.max_over_ranks(float(rank)) == float(world - 1)
        dist.barrier()
        dist.shutdown()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc() or repr(e)))


def test_two_gloo_ranks_shard_and_sum():
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] == "ok" for r in res), res


def _gate_worker(rank: int, world: int, port: int, q, mode: str):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port))
        sys.path.insert(0, ROOT)
        from bunker_b200 import dist
        dist.init("gloo")
        gate = dist.StepGate()
        steps_done = 0
        try:
            for step in range(8):
                if rank == 1 and step == 3:
                    if mode == "leaves":
                        gate.leave()          # between steps, nothing of this rank in flight
                    break                      # "dies": simply never shows up again
                gate.arrive(step, timeout_s=1.5)
                steps_done += 1                # the device step would be launched here
            q.put((rank, "done", steps_done))
        except dist.PeerLost as e:
            q.put((rank, "peer lost", steps_done, str(e)))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc() or repr(e)))


@pytest.mark.parametrize("mode", ["leaves", "dies"])
def test_rank_gone_between_steps_is_an_error_not_a_hang(mode):
    """Two gloo ranks step through the host-side gate that precedes every tensor-parallel launch.  Rank 1 goes away
    after three steps -- once announcing it, once silently.  Rank 0 must get PeerLost at the gate of step 3 (at once
    when the leave was announced, after the gate's timeout otherwise) having launched exactly three steps."""
    import multiprocessing as mp
    import time
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gate_worker, args=(r, 2, port, q, mode)) for r in range(2)]
    t0 = time.monotonic()
    for p in procs:
        p.start()
    res = {r[0]: r for r in (q.get(timeout=120) for _ in procs)}
    for p in procs:
        p.join(timeout=30)
    assert res[1][1] == "done" and res[1][2] == 3, res
    assert res[0][1] == "peer lost" and res[0][2] == 3, res
    assert ("left before step 3" in res[0][3]) if mode == "leaves" else ("did not reach step 3" in res[0][3]), res
    assert time.monotonic() - t0 < 100


def test_split_rule_uneven():
    sys.path.insert(0, ROOT)
    from bunker_b200 import model as M
    assert M.split_counts(68, 8) == [9, 9, 9, 9, 8, 8, 8, 8]         # FFN 17408 = 68 superblocks over 8 ranks
    c4 = M.CONFIG_HYBRID_64L
    d = [M.local_dims(c4, r, 8) for r in range(8)]
    assert sum(x["inter"] for x in d) == c4.intermediate and d[4]["inter_off"] == 9 * 4 * 256
    assert sum(x["vocab"] for x in d) == c4.vocab
    assert [x["kv0"] for x in d] == [0, 0, 1, 1, 2, 2, 3, 3] and all(x["Hkv"] == 1 for x in d)
