"""One tensor-parallel rank of the GPU parity test.  Launched by tests/test_gpu_tp.py (or by hand) as
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/tp_worker.py [steps] [batch] [ffn width per rank]
Every rank decodes with the library and compares its tokens and its shard of the logits, bit for bit, with the
CPU oracle emulating the same N ranks."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bunker_b200 import dist  # noqa: E402
from bunker_b200 import model as M  # noqa: E402
from bunker_b200 import runtime as R  # noqa: E402


def main():
    steps = int(sys.argv[1]) if len(sys.argv) > 1 else 40
    B = int(sys.argv[2]) if len(sys.argv) > 2 else 2
    inter_per_rank = int(sys.argv[3]) if len(sys.argv) > 3 else 0   # > 0: FFN width per rank (a K too wide for one
                                                                    # tensor-core launch takes the split-K / column-pair path)
    rank, world = dist.init("nccl")
    local = int(os.environ.get("LOCAL_RANK", rank))
    R.cu(local)
    from oracle.model_oracle import OracleModel
    cfg = M.CONFIG_TINY.with_(gdn_k_heads=max(2, world), gdn_v_heads=2 * max(2, world), attn_q_heads=max(4, world),
                              attn_kv_heads=2 if world <= 2 else 1, max_len=64 + steps,
                              intermediate=(inter_per_rank * world) if inter_per_rank else 256 * max(4, world) + 256,
                              vocab=4099)
    w = M.synth_weights(cfg)
    gm = M.DecodeModel(cfg, w, batch=B, device=local, tp_rank=rank, tp_size=world)
    info = gm.info()
    om = OracleModel(cfg, w, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"], tp=world)
    d = M.local_dims(cfg, rank, world)
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, (8, B)).astype(np.int32)
    ids_g = ids_o = None
    for t in range(8 + steps):
        ids_o, val_o = om.step(prompt[t] if t < 8 else ids_o)
        ids_g, val_g = gm.step(prompt[t] if t < 8 else ids_g)
        assert np.array_equal(ids_g, ids_o), f"rank {rank} step {t}: gpu {ids_g} oracle {ids_o}"
        assert np.array_equal(val_g.view(np.uint32), val_o.view(np.uint32)), f"rank {rank} step {t}: max logit differs"
        if t in (0, 7, 8 + steps - 1):
            mine = om.logits[:, d["vocab_off"]:d["vocab_off"] + d["vocab"]]
            assert np.array_equal(gm.logits().view(np.uint32), np.ascontiguousarray(mine).view(np.uint32)), \
                f"rank {rank} step {t}: logits shard differs"
    # device-feedback run equals the per-token API
    gm.reset()
    for t in range(8):
        gm.step(prompt[t], read=False)
    gm.run(steps)
    assert R.cuSync() == 0, R.last_error()
    hist = gm.tokens(7, steps + 1)
    om.reset()
    want = om.generate(prompt, steps + 1)
    assert np.array_equal(hist, want), f"rank {rank}: device-feedback stream differs"
    gm.destroy()
    dist.barrier()
    if rank == 0:
        print(f"TP{world} OK: {8 + steps} steps, tokens and logits shards identical to the oracle on every rank")
    dist.shutdown()


if __name__ == "__main__":
    main()
