"""Decode throughput of the scaled 64-layer configuration (hidden 5120, FFN 17408, 14.1 GB of Q4_K weights) on one B200.

    python -m bunker_b200.scaled_decode [--batch 1] [--context 2048] [--steps 128]

The context is filled token by token through the decode step itself (graph replays with the token fed back on the
device), then `steps` further steps are timed with CUDA events.  Weights: layers 0-3 are drawn as `synth_weights` draws
them and the other 60 layers reuse those arrays on the host; the device still holds 64 distinct copies, so every step
streams the full 14.1 GB.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np

from . import model as M
from . import runtime as R


def tiled_weights(cfg: M.ModelConfig) -> dict[str, np.ndarray]:
    small = M.synth_weights(cfg.with_(n_layers=4))
    out = {}
    for name, _, _ in M.tensor_specs(cfg):
        if name in small:
            out[name] = small[name]
        else:
            li = int(name.split(".")[2])
            out[name] = small[name.replace(f"layers.{li}.", f"layers.{li % 4}.")]
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=128)
    a = ap.parse_args()
    cfg = M.CONFIG_HYBRID_64L.with_(max_len=(a.context + a.steps + 64 + 63) // 64 * 64)
    t0 = time.time()
    w = tiled_weights(cfg)
    R.cu(0)
    gm = M.DecodeModel(cfg, w, batch=a.batch)
    tok = np.random.default_rng(1).integers(0, cfg.vocab, (a.batch,)).astype(np.int32)
    gm.step(tok, read=False)
    gm.run(a.context - 1)
    assert R.cuSync() == 0, R.last_error()
    e0, e1 = R.Event(), R.Event()
    e0.record()
    gm.run(a.steps)
    e1.record()
    e1.synchronize()
    assert R.cuSync() == 0, R.last_error()
    ms = e0.elapsed_ms(e1) / a.steps
    wb = M.weight_bytes(cfg)
    prof = gm.step_profiled()
    print(json.dumps({
        "workload": f"64-layer hybrid Q4_K decode (hidden 5120, FFN 17408), batch {a.batch}, context {a.context}",
        "tok_s": a.batch / ms * 1e3, "ms_per_step": ms, "steps": a.steps, "weight_bytes_per_step": wb,
        "weight_stream_gbs": wb / ms / 1e6, "kernels_per_step": gm.info()["kernels_per_step"],
        "per_op_ms": {k: round(v[0], 4) for k, v in prof.items()}, "setup_s": round(time.time() - t0, 1)}), flush=True)
    gm.destroy()


if __name__ == "__main__":
    main()
