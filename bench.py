#!/usr/bin/env python
"""Decode throughput of the 24-layer hybrid Q4_K model (hidden 2048, vocabulary 151,936) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One "step" is one decode step: one token for each of the B sequences through all 24 layers and the
lm_head.  Weights are random-init Q4_K (synthetic), the prompt is 32 random token ids.  The step's
inputs (1.1 GB of weights) exceed L2, so no flush is needed between timed steps.

`value`  : tokens/s over K graph-replayed steps with the token fed back on the device (inputs resident).
`e2e`    : tokens/s over K calls of the per-token API with HOST buffers: token ids copied host->device,
           (id, logit) copied device->host and synchronised every step (the reference's loop, src/runner.ts:133-160).
`roofline`: the dominant kernel (gemv_q4k_kernel) over all its launches inside the step: weight bytes / (step time x
           the GEMV share of a per-op CUDA-event profile); `lm_head_alone` = the same kernel on its largest launch, timed
           back to back between two events.
`batch8`, `batch32`: the resident leg repeated at batch 8 (the metric's second batch size) and, on one GPU, at batch 32
           (the tcgen05 tile path).
`ops`    : stand-alone roofline lines of the GEMV (4096x4096 over rotating weight copies), the GDN step (batch 1, 8) and
           decode attention (cache 1024 / 4096 / 32768 rows, batch 1, 8): median / min / max of 5 timed regions each.
`cpu_baseline` / `--impl reference`: the CPU oracle (C restatement of the reference's op math, OpenMP) on the
           host cores.  The reference is TypeScript for bun with Triton-generated GPU kernels; neither bun
           nor its shim exist here, so kind = "port".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 32
# dram__bytes_read.sum + dram__bytes_write.sum of one lm_head GEMV launch at batch 1, from an ncu capture of that
# launch (two launches of gemv_q4k_kernel, --clock-control none)
NCU_GEMV_LMHEAD_TRAFFIC = 180382976
METRIC = "q4k_hybrid_decode_tok_s"
CPU_SINGLE_THREAD = None   # filled by cpu_tokens_per_s


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs (read-only queries)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_config(steps: int, warmup: int, config: int = 3):
    """configs[3] (24 layers, hidden 2048, 32-token prompt) or configs[4] (64 layers, hidden 5120, FFN 17408,
    2048-token context) -> (model config, prompt length, workload description)"""
    from bunker_b200 import model as M
    if config == 4:
        need = 2048 + warmup + steps + 8
        return (M.CONFIG_HYBRID_64L.with_(max_len=(need + 63) // 64 * 64), 2048,
                "configs[4] scaled hybrid 64-layer Q4_K decode (hidden 5120, FFN 17408, vocab 151936)")
    need = PROMPT_LEN + warmup + steps + 8
    return (M.CONFIG_HYBRID_24L.with_(max_len=(max(need, 320) + 63) // 64 * 64), PROMPT_LEN,
            "configs[3] hybrid 24-layer Q4_K decode (hidden 2048, vocab 151936)")


def oracle_parity(cfg, weights, info, got, prompt, world: int):
    """Rank 0: the first argmax ids of the run (`got`, from the model's own token history) against the CPU oracle with
    its emulation of `world` tensor-parallel ranks and the library's attention split."""
    from oracle import oracle as O
    from oracle.model_oracle import OracleModel
    O.set_threads(os.cpu_count() or 1)
    B, n_steps = prompt.shape[1], got.shape[0]
    om = OracleModel(cfg, weights, batch=B, split_len=info["split_len"], attn_warps=info["attn_warps"], tp=world)
    same = True
    t0 = time.perf_counter()
    for t in range(n_steps):
        ids, _ = om.step(prompt[t])
        same = same and bool(np.array_equal(ids, got[t]))
    return {"steps_checked": n_steps, "identical_tokens": same, "oracle_tp": world, "seconds": round(time.perf_counter() - t0, 1)}


def cpu_tokens_per_s(cfg, weights, batch: int, steps: int, warmup: int, budget_s: float = 150.0):
    """Oracle decode on the host cores.  Runs the full model when K steps fit the budget, else a 1/6 sample
    (4 of 24 layers in the same 3:1 layer mix and 1/6 of the lm_head rows) with the rate scaled by 1/6."""
    from oracle import oracle as O
    from oracle.model_oracle import OracleModel
    # a launcher (torch.distributed.run) exports OMP_NUM_THREADS=1 to its workers: ask for every host core explicitly
    threads = O.set_threads(os.cpu_count() or 1)
    full = f"model.layers.{cfg.n_layers - 1}.mlp.down_proj.weight" in weights
    t_full = float("inf")
    if full:
        om = OracleModel(cfg, weights, batch=batch, split_len=64)
        tok = np.zeros((batch,), np.int32)
        t0 = time.perf_counter()
        om.step(tok)
        t_full = time.perf_counter() - t0
    tok = np.zeros((batch,), np.int32)
    scale, sample = 1.0, "full model, every step one whole token"
    if t_full * (steps + warmup) > budget_s:
        from bunker_b200 import model as M
        small = cfg.with_(n_layers=4, vocab=(cfg.vocab // 6 + 255) // 256 * 256)
        names = {n for n, _, _ in M.tensor_specs(small)}
        w2 = {n: (weights[n][: small.vocab] if n == "embed.weight" else weights[n]) for n in names}
        om = OracleModel(small, w2, batch=batch, split_len=64)
        scale = M.weight_bytes(small) / M.weight_bytes(cfg)
        sample = (f"per step 4 of {cfg.n_layers} layers (3 GDN + 1 attention) and {small.vocab} of {cfg.vocab} lm_head rows "
                  f"= {scale:.4f} of the weight bytes; rate scaled by that factor")
    for _ in range(warmup):
        om.step(tok)
        if om.pos >= om.cfg.max_len - 1:
            om.reset()
    t0 = time.perf_counter()
    for _ in range(steps):
        om.step(tok)
        if om.pos >= om.cfg.max_len - 1:
            om.reset()
    dt = time.perf_counter() - t0
    # the same loops on ONE thread (two steps of the same sample): the scalar port of the reference's host loops
    global CPU_SINGLE_THREAD
    O.set_threads(1)
    t1 = time.perf_counter()
    for _ in range(2):
        om.step(tok)
        if om.pos >= om.cfg.max_len - 1:
            om.reset()
    CPU_SINGLE_THREAD = {"value": 2 * batch / (time.perf_counter() - t1) * scale, "unit": "tok/s", "cores": 1, "steps": 2}
    O.set_threads(threads)
    return steps * batch / dt * scale, dt / steps * 1e3, sample, threads


def run_reference(args):
    """CPU arm: the oracle port on all host cores, same config, metric and unit."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from bunker_b200 import model as M
    cfg, plen, wname = make_config(args.steps, args.warmup, args.config)
    weights = M.synth_weights(cfg.with_(n_layers=4)) if args.config == 4 else M.synth_weights(cfg)   # the sample uses 4 layers
    val, ms, sample, cores = cpu_tokens_per_s(cfg, weights, args.batch, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8xint4->int32, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"{wname}, batch {args.batch}, {plen}-token random prompt then greedy", "batch": args.batch,
                   "parallelism": "cpu", "inputs": "weights larger than L2, no flush", "max_len": cfg.max_len},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample,
                         "single_thread": CPU_SINGLE_THREAD},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference is TypeScript for bun + Triton-generated kernels; bun is absent, so its op math runs as the C port",
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    from bunker_b200 import model as M
    from bunker_b200 import runtime as R

    from bunker_b200 import dist
    K, W, B = args.steps, args.warmup, args.batch
    rank, world = dist.init("nccl") if args.gpus > 1 else (0, 1)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run), found {world}")
    local = dist.env_rank()[2] if world > 1 else 0
    cfg, PLEN, wname = make_config(K, W, args.config)
    weights = M.synth_weights(cfg)        # every layer drawn on its own
    R.cu(local)
    gm = M.DecodeModel(cfg, weights, batch=B, device=local, tp_rank=rank, tp_size=world)
    info = gm.info()
    prompt = np.random.default_rng(0xB0B0 + 1000 * args.config).integers(0, cfg.vocab, (PLEN, B)).astype(np.int32)

    def feed_prompt(read_last: bool = False):
        # a long context goes through the multi-token prompt path where that exists (one GPU, up to 8 sequences);
        # otherwise token by token through the decode step; the last token always takes the decode step
        if PLEN > 64 and world == 1 and B <= 8:
            gm.prefill(prompt[:-1], read=False)
        else:
            for t in range(PLEN - 1):
                gm.step(prompt[t], read=False)
        return gm.step(prompt[-1], read=read_last)

    wbytes = M.weight_bytes(cfg)          # whole model; every rank streams 1/world of it (plus the lm_head shard)
    hbm_peak, peak_src = load_peaks()
    hbm_peak *= world

    # ---- resident leg: prompt, W warm-up steps, K timed graph replays with device-side token feedback ----
    feed_prompt()
    gm.run(W)
    assert R.cuSync() == 0, R.last_error()
    dist.barrier()
    sampler = ClockSampler(local)
    e0, e1 = R.Event(), R.Event()
    l0 = R.launch_count()
    with sampler:
        e0.record()
        gm.run(K)
        e1.record()
        e1.synchronize()
    assert R.cuSync() == 0, R.last_error()
    dist.barrier()
    ms = dist.max_over_ranks(e0.elapsed_ms(e1))
    launches = R.launch_count() - l0
    value = K * B / (ms * 1e-3)
    tokens_resident = gm.tokens(PLEN + W, K)
    # the same region four more times from the same starting state (reset, prompt, warm-up): spread of the measurement
    region_ms = [ms / K]
    for _ in range(4 if args.config == 3 else 1):
        gm.reset()
        feed_prompt()
        gm.run(W)
        assert R.cuSync() == 0, R.last_error()
        dist.barrier()
        r0, r1 = R.Event(), R.Event()
        r0.record()
        gm.run(K)
        r1.record()
        r1.synchronize()
        dist.barrier()
        region_ms.append(dist.max_over_ranks(r0.elapsed_ms(r1)) / K)

    # ---- per-op profile of one eager step (event pair around every launch; launch-bound, shares only) ----
    prof = gm.step_profiled()

    # ---- roofline of the dominant kernel: the GEMV on its largest launch (this rank's lm_head shard, 175 MB at N=1,
    #      larger than L2), back to back on the library stream between two events ----
    from bunker_b200 import ops
    d = M.local_dims(cfg, rank, world)
    H, Vl = cfg.hidden, d["vocab"]
    rowb = H // 256 * 144
    table = gm.slab.ptr + gm.offsets["embed.weight"] + d["vocab_off"] * rowb
    xin = R.DeviceBuffer.from_numpy(np.random.default_rng(1).integers(0, 65535, (B, H)).astype(np.uint16) & 0x3FFF | 0x3C00)
    nw_ptr = gm.slab.ptr + gm.offsets["final.norm.weight"]
    lg = R.DeviceBuffer(B * Vl * 4)
    seg = [ops.gemv_seg(table, Vl, lg.ptr, R.BK_EPI_F32)]
    reps = 20
    for _ in range(3):
        ops.gemv(xin.ptr, H, B, seg, prologue=R.BK_PRO_RMSNORM, norm_w=nw_ptr)
    g0, g1 = R.Event(), R.Event()
    g0.record()
    for _ in range(reps):
        ops.gemv(xin.ptr, H, B, seg, prologue=R.BK_PRO_RMSNORM, norm_w=nw_ptr)
    g1.record()
    g1.synchronize()
    gemv_us = g0.elapsed_ms(g1) * 1e3 / reps
    gemv_bytes = Vl * rowb + B * H * 2 + H * 2 + B * Vl * 4      # Q4_K rows + bf16 x + norm weights + f32 logits
    achieved = gemv_bytes / (gemv_us * 1e-6) / 1e9
    xin.free(), lg.free()

    # ---- end-to-end leg: host token in, host (id, logit) out, every step ----
    gm.reset()
    ids, _ = feed_prompt(read_last=True)
    first_ids = gm.tokens(0, 8) if PLEN <= 64 else None   # checked against the CPU oracle once the GPU legs are done
    for _ in range(W):
        ids, _ = gm.step(ids)
    e2, e3 = R.Event(), R.Event()
    e2.record()
    t0 = time.perf_counter()
    toks = []
    for _ in range(K):
        ids, _ = gm.step(ids)
        toks.append(ids)
    e3.record()
    e3.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = dist.max_over_ranks(max(e2.elapsed_ms(e3), wall_ms))
    same_stream = bool(np.array_equal(np.stack(toks), tokens_resident))

    # ---- the metric's second batch size: the same resident leg at batch 8 (skipped when --batch is given) ----
    def extra_leg(Bx: int, kernel: str):
        """The resident leg repeated at another batch size (same model, same prompt length, K timed graph replays)."""
        nonlocal gm
        gm.destroy()
        gx = M.DecodeModel(cfg, weights, batch=Bx, device=local, tp_rank=rank, tp_size=world)
        px = np.random.default_rng(0xB0B0 + 3000 + Bx).integers(0, cfg.vocab, (PLEN, Bx)).astype(np.int32)
        for t in range(PLEN):
            gx.step(px[t], read=False)
        gx.run(W)
        assert R.cuSync() == 0, R.last_error()
        dist.barrier()
        b0, b1 = R.Event(), R.Event()
        b0.record()
        gx.run(K)
        b1.record()
        b1.synchronize()
        dist.barrier()
        msx = dist.max_over_ranks(b0.elapsed_ms(b1))
        gm = gx
        return {"value": K * Bx / (msx * 1e-3), "unit": "tok/s", "batch": Bx, "ms_per_step": msx / K,
                "frac_of_hbm": wbytes / (msx / K * 1e-3) / 1e9 / hbm_peak,
                "kernels_per_step": gx.info()["kernels_per_step"], "gemv_kernel": kernel}

    # ---- the metric's second batch size (batch 8), and batch 32 on one GPU (the tcgen05 tile path) ----
    batch8 = batch32 = None
    if B == 1 and not args.no_batch8 and args.config == 3:
        batch8 = extra_leg(8, "gemv_q4k_mma_kernel (int8 mma.sync m16n8k32)")
        if world == 1:
            batch32 = extra_leg(32, "gemv_q4k_umma_kernel (tcgen05.mma kind::i8, TMEM accumulators) for launches of 1024+ rows, "
                                    "gemv_q4k_mma_kernel for the rest")
    if rank != 0:
        gm.destroy()
        dist.shutdown()
        return
    parity = oracle_parity(cfg, weights, info, first_ids, prompt, world) if first_ids is not None else None
    if world == 1:
        cpu_val, cpu_ms, cpu_sample, cpu_threads = cpu_tokens_per_s(cfg, weights, B, steps=6, warmup=1, budget_s=30.0)
        cpu = {"value": cpu_val, "unit": "tok/s", "cores": cpu_threads, "kind": "port",
               "sample": cpu_sample + "; 6 timed steps", "ms_per_step": cpu_ms, "single_thread": CPU_SINGLE_THREAD}
    else:
        cpu = None   # reported at N=1 only

    # GEMV over ALL its launches inside the step: the per-op event profile gives the GEMV classes' share of an eagerly
    # launched step, the graph-replayed step time scales it; bytes = every Q4_K weight byte of this rank's shard
    gemv_cls = ("gemv_proj", "gemv_out", "gemv_gateup", "gemv_down", "gemv_lmhead")
    eager_ms = sum(v[0] for v in prof.values())
    gemv_share = sum(prof[k][0] for k in gemv_cls) / eager_ms if eager_ms > 0 else 0.0
    gemv_calls = sum(prof[k][1] for k in gemv_cls)
    step_us = ms / K * 1e3
    gemv_in_step_us = gemv_share * step_us
    wbytes_rank = wbytes / world
    in_step_gbs = wbytes_rank / (gemv_in_step_us * 1e-6) / 1e9 if gemv_in_step_us > 0 else 0.0
    peak1 = hbm_peak / world
    ops_lines = None
    if world == 1 and not args.no_ops and args.config == 3:
        from bunker_b200 import opbench
        ops_lines = opbench.run_all(peak1)

    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K,
        "ms_per_step_regions": {"median": float(np.median(region_ms)), "min": float(min(region_ms)),
                                "max": float(max(region_ms)), "n": len(region_ms),
                                "note": "the timed K-step region repeated from the same state; value uses the first"}, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8xint4->int32, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"{wname}, batch {B}, {PLEN}-token random prompt then greedy", "batch": B,
                   "parallelism": f"tp{world}",
                   "inputs": f"weights ({wbytes / 1e9:.2f} GB/step) larger than L2, no flush", "max_len": cfg.max_len,
                   "attn_split_len": info["split_len"], "kernels_per_step": info["kernels_per_step"]},
        "clocks": sampler.summary(),
        "e2e": {"value": K * B / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 8 * B, "ms_per_step": e2e_ms / K, "same_tokens_as_resident_leg": same_stream,
                "transfer": ("mapped pinned host memory: the embed kernel reads the token, the argmax kernel writes id and logit"
                             if world == 1 else "cudaMemcpyAsync from/to pinned host memory")},
        "gpu_launches": int(launches),
        "parity_vs_oracle": parity,
        "roofline": {"bound": "hbm", "kernel": (f"gemv_q4k_kernel<{B},8>" if B <= 1 else "gemv_q4k_mma_kernel" if B < 16 or world > 1
                                                else "gemv_q4k_umma_kernel (tcgen05 int8, launches of 1024+ rows) + gemv_q4k_mma_kernel"),
                     "achieved": in_step_gbs, "peak": peak1, "unit": "GB/s", "frac": in_step_gbs / peak1,
                     "traffic": (int(wbytes_rank / max(gemv_calls, 1) * NCU_GEMV_LMHEAD_TRAFFIC / 175646208)
                                 if (world == 1 and B == 1) else None),
                     "peak_source": peak_src,
                     "scope": (f"all {gemv_calls} GEMV launches of one decode step: weight bytes / (graph-replayed step time x the "
                               "GEMV classes' share of the per-op CUDA-event profile); traffic = the lm_head capture's "
                               "DRAM bytes scaled by weight bytes"),
                     "avg_launch_us": gemv_in_step_us / max(gemv_calls, 1),
                     "algorithmic_bytes_per_launch": wbytes_rank / max(gemv_calls, 1), "launches_timed": gemv_calls,
                     "gemv_share_of_step": gemv_share,
                     "lm_head_alone": {"achieved": achieved, "frac": achieved / peak1,
                                       "traffic": NCU_GEMV_LMHEAD_TRAFFIC if (world == 1 and B == 1) else None,
                                       "launch": f"lm_head shard [{Vl} x {H}] Q4_K, RMSNorm+Q8_1 prologue, batch {B}, "
                                                 f"{reps} back-to-back launches between two events",
                                       "avg_launch_us": gemv_us, "algorithmic_bytes_per_launch": gemv_bytes}},
        "ops": ops_lines,
        "model_roofline": {"weight_bytes_per_step": wbytes, "achieved_gbs": wbytes / (ms / K * 1e-3) / 1e9,
                           "frac_of_hbm": wbytes / (ms / K * 1e-3) / 1e9 / hbm_peak,
                           "roofline_tok_s": hbm_peak * 1e9 / wbytes * B},
        "per_op_ms": {k: round(v[0], 5) for k, v in prof.items()},
        "per_op_calls": {k: v[1] for k, v in prof.items()},
        "batch8": batch8,
        "batch32": batch32,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    gm.destroy()
    dist.shutdown()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--config", type=int, default=3, choices=[3, 4],
                    help="3: the 24-layer model the metric is quoted on (default); 4: the scaled 64-layer model, 2048-token context")
    ap.add_argument("--no-batch8", action="store_true", help="skip the extra batch-8 and batch-32 legs of the default run")
    ap.add_argument("--no-ops", action="store_true", help="skip the stand-alone per-kernel roofline lines (key `ops`)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
