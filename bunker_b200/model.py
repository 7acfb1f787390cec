"""Model declaration and decode driver for the hybrid (gated-DeltaNet + gated-attention) decode step.

Mirrors bunker's src/model.ts (dims `D`, tensor names, layer pattern) and src/runner.ts
(`runGraphDecode`): the graph there is a list of per-op nodes launched from TypeScript; here the
same tensor names are registered with the library, which owns the fused kernels and the CUDA
graph, and the host makes one call per token.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Iterable

import numpy as np

from . import runtime as R
from . import synth


@dataclass(frozen=True)
class ModelConfig:
    """Field names follow `D` of src/model.ts:14-18 where one exists."""
    hidden: int            # H
    n_layers: int          # NL
    vocab: int             # VOCAB
    gdn_k_heads: int       # LKH
    gdn_v_heads: int       # LVH
    attn_q_heads: int      # NH
    attn_kv_heads: int     # NKV
    intermediate: int      # INTER
    full_attn_interval: int = 4  # FAI
    head_dim: int = 256    # HD
    rot_dim: int = 64      # ROT_DIM
    max_len: int = 512     # MAX_LEN (the reference fixes 128)
    eps: float = 1e-6      # EPS
    rope_theta: float = 1e7
    name: str = "custom"

    @property
    def conv_width(self) -> int:  # QKVD
        return 2 * self.gdn_k_heads * 128 + self.gdn_v_heads * 128

    @property
    def z_dim(self) -> int:  # ZD
        return self.gdn_v_heads * 128

    @property
    def qgate_dim(self) -> int:  # QGATE
        return self.attn_q_heads * 2 * self.head_dim

    @property
    def kv_dim(self) -> int:  # KV_DIM
        return self.attn_kv_heads * self.head_dim

    def is_full(self, layer: int) -> bool:
        """src/model.ts:61"""
        return layer % self.full_attn_interval == self.full_attn_interval - 1

    def with_(self, **kw) -> "ModelConfig":
        d = dict(self.__dict__)
        d.update(kw)
        return ModelConfig(**d)


# the 24-layer benchmark configuration: hidden 2048, 24 layers [GDN,GDN,GDN,attn]x6, 16/32 GDN heads, 16/2 attention heads,
# FFN 6144, vocabulary 151936, tied embedding
CONFIG_HYBRID_24L = ModelConfig(hidden=2048, n_layers=24, vocab=151936, gdn_k_heads=16, gdn_v_heads=32,
                                attn_q_heads=16, attn_kv_heads=2, intermediate=6144, name="hybrid-24L-2048")
# the scaled 64-layer configuration: hidden 5120, 64 layers, 16/48 GDN heads, 24/4 attention heads, FFN 17408
CONFIG_HYBRID_64L = ModelConfig(hidden=5120, n_layers=64, vocab=151936, gdn_k_heads=16, gdn_v_heads=48,
                                attn_q_heads=24, attn_kv_heads=4, intermediate=17408, max_len=4096,
                                name="hybrid-64L-5120")
# a small model of the same architecture for the parity tests
CONFIG_TINY = ModelConfig(hidden=512, n_layers=4, vocab=4096, gdn_k_heads=2, gdn_v_heads=4, attn_q_heads=4,
                          attn_kv_heads=1, intermediate=1024, max_len=320, name="hybrid-tiny")


def layer_prefix(layer: int) -> str:
    return f"model.layers.{layer}"


def tensor_specs(cfg: ModelConfig) -> list[tuple[str, str, tuple[int, ...]]]:
    """(name, kind, shape) for every weight; kind is "q4k" ([N, K] Q4_K rows), "bf16" or "f32".
    Names are the externals of buildModelGraph (src/model.ts:49-196)."""
    H = cfg.hidden
    out: list[tuple[str, str, tuple[int, ...]]] = [("embed.weight", "q4k", (cfg.vocab, H)),
                                                   ("final.norm.weight", "bf16", (H,))]
    for li in range(cfg.n_layers):
        p = layer_prefix(li)
        out.append((f"{p}.input_layernorm.weight", "bf16", (H,)))
        if not cfg.is_full(li):
            q = f"{p}.linear_attn"
            out += [(f"{q}.in_proj_qkv.weight", "q4k", (cfg.conv_width, H)),
                    (f"{q}.in_proj_z.weight", "q4k", (cfg.z_dim, H)),
                    (f"{q}.in_proj_a.weight", "q4k", (cfg.gdn_v_heads, H)),
                    (f"{q}.in_proj_b.weight", "q4k", (cfg.gdn_v_heads, H)),
                    (f"{q}.conv1d.weight", "bf16", (cfg.conv_width, 4)),
                    (f"{q}.A_log", "f32", (cfg.gdn_v_heads,)),
                    (f"{q}.dt_bias", "bf16", (cfg.gdn_v_heads,)),
                    (f"{q}.norm.weight", "f32", (128,)),
                    (f"{q}.out_proj.weight", "q4k", (H, cfg.z_dim))]
        else:
            q = f"{p}.self_attn"
            out += [(f"{q}.q_proj.weight", "q4k", (cfg.qgate_dim, H)),
                    (f"{q}.k_proj.weight", "q4k", (cfg.kv_dim, H)),
                    (f"{q}.v_proj.weight", "q4k", (cfg.kv_dim, H)),
                    (f"{q}.q_norm.weight", "bf16", (cfg.head_dim,)),
                    (f"{q}.k_norm.weight", "bf16", (cfg.head_dim,)),
                    (f"{q}.o_proj.weight", "q4k", (H, cfg.attn_q_heads * cfg.head_dim))]
        out += [(f"{p}.post_attention_layernorm.weight", "bf16", (H,)),
                (f"{p}.mlp.gate_proj.weight", "q4k", (cfg.intermediate, H)),
                (f"{p}.mlp.up_proj.weight", "q4k", (cfg.intermediate, H)),
                (f"{p}.mlp.down_proj.weight", "q4k", (H, cfg.intermediate))]
    return out


def weight_bytes(cfg: ModelConfig) -> int:
    """Bytes of Q4_K linear weights one decode step streams (each matrix once; the tied table once, as lm_head)."""
    return sum(s[0] * s[1] // 256 * 144 for _, k, s in tensor_specs(cfg) if k == "q4k")


def synth_weights(cfg: ModelConfig, seed: int = 3) -> dict[str, np.ndarray]:
    """Random-init weights: Q4_K drawn as in the GEMV configuration, norm weights bf16 N(0,0.02) under (1+w),
    A_log U(-2,0), dt_bias bf16 N(0,1), GDN norm f32 1+N(0,0.02), conv taps bf16 N(0,0.3)."""
    w: dict[str, np.ndarray] = {}
    for i, (name, kind, shape) in enumerate(tensor_specs(cfg)):
        rng = synth.rng_for(seed, i)
        if kind == "q4k":
            w[name] = synth.q4k_weights(rng, shape[0], shape[1])
        elif name.endswith("A_log"):
            w[name] = rng.uniform(-2.0, 0.0, size=shape).astype(np.float32)
        elif name.endswith("dt_bias"):
            w[name] = synth.normal_bf16(rng, shape, 1.0)
        elif name.endswith("linear_attn.norm.weight"):
            w[name] = (1.0 + rng.normal(0.0, 0.02, size=shape)).astype(np.float32)
        elif name.endswith("conv1d.weight"):
            w[name] = synth.normal_bf16(rng, shape, 0.3)
        else:  # RMSNorm and q/k-norm weights, stored as w with (1+w) applied by the op
            w[name] = synth.normal_bf16(rng, shape, 0.02)
    return w


bkModelConfig = R.bkModelConfig


def split_counts(total: int, n: int) -> list[int]:
    """total items over n ranks, the remainder to the lowest ranks (the rule the library applies to FFN
    superblocks and vocabulary rows)."""
    base, extra = divmod(total, n)
    return [base + (1 if r < extra else 0) for r in range(n)]


def local_dims(cfg: ModelConfig, rank: int, n: int) -> dict:
    """Shard shapes of one tensor-parallel rank (heads per rank, KV heads split or replicated,
    row-parallel K slices in whole superblocks)."""
    assert cfg.gdn_k_heads % n == 0 and cfg.gdn_v_heads % n == 0 and cfg.attn_q_heads % n == 0
    hkv = cfg.attn_kv_heads
    assert hkv % n == 0 or n % hkv == 0
    hq_l = cfg.attn_q_heads // n
    if hkv >= n:
        kv_l, kv0 = hkv // n, rank * (hkv // n)
    else:
        kv_l, kv0 = 1, (rank * hq_l) // (cfg.attn_q_heads // hkv)
    sb = split_counts(cfg.intermediate // 256, n)
    vr = split_counts(cfg.vocab, n)
    return {"Hk": cfg.gdn_k_heads // n, "Hv": cfg.gdn_v_heads // n, "Hq": hq_l, "Hkv": kv_l, "kv0": kv0,
            "inter": sb[rank] * 256, "inter_off": sum(sb[:rank]) * 256, "vocab": vr[rank], "vocab_off": sum(vr[:rank])}


def _q4k_rows(W: np.ndarray, rows) -> np.ndarray:
    return np.ascontiguousarray(W[rows])


def _q4k_kslice(W: np.ndarray, K: int, k0: int, k1: int) -> np.ndarray:
    N = W.shape[0]
    W3 = W.reshape(N, K // 256, 144)
    return np.ascontiguousarray(W3[:, k0 // 256:k1 // 256]).reshape(N, -1)


def shard_plan(cfg: ModelConfig, name: str, rank: int, n: int):
    """How rank `rank` of `n` cuts tensor `name`: ("rows", index array) for column-parallel tensors (qkv/z/a/b rows of
    the rank's key and value heads, q/k/v rows of its query heads and their KV head, gate/up: its FFN rows),
    ("k", k0, k1) for row-parallel ones (out_proj, o_proj, down: all rows, the rank's K range, whole superblocks), None
    for replicated ones (norm weights, the embedding table)."""
    if n == 1:
        return None
    d = local_dims(cfg, rank, n)
    D, HD = 128, cfg.head_dim
    keydim = cfg.gdn_k_heads * D
    hk = np.arange(rank * d["Hk"] * D, (rank + 1) * d["Hk"] * D)
    hv = np.arange(rank * d["Hv"] * D, (rank + 1) * d["Hv"] * D)
    if name.endswith("in_proj_qkv.weight") or name.endswith("conv1d.weight"):
        return ("rows", np.concatenate([hk, keydim + hk, 2 * keydim + hv]))
    if name.endswith("in_proj_z.weight"):
        return ("rows", hv)
    if name.endswith(("in_proj_a.weight", "in_proj_b.weight", "A_log", "dt_bias")):
        return ("rows", np.arange(rank * d["Hv"], (rank + 1) * d["Hv"]))
    if name.endswith("linear_attn.out_proj.weight"):
        return ("k", rank * d["Hv"] * D, (rank + 1) * d["Hv"] * D)
    if name.endswith("q_proj.weight"):
        return ("rows", np.arange(rank * d["Hq"] * 2 * HD, (rank + 1) * d["Hq"] * 2 * HD))
    if name.endswith(("k_proj.weight", "v_proj.weight")):
        return ("rows", np.arange(d["kv0"] * HD, (d["kv0"] + d["Hkv"]) * HD))
    if name.endswith("o_proj.weight"):
        return ("k", rank * d["Hq"] * HD, (rank + 1) * d["Hq"] * HD)
    if name.endswith(("gate_proj.weight", "up_proj.weight")):
        return ("rows", np.arange(d["inter_off"], d["inter_off"] + d["inter"]))
    if name.endswith("down_proj.weight"):
        return ("k", d["inter_off"], d["inter_off"] + d["inter"])
    return None


def shard_weights(cfg: ModelConfig, weights: dict[str, np.ndarray], rank: int, n: int) -> dict[str, np.ndarray]:
    """The tensors rank `rank` of `n` registers, cut from the full (quantised) tensors as shard_plan says."""
    if n == 1:
        return weights
    out: dict[str, np.ndarray] = {}
    for name, kind, shape in tensor_specs(cfg):
        w, plan = weights[name], shard_plan(cfg, name, rank, n)
        if plan is None:
            out[name] = w
        elif plan[0] == "rows":
            out[name] = _q4k_rows(w, plan[1])
        else:
            out[name] = _q4k_kslice(w, shape[1], plan[1], plan[2])
    return out


class DecodeModel:
    """Weights on the device + the library's step graph.  `weights` maps tensor names to numpy arrays."""

    def __init__(self, cfg: ModelConfig, weights: dict[str, np.ndarray], batch: int = 1, device: int = 0,
                 tp_rank: int = 0, tp_size: int = 1, step_mode: int = 0):
        """`weights` holds the FULL tensors; with tp_size > 1 this rank's shard is cut here and the ranks rendezvous
        through bunker_b200.dist (torch.distributed must already be initialised).  step_mode: 0 the library's choice,
        1 one launch per op, 2 the persistent step kernel (bkModelSetStepMode)."""
        self.cfg, self.batch, self.tp_rank, self.tp_size = cfg, batch, tp_rank, tp_size
        lib = R.cu(device)
        specs = tensor_specs(cfg)
        weights = shard_weights(cfg, weights, tp_rank, tp_size)
        self.comm = 0
        if tp_size > 1:
            self._create_comm(lib)
        # one slab, addressed by offset (prototypes/decode.ts:64-75), 256-byte aligned tensors
        offs, total = {}, 0
        for name, _, _ in specs:
            offs[name] = total
            total += (weights[name].nbytes + 255) // 256 * 256
        self.slab = R.DeviceBuffer(total)
        self.offsets = offs
        for name, _, _ in specs:
            a = np.ascontiguousarray(weights[name])
            R.cuHtoD(self.slab.ptr + offs[name], a)
        self._create(lib, {name: (self.slab.ptr + offs[name], weights[name].nbytes) for name, _, _ in specs}, step_mode)


    def _create_comm(self, lib) -> None:
        """Exchange buffer of this rank, exported to and mapped from its peers (CUDA IPC handles through the process group)."""
        from . import dist
        h = C.c_uint64(0)
        R._check(lib.bkCommCreate(self.tp_rank, self.tp_size, self.batch * self.cfg.hidden * 4, C.byref(h)))
        self.comm = h.value
        mine = (C.c_uint8 * 64)()
        R._check(lib.bkCommExportHandle(self.comm, mine))
        allh = b"".join(dist.all_gather_bytes(bytes(mine)))
        R._check(lib.bkCommImportPeers(self.comm, (C.c_uint8 * len(allh)).from_buffer_copy(allh)))

    def _create(self, lib, tensor_ptrs: dict, step_mode: int) -> None:
        """bkModelCreate + one bkModelSetTensor per weight (device pointer, bytes) + bkModelFinalize."""
        cfg, batch, tp_rank, tp_size = self.cfg, self.batch, self.tp_rank, self.tp_size
        c = bkModelConfig(hidden=cfg.hidden, n_layers=cfg.n_layers, full_attn_interval=cfg.full_attn_interval,
                          vocab=cfg.vocab, gdn_k_heads=cfg.gdn_k_heads, gdn_v_heads=cfg.gdn_v_heads,
                          attn_q_heads=cfg.attn_q_heads, attn_kv_heads=cfg.attn_kv_heads, head_dim=cfg.head_dim,
                          rot_dim=cfg.rot_dim, intermediate=cfg.intermediate, max_len=cfg.max_len, batch=batch,
                          tp_rank=tp_rank, tp_size=tp_size, eps=cfg.eps, rope_theta=cfg.rope_theta)
        h = C.c_uint64(0)
        R._check(lib.bkModelCreate(C.byref(c), C.byref(h)))
        self.handle = h.value
        for name, (ptr, nbytes) in tensor_ptrs.items():
            R._check(lib.bkModelSetTensor(self.handle, name.encode(), ptr, nbytes))
        if tp_size > 1:
            from . import dist
            R._check(lib.bkModelSetComm(self.handle, self.comm))
            assert R.cuSync() == 0
            dist.barrier()       # finalize runs one step that exchanges with the peers: enter it together
        if step_mode:
            R._check(lib.bkModelSetStepMode(self.handle, step_mode))
        R._check(lib.bkModelFinalize(self.handle))
        if tp_size > 1:
            dist.barrier()
        self._ids = (C.c_int32 * batch)()
        self._out = (C.c_int32 * batch)()
        self._val = (C.c_float * batch)()

    @classmethod
    def from_device(cls, cfg: ModelConfig, tensor_ptrs: dict, slab, batch: int = 1, device: int = 0,
                    step_mode: int = 0, tp_rank: int = 0, tp_size: int = 1) -> "DecodeModel":
        """A model over weights that already sit in device memory (the loader's path): tensor_ptrs maps every name of
        tensor_specs(cfg) to (device pointer, bytes) of this rank's shard; `slab` is the DeviceBuffer that owns them."""
        self = object.__new__(cls)
        self.cfg, self.batch, self.tp_rank, self.tp_size, self.comm = cfg, batch, tp_rank, tp_size, 0
        lib = R.cu(device)
        if tp_size > 1:
            self._create_comm(lib)
        self.slab = slab
        self.offsets = {n: p - slab.ptr for n, (p, _) in tensor_ptrs.items()}
        self._create(lib, tensor_ptrs, step_mode)
        return self

    def info(self) -> dict:
        sl, w, k, st = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int64()
        R._check(R.cu().bkModelInfo(self.handle, C.byref(sl), C.byref(w), C.byref(k), C.byref(st)))
        return {"split_len": sl.value, "attn_warps": w.value, "kernels_per_step": k.value, "steps": st.value}

    def reset(self) -> None:
        if self.tp_size > 1:
            from . import dist
            assert R.cuSync() == 0
            dist.barrier()
        R._check(R.cu().bkModelReset(self.handle))
        if self.tp_size > 1:
            assert R.cuSync() == 0
            dist.barrier()

    def step(self, tokens: Iterable[int] | None = None, read: bool = True):
        """One token per sequence.  tokens=None feeds back the previous argmax on the device."""
        tp = None
        if tokens is not None:
            for i, t in enumerate(tokens):
                self._ids[i] = int(t)
            tp = self._ids
        if read:
            R._check(R.cu().bkDecodeStep(self.handle, tp, self._out, self._val))
            return np.array(self._out[:], np.int32), np.array(self._val[:], np.float32)
        R._check(R.cu().bkDecodeStep(self.handle, tp, None, None))
        return None

    def step_eager(self) -> None:
        """One step enqueued without the CUDA graph, token fed back on the device (diagnostic timelines apply to it)."""
        R._check(R.cu().bkDecodeStepEager(self.handle))

    def run(self, n_steps: int) -> None:
        R._check(R.cu().bkDecodeRun(self.handle, n_steps))

    def prefill(self, tokens: np.ndarray, read: bool = True, chunk: int | None = None):
        """Prompt tokens [T, batch] in passes of up to 64 // batch tokens (the projections see all their columns at once;
        same state and results as T calls of step()).  Returns (ids, vals) after the last token when read is set."""
        tokens = np.ascontiguousarray(tokens, np.int32).reshape(-1, self.batch)
        per = max(1, 64 // self.batch) if chunk is None else chunk
        out = None
        for t0 in range(0, tokens.shape[0], per):
            part = np.ascontiguousarray(tokens[t0:t0 + per])
            last = t0 + per >= tokens.shape[0]
            R._check(R.cu().bkModelPrefill(self.handle, part.ctypes.data_as(C.POINTER(C.c_int32)), part.shape[0],
                                           self._out if (read and last) else None, self._val if (read and last) else None))
            if read and last:
                out = (np.array(self._out[:], np.int32), np.array(self._val[:], np.float32))
        return out

    PROFILE_CLASSES = ("embed", "gemv_proj", "gdn", "attn", "gemv_out", "gemv_gateup", "gemv_down", "gemv_lmhead",
                       "argmax", "exchange", "quant")

    def step_profiled(self) -> dict[str, tuple[float, int]]:
        """One eager step (device token feedback) with an event pair around every op: {class: (ms, calls)}."""
        n = len(self.PROFILE_CLASSES)
        ms, cnt = (C.c_float * n)(), (C.c_int32 * n)()
        R._check(R.cu().bkDecodeStepProfiled(self.handle, ms, cnt, n))
        return {k: (ms[i], cnt[i]) for i, k in enumerate(self.PROFILE_CLASSES)}

    def tokens(self, first_step: int, n_steps: int) -> np.ndarray:
        out = np.empty((n_steps, self.batch), np.int32)
        R._check(R.cu().bkModelTokens(self.handle, first_step, n_steps, out.ctypes.data_as(C.POINTER(C.c_int32))))
        return out

    def buffer(self, name: str) -> int:
        p = C.c_uint64()
        R._check(R.cu().bkModelBuffer(self.handle, name.encode(), C.byref(p)))
        return p.value

    def logits(self) -> np.ndarray:
        """f32 [B, rows of this rank's lm_head shard] (the whole vocabulary on a single GPU)."""
        out = np.empty((self.batch, local_dims(self.cfg, self.tp_rank, self.tp_size)["vocab"]), np.float32)
        R.cuDtoH(out, self.buffer("logits"))
        return out

    def destroy(self) -> None:
        if self.handle:
            R._check(R.cu().bkModelDestroy(self.handle))
            self.handle = 0
            self.slab.free()
            if self.comm:
                from . import dist
                assert R.cuSync() == 0
                dist.barrier()   # nobody unmaps a buffer a peer may still read
                R._check(R.cu().bkCommDestroy(self.comm))
                self.comm = 0


def runGraphDecode(model: DecodeModel, prompt: np.ndarray, gen_len: int,
                   onToken: Callable[[int, np.ndarray, np.ndarray], None] | None = None) -> np.ndarray:
    """src/runner.ts:116-162.  prompt: int32 [T, B] fed one token at a time through the same step
    (prototypes/decode.ts:952-1061); then gen_len-1 more greedy steps feeding the argmax back.  Every step does
    the host round trip the reference does: token up, (idx, val) down.  Returns generated ids [gen_len, B]."""
    prompt = np.asarray(prompt, np.int32).reshape(len(prompt), -1)
    out = []
    ids = None
    for t in range(prompt.shape[0]):
        ids, val = model.step(prompt[t])
        if onToken:
            onToken(t, ids, val)
    out.append(ids)
    for g in range(1, gen_len):
        ids, val = model.step(ids)
        if onToken:
            onToken(prompt.shape[0] + g - 1, ids, val)
        out.append(ids)
    return np.stack(out)
