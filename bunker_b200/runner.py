"""Per-op decode driver: the shape of bunker's runner (src/runner.ts:133-160 over the graph of src/model.ts:49-196) on
top of the cuLaunch surface -- every op of a decode step is one `cuLaunch(loadOp(name), ...)` with 8-byte slots, buffers
come from `cuAlloc`, positions and the conv-state parity are kept by the host.

It exists to show (and test) that a host which schedules ops itself can drop the library in op by op; the fast path is
`DecodeModel` (whole step in a CUDA graph inside the library).  Both produce the same bits: the fused prologues and
epilogues of the step path are the compositions of the ops launched here.
"""
from __future__ import annotations

import numpy as np

from . import ops
from . import runtime as R
from .model import ModelConfig, layer_prefix, tensor_specs
from .runtime import BK_EPI_ADD_BF16, BK_EPI_BF16, BK_EPI_F32, BK_EPI_SWIGLU, cuAlloc, cuHtoD, cuLaunch, loadOp

_G, _B = [1, 1, 1], [1, 1, 1]   # grid/block are accepted for signature parity and ignored


class OpRunner:
    def __init__(self, cfg: ModelConfig, weights: dict[str, np.ndarray], batch: int = 1):
        self.cfg, self.B = cfg, batch
        R.cu()
        self.w = {}
        for name, _, _ in tensor_specs(cfg):
            a = np.ascontiguousarray(weights[name])
            p = cuAlloc(a.nbytes)
            cuHtoD(p, a)
            self.w[name] = p
        B, H = batch, cfg.hidden
        Cw, ZD, Hv = cfg.conv_width, cfg.z_dim, cfg.gdn_v_heads
        QG, KVD, AW = cfg.qgate_dim, cfg.kv_dim, cfg.attn_q_heads * cfg.head_dim
        z = lambda n: R.DeviceBuffer.zeros(n)   # noqa: E731
        self.x = [z(B * H * 2), z(B * H * 2)]
        self.xn, self.h1 = z(B * H * 2), z(B * H * 2)
        kmax = max(H, cfg.intermediate, ZD, AW)
        self.xq = z(B * kmax // 32 * 36)
        self.qkv, self.z, self.a, self.b = z(B * Cw * 2), z(B * ZD * 2), z(B * Hv * 4), z(B * Hv * 4)
        self.attn_out = z(B * max(ZD, AW) * 2)
        self.qg, self.k, self.v = z(B * QG * 2), z(B * KVD * 2), z(B * KVD * 2)
        self.act = z(B * cfg.intermediate * 2)
        self.logits = z(B * cfg.vocab * 4)
        self.ids, self.val, self.pos_dev = z(B * 4), z(B * 4), z(B * 4)
        self.argmax_scratch = z(ops.argmax_scratch_bytes(B))
        self.split_len, _ = ops.attn_plan(cfg.max_len, B, cfg.attn_kv_heads)
        self.attn_scratch = z(ops.attn_scratch_bytes(B, cfg.attn_q_heads, cfg.head_dim, cfg.max_len, self.split_len))
        cos_t, sin_t = ops.rope_tables(cfg.max_len, cfg.rot_dim, cfg.rope_theta)
        self.cos_t, self.sin_t = R.DeviceBuffer.from_numpy(cos_t), R.DeviceBuffer.from_numpy(sin_t)
        self.state = []
        for li in range(cfg.n_layers):
            if cfg.is_full(li):
                kv = B * cfg.attn_kv_heads * cfg.max_len * cfg.head_dim * 2
                self.state.append({"kc": z(kv), "vc": z(kv)})
            else:
                self.state.append({"conv": [z(B * 3 * Cw * 2), z(B * 3 * Cw * 2)], "S": z(B * Hv * 128 * 128 * 4)})
        self.pos = 0
        self.k_ops = {n: loadOp(n) for n in ("embed", "rmsnorm", "gemm", "quant_q8_1_bf16", "gdn_delta_rule", "fa2_attn", "argmax")}

    def _launch(self, name: str, args) -> None:
        rc = cuLaunch(self.k_ops[name], _G, _B, args)
        if rc != 0:
            raise R.BunkerCudaError(rc, f"{name}: {R.last_error()}")

    def _norm_quant(self, x: int, w: int, K: int) -> None:
        self._launch("rmsnorm", [x, w, self.xn.ptr, K, self.B, float(self.cfg.eps)])
        self._launch("quant_q8_1_bf16", [self.xn.ptr, self.xq.ptr, K, self.B])

    def _gemm(self, W: int, out: int, N: int, K: int, epi: int, residual: int = 0, W2: int = 0) -> None:
        self._launch("gemm", [self.xq.ptr, W, out, N, K, self.B, epi, residual, W2])

    def step(self, tokens: np.ndarray):
        cfg, B, H = self.cfg, self.B, self.cfg.hidden
        w = self.w
        ids = np.ascontiguousarray(tokens, np.int32).reshape(B)
        cuHtoD(self.ids.ptr, ids)
        cuHtoD(self.pos_dev.ptr, np.full((B,), self.pos, np.int32))
        self._launch("embed", [w["embed.weight"], self.x[0].ptr, self.ids.ptr, H, B])
        cur = 0
        par = self.pos & 1
        for li in range(cfg.n_layers):
            p, st, x = layer_prefix(li), self.state[li], self.x[cur].ptr
            self._norm_quant(x, w[f"{p}.input_layernorm.weight"], H)
            if not cfg.is_full(li):
                q = f"{p}.linear_attn"
                self._gemm(w[f"{q}.in_proj_qkv.weight"], self.qkv.ptr, cfg.conv_width, H, BK_EPI_BF16)
                self._gemm(w[f"{q}.in_proj_z.weight"], self.z.ptr, cfg.z_dim, H, BK_EPI_BF16)
                self._gemm(w[f"{q}.in_proj_a.weight"], self.a.ptr, cfg.gdn_v_heads, H, BK_EPI_F32)
                self._gemm(w[f"{q}.in_proj_b.weight"], self.b.ptr, cfg.gdn_v_heads, H, BK_EPI_F32)
                self._launch("gdn_delta_rule", [self.qkv.ptr, self.z.ptr, self.a.ptr, self.b.ptr, w[f"{q}.conv1d.weight"],
                                                st["conv"][par].ptr, st["conv"][par ^ 1].ptr, w[f"{q}.A_log"], w[f"{q}.dt_bias"],
                                                w[f"{q}.norm.weight"], st["S"].ptr, st["S"].ptr, self.attn_out.ptr, B,
                                                cfg.gdn_k_heads, cfg.gdn_v_heads, 1, 0])
                self._launch("quant_q8_1_bf16", [self.attn_out.ptr, self.xq.ptr, cfg.z_dim, B])
                self._gemm(w[f"{q}.out_proj.weight"], self.h1.ptr, H, cfg.z_dim, BK_EPI_ADD_BF16, residual=x)
            else:
                q = f"{p}.self_attn"
                aw = cfg.attn_q_heads * cfg.head_dim
                self._gemm(w[f"{q}.q_proj.weight"], self.qg.ptr, cfg.qgate_dim, H, BK_EPI_BF16)
                self._gemm(w[f"{q}.k_proj.weight"], self.k.ptr, cfg.kv_dim, H, BK_EPI_BF16)
                self._gemm(w[f"{q}.v_proj.weight"], self.v.ptr, cfg.kv_dim, H, BK_EPI_BF16)
                self._launch("fa2_attn", [self.qg.ptr, self.k.ptr, self.v.ptr, w[f"{q}.q_norm.weight"], w[f"{q}.k_norm.weight"],
                                          self.cos_t.ptr, self.sin_t.ptr, st["kc"].ptr, st["vc"].ptr, self.pos_dev.ptr,
                                          self.attn_out.ptr, self.attn_scratch.ptr, B, cfg.attn_q_heads, cfg.attn_kv_heads,
                                          cfg.head_dim, cfg.rot_dim // 2, cfg.max_len, self.split_len, cfg.max_len - 1,
                                          float(1.0 / np.sqrt(np.float32(cfg.head_dim))), 0])
                self._launch("quant_q8_1_bf16", [self.attn_out.ptr, self.xq.ptr, aw, B])
                self._gemm(w[f"{q}.o_proj.weight"], self.h1.ptr, H, aw, BK_EPI_ADD_BF16, residual=x)
            self._norm_quant(self.h1.ptr, w[f"{p}.post_attention_layernorm.weight"], H)
            self._gemm(w[f"{p}.mlp.gate_proj.weight"], self.act.ptr, cfg.intermediate, H, BK_EPI_SWIGLU,
                       W2=w[f"{p}.mlp.up_proj.weight"])
            self._launch("quant_q8_1_bf16", [self.act.ptr, self.xq.ptr, cfg.intermediate, B])
            self._gemm(w[f"{p}.mlp.down_proj.weight"], self.x[cur ^ 1].ptr, H, cfg.intermediate, BK_EPI_ADD_BF16,
                       residual=self.h1.ptr)
            cur ^= 1
        self._norm_quant(self.x[cur].ptr, w["final.norm.weight"], H)
        self._gemm(w["embed.weight"], self.logits.ptr, cfg.vocab, H, BK_EPI_F32)
        self._launch("argmax", [self.logits.ptr, self.ids.ptr, self.val.ptr, self.argmax_scratch.ptr, cfg.vocab, B])
        self.pos += 1
        return self.ids.download(np.int32, (B,)), self.val.download(np.float32, (B,))

    def logits_host(self) -> np.ndarray:
        return self.logits.download(np.float32, (self.B, self.cfg.vocab))
