"""Whole decode step on the CPU oracle (test infrastructure only; never imported by the package).

Composition of the oracle ops in the order of bunker's tuned decode loop (prototypes/decode.ts:952-1062)
with Q4_K x Q8_1 GEMVs in place of its bf16 GEMMs.  `tp` emulates tensor-parallel ranks: row-parallel
GEMVs (out_proj, o_proj, down) are computed per K-slice and the partials added in rank order.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O


class OracleModel:
    def __init__(self, cfg, weights: dict, batch: int, split_len: int, attn_warps: int = 8, tp: int = 1,
                 gemv_order: str | None = None, tile_min_rows: int | None = None):
        """gemv_order: "lanes" (the batch <= 8 kernels: units over lanes, butterfly) or "tile" (the dense tile path
        for every launch of at least 4096 rows, all its segments together, or at least 1024 rows and K >= 2048 -- the
        library's rule for BK_GEMV_ORDER_AUTO; tile_min_rows replaces both row thresholds, as bkTuneTileMinRows does);
        None picks what the library picks for this batch (tile from 16 sequences on, on one GPU)."""
        self.cfg, self.w, self.B, self.split_len, self.W, self.tp = cfg, weights, batch, split_len, attn_warps, tp
        self.gemv_order = gemv_order or ("tile" if (batch >= 16 and tp == 1) else "lanes")
        self.tile_min_rows = tile_min_rows
        self.cos_t, self.sin_t = O.rope_tables(cfg.max_len, cfg.rot_dim, cfg.rope_theta)
        self.reset()

    def reset(self):
        c, B = self.cfg, self.B
        self.pos = 0
        self.conv = {}
        self.S = {}
        self.kc = {}
        self.vc = {}
        for li in range(c.n_layers):
            if c.is_full(li):
                self.kc[li] = np.zeros((B, c.attn_kv_heads, c.max_len, c.head_dim), np.uint16)
                self.vc[li] = np.zeros_like(self.kc[li])
            else:
                self.conv[li] = np.zeros((B, 3, c.conv_width), np.uint16)
                self.S[li] = np.zeros((B, c.gdn_v_heads, 128, 128), np.float32)

    def _gemv(self, name: str, N: int, K: int, xq: np.ndarray, launch_rows: int) -> np.ndarray:
        """launch_rows: rows of the whole launch this projection is a segment of (it decides the f32 order)."""
        big, cut = (4096, 1024) if self.tile_min_rows is None else (self.tile_min_rows, self.tile_min_rows)
        tile = self.gemv_order == "tile" and (launch_rows >= big or (launch_rows >= cut and K >= 2048))
        return (O.gemv_q4k_q8_tile if tile else O.gemv_q4k_q8)(self.w[name], N, K, xq)

    def _gemv_rowpar(self, name: str, N: int, K: int, x_bf16: np.ndarray) -> np.ndarray:
        """f32 [B, N]; with tp > 1 the K dimension is cut into tp slices of whole superblocks."""
        if self.tp == 1:
            return self._gemv(name, N, K, O.q8_1_quantize_bf16(x_bf16), N)
        W = np.ascontiguousarray(self.w[name]).reshape(N, K // 256, 144)
        nsb = K // 256
        base, extra = divmod(nsb, self.tp)
        parts, s0 = [], 0
        for r in range(self.tp):
            n = base + (1 if r < extra else 0)
            Wr = np.ascontiguousarray(W[:, s0:s0 + n]).reshape(N, n * 144)
            xr = np.ascontiguousarray(x_bf16[:, s0 * 256:(s0 + n) * 256])
            parts.append(O.gemv_q4k_q8(Wr, N, n * 256, O.q8_1_quantize_bf16(xr)))   # tensor parallel: lanes order
            s0 += n
        return O.sum_ranks(np.stack(parts))

    def step(self, tokens):
        c, B, w = self.cfg, self.B, self.w
        H = c.hidden
        tokens = np.asarray(tokens, np.int32).reshape(B)
        pos = np.full((B,), self.pos, np.int32)
        x = O.embed_q4k(w["embed.weight"], H, tokens)
        for li in range(c.n_layers):
            p = f"model.layers.{li}"
            xq = O.q8_1_quantize_bf16(O.rmsnorm(x, w[f"{p}.input_layernorm.weight"], c.eps))
            if not c.is_full(li):
                q = f"{p}.linear_attn"
                rows = c.conv_width + c.z_dim + 2 * c.gdn_v_heads   # one launch, four segments
                qkv = O.epilogue_cast(self._gemv(f"{q}.in_proj_qkv.weight", c.conv_width, H, xq, rows))
                z = O.epilogue_cast(self._gemv(f"{q}.in_proj_z.weight", c.z_dim, H, xq, rows))
                a = self._gemv(f"{q}.in_proj_a.weight", c.gdn_v_heads, H, xq, rows)
                b = self._gemv(f"{q}.in_proj_b.weight", c.gdn_v_heads, H, xq, rows)
                conv_out, self.conv[li] = O.conv1d_step(qkv, self.conv[li], w[f"{q}.conv1d.weight"])
                self.S[li], o_raw = O.gdn_step(conv_out, a, b, w[f"{q}.A_log"], w[f"{q}.dt_bias"], self.S[li],
                                               c.gdn_k_heads, c.gdn_v_heads)
                attn = O.gdn_gate_norm(o_raw, z, w[f"{q}.norm.weight"], c.gdn_v_heads)
                y = self._gemv_rowpar(f"{q}.out_proj.weight", H, c.z_dim, attn)
            else:
                q = f"{p}.self_attn"
                rows = c.qgate_dim + 2 * c.kv_dim
                qg = O.epilogue_cast(self._gemv(f"{q}.q_proj.weight", c.qgate_dim, H, xq, rows))
                k = O.epilogue_cast(self._gemv(f"{q}.k_proj.weight", c.kv_dim, H, xq, rows))
                v = O.epilogue_cast(self._gemv(f"{q}.v_proj.weight", c.kv_dim, H, xq, rows))
                HD = c.head_dim
                qn = O.headnorm_rope(qg, 2 * HD, w[f"{q}.q_norm.weight"], self.cos_t, self.sin_t, pos, c.attn_q_heads, HD)
                kn = O.headnorm_rope(k, HD, w[f"{q}.k_norm.weight"], self.cos_t, self.sin_t, pos, c.attn_kv_heads, HD)
                self.kc[li][:, :, self.pos] = kn.reshape(B, c.attn_kv_heads, HD)
                self.vc[li][:, :, self.pos] = v.reshape(B, c.attn_kv_heads, HD)
                gate = np.ascontiguousarray(qg.reshape(B, c.attn_q_heads, 2, HD)[:, :, 1])
                attn = O.attn_decode(qn, gate, HD, self.kc[li], self.vc[li], pos, c.attn_q_heads, c.attn_kv_heads, HD,
                                     self.split_len, self.W, 1.0 / float(np.sqrt(np.float32(HD))))
                y = self._gemv_rowpar(f"{q}.o_proj.weight", H, c.attn_q_heads * HD, attn)
            h1 = O.epilogue_add(y, x)
            xq2 = O.q8_1_quantize_bf16(O.rmsnorm(h1, w[f"{p}.post_attention_layernorm.weight"], c.eps))
            g = self._gemv(f"{p}.mlp.gate_proj.weight", c.intermediate, H, xq2, 2 * c.intermediate)
            u = self._gemv(f"{p}.mlp.up_proj.weight", c.intermediate, H, xq2, 2 * c.intermediate)
            act = O.swiglu(g, u)
            y2 = self._gemv_rowpar(f"{p}.mlp.down_proj.weight", H, c.intermediate, act)
            x = O.epilogue_add(y2, h1)
        xqf = O.q8_1_quantize_bf16(O.rmsnorm(x, w["final.norm.weight"], c.eps))
        self.logits = self._gemv("embed.weight", c.vocab, H, xqf, c.vocab)
        idx, val = O.argmax(self.logits)
        self.pos += 1
        return idx, val

    def generate(self, prompt: np.ndarray, gen_len: int) -> np.ndarray:
        prompt = np.asarray(prompt, np.int32).reshape(len(prompt), -1)
        ids = None
        for t in range(prompt.shape[0]):
            ids, _ = self.step(prompt[t])
        out = [ids]
        for _ in range(1, gen_len):
            ids, _ = self.step(ids)
            out.append(ids)
        return np.stack(out)
