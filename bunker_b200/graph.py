"""Graph front end: bunker's declarative decode graph (src/model.ts) driven onto the fused kernels of this library.

bunker declares one token step as a Graph of nodes (embed, rmsnorm, gemm, conv1d_decode, gdn_delta_rule, qnorm, rope,
knorm, ropek, fa2_attn, cast, add, swiglu, argmax -- src/model.ts:46-204), lets a search partition the nodes into
kernels (src/fusion.ts `explore`), and runs the compiled schedule with `runGraphDecode` (src/runner.ts:116-162), the
caller supplying `resolve(name)` for weights / state and rotating the state buffers in `onToken`
(prototypes/decode_graph.ts:67-151).  Here the same Graph objects are accepted, but the partition is STATIC: node groups
are matched onto the fixed fused kernels --

    embed                                   -> bkEmbedQ4K
    rmsnorm + the gemms that read it        -> one GEMV launch, RMSNorm+Q8_1 prologue, one segment per gemm
    rmsnorm + gate gemm + up gemm + swiglu  -> one GEMV launch with the SwiGLU epilogue
    conv1d_decode + gdn_delta_rule          -> bkGdnStep
    qnorm + rope + knorm + ropek + fa2_attn -> bkAttnDecode
    gemm + cast + add                       -> one GEMV launch with the residual epilogue (one rounding)
    argmax                                  -> bkArgmax

-- so a `runner.ts`-style caller drives the library without knowing how ops are fused.  A graph whose nodes do not fall
into these groups is rejected with the node that did not match.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import numpy as np

from . import ops
from . import runtime as R
from .model import ModelConfig
from .runtime import BK_EPI_ADD_BF16, BK_EPI_BF16, BK_EPI_F32, BK_EPI_SWIGLU, BK_PRO_BF16, BK_PRO_RMSNORM

_ESZ = {"bf16": 2, "f32": 4, "i32": 4}


# ---- Graph IR (src/fusion.ts:47-66,123-184) -------------------------------------------------------------------
@dataclass
class TensorType:
    shape: tuple
    dtype: str

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * _ESZ[self.dtype] if self.shape else _ESZ[self.dtype]


@dataclass
class Tensor:
    name: str
    type: TensorType
    role: str = "data"            # data | weight | state | scalar
    producer: "GraphNode | None" = None
    consumers: list = field(default_factory=list)


@dataclass
class Port:
    name: str
    tensorName: str
    type: TensorType
    role: str


@dataclass
class GraphNode:
    id: int
    op: str
    inputs: list
    outputs: list
    grid: tuple
    params: dict

    def inp(self, name: str) -> str:
        return next(p.tensorName for p in self.inputs if p.name == name)


class Graph:
    def __init__(self):
        self.nodes: list[GraphNode] = []
        self.tensors: dict[str, Tensor] = {}

    def input(self, name: str, type: TensorType, role: str = "data") -> Tensor:
        t = self.tensors.get(name)
        if t is None:
            t = self.tensors[name] = Tensor(name, type, role)
        return t

    def node(self, op: str, inputs, outputs, grid=(1, 1, 1), params=None) -> GraphNode:
        n = GraphNode(len(self.nodes), op, [], [], tuple(grid), dict(params or {}))
        for pname, t in inputs:
            t = self.tensors[t] if isinstance(t, str) else t
            n.inputs.append(Port(pname, t.name, t.type, t.role))
            t.consumers.append(n)
        for o in outputs:
            oname, otype = o[0], o[1]
            role = o[2] if len(o) > 2 else "data"
            full = f"n{n.id}_{oname}"
            n.outputs.append(Port(oname, full, otype, role))
            self.tensors[full] = Tensor(full, otype, role, producer=n)
        self.nodes.append(n)
        return n

    def t(self, name: str) -> Tensor:
        return self.tensors[name]

    def out(self, node: GraphNode, name: str = "out") -> str:
        return f"n{node.id}_{name}"

    def externals(self) -> list[str]:
        return [t.name for t in self.tensors.values() if t.producer is None]


# ---- the model as a graph (src/model.ts:46-204, dims from the config) -----------------------------------------
def buildModelGraph(cfg: ModelConfig, M: int = 1) -> Graph:
    g = Graph()
    H, V, HD = cfg.hidden, cfg.vocab, cfg.head_dim
    QKVD, ZD, LVH, INTER = cfg.conv_width, cfg.z_dim, cfg.gdn_v_heads, cfg.intermediate
    QGATE, KVD, NH, NKV, ML = cfg.qgate_dim, cfg.kv_dim, cfg.attn_q_heads, cfg.attn_kv_heads, cfg.max_len
    bf = lambda *s: TensorType(tuple(s), "bf16")     # noqa: E731
    f32 = lambda *s: TensorType(tuple(s), "f32")     # noqa: E731
    tk = g.input("token_id", TensorType((), "i32"), "scalar")
    pos = g.input("pos", TensorType((), "i32"), "scalar")
    L = lambda li: f"model.layers.{li}"              # noqa: E731
    W = lambda name, *s: g.input(name, bf(*s), "weight")   # noqa: E731
    emb = g.node("embed", [("E", W("embed.weight", V, H)), ("id", tk)], [("out", bf(M, H))], (1, 1, 1), {"H": H})
    h = g.out(emb)
    gemm = lambda a, wname, N, K, out_t, **kw: g.node(   # noqa: E731
        "gemm", [("A", a), ("B", W(wname, N, K))], [("out", out_t)], (1, -(-N // 64), 1), dict(M=M, N=N, K=K, **kw))
    for li in range(cfg.n_layers):
        full = cfg.is_full(li)
        normed = g.node("rmsnorm", [("x", h), ("w", W(f"{L(li)}.input_layernorm.weight", H))], [("out", bf(M, H))], (1, 1, 1), {"N": H})
        nx = g.out(normed)
        if not full:
            p = f"{L(li)}.linear_attn"
            qkv = gemm(nx, f"{p}.in_proj_qkv.weight", QKVD, H, bf(M, QKVD), cast=True)
            zg = gemm(nx, f"{p}.in_proj_z.weight", ZD, H, bf(M, ZD), cast=True)
            conv = g.node("conv1d_decode",
                          [("qkv", g.out(qkv)), ("state", g.input(f"{L(li)}.conv_state_in", bf(M, 3, QKVD), "state")),
                           ("w", W(f"{p}.conv1d.weight", QKVD, 4))],
                          [("out", bf(M, QKVD)), (f"{L(li)}.conv_state_new", bf(M, 3, QKVD), "state")], (-(-QKVD // 1024), 1, 1),
                          {"QKVD": QKVD})
            ap = gemm(nx, f"{p}.in_proj_a.weight", LVH, H, f32(M, LVH))
            bp = gemm(nx, f"{p}.in_proj_b.weight", LVH, H, f32(M, LVH))
            gdn = g.node("gdn_delta_rule",
                         [("conv_out", g.out(conv)), ("z", g.out(zg)), ("A_log", g.input(f"{p}.A_log", f32(LVH), "weight")),
                          ("dt_bias", W(f"{p}.dt_bias", LVH)), ("a_p", g.out(ap)), ("b_p", g.out(bp)),
                          ("norm_w", g.input(f"{p}.norm.weight", f32(128), "weight")),
                          ("s_state", g.input(f"{L(li)}.s_state_in", f32(M, LVH, 128, 128), "state"))],
                         [("out", bf(M, ZD)), (f"{L(li)}.s_state_new", f32(M, LVH, 128, 128), "state")], (LVH, 1, 1),
                         {"LVH": LVH, "LKH": cfg.gdn_k_heads, "QKVD": QKVD, "ZD": ZD})
            proj = gemm(g.out(gdn), f"{p}.out_proj.weight", H, ZD, f32(M, H))
        else:
            p = f"{L(li)}.self_attn"
            qp = gemm(nx, f"{p}.q_proj.weight", QGATE, H, bf(M, QGATE), cast=True)
            kp = gemm(nx, f"{p}.k_proj.weight", KVD, H, bf(M, KVD), cast=True)
            vp = gemm(nx, f"{p}.v_proj.weight", KVD, H, bf(M, KVD), cast=True)
            qn = g.node("qnorm", [("q", g.out(qp)), ("w", W(f"{p}.q_norm.weight", HD))], [("out", bf(M, NH * HD))], (NH, 1, 1), {"HD": HD, "NH": NH})
            cos_t = g.input("rope_cos", f32(ML, cfg.rot_dim // 2), "weight")
            sin_t = g.input("rope_sin", f32(ML, cfg.rot_dim // 2), "weight")
            g.node("rope", [("Q", g.out(qn)), ("C", cos_t), ("S", sin_t), ("P", pos)], [], (NH, 1, 1), {"HD": HD})
            kn = g.node("knorm", [("k", g.out(kp)), ("w", W(f"{p}.k_norm.weight", HD))], [("out", bf(M, KVD))], (NKV, 1, 1), {"HD": HD, "NKV": NKV})
            g.node("ropek", [("K", g.out(kn)), ("C", cos_t), ("S", sin_t), ("P", pos)], [], (NKV, 1, 1), {"HD": HD})
            kv_t = bf(M, NKV * ML, HD)     # per KV head (the reference replicates per query head, src/emitters.ts:202)
            fa2 = g.node("fa2_attn",
                         [("q", g.out(qn)), ("k", g.out(kn)), ("v", g.out(vp)), ("qgate", g.out(qp)),
                          ("kc_in", g.input(f"{L(li)}.kv_k_in", kv_t, "state")), ("vc_in", g.input(f"{L(li)}.kv_v_in", kv_t, "state")),
                          ("P", pos)],
                         [("out", bf(M, NH * HD)), (f"{L(li)}.kv_k_new", kv_t, "state"), (f"{L(li)}.kv_v_new", kv_t, "state")],
                         (NH, 1, 1), {"HD": HD, "NH": NH, "NKV": NKV, "MAX_LEN": ML})
            proj = gemm(g.out(fa2), f"{p}.o_proj.weight", H, NH * HD, f32(M, H))
        cast_o = g.node("cast", [("x", g.out(proj))], [("out", bf(M, H))], (1, -(-H // 64), 1), {"to": "bf16", "N": H})
        after = g.node("add", [("a", g.out(cast_o)), ("b", h)], [("out", bf(M, H))], (1, -(-H // 64), 1), {"N": H})
        h = g.out(after)
        normed2 = g.node("rmsnorm", [("x", h), ("w", W(f"{L(li)}.post_attention_layernorm.weight", H))], [("out", bf(M, H))], (1, 1, 1), {"N": H})
        gate = gemm(g.out(normed2), f"{L(li)}.mlp.gate_proj.weight", INTER, H, f32(M, INTER))
        up = gemm(g.out(normed2), f"{L(li)}.mlp.up_proj.weight", INTER, H, f32(M, INTER))
        act = g.node("swiglu", [("g", g.out(gate)), ("u", g.out(up))], [("out", bf(M, INTER))], (-(-INTER // 1024), 1, 1), {"N": INTER})
        down = gemm(g.out(act), f"{L(li)}.mlp.down_proj.weight", H, INTER, f32(M, H))
        cast_d = g.node("cast", [("x", g.out(down))], [("out", bf(M, H))], (1, -(-H // 64), 1), {"to": "bf16", "N": H})
        xnew = g.node("add", [("a", h), ("b", g.out(cast_d))], [("out", bf(M, H))], (1, -(-H // 64), 1), {"N": H})
        h = g.out(xnew)
    fn = g.node("rmsnorm", [("x", h), ("w", W("final.norm.weight", H))], [("out", bf(M, H))], (1, 1, 1), {"N": H})
    logits = gemm(g.out(fn), "lm_head.weight", V, H, f32(M, V))
    g.node("argmax", [("logits", g.out(logits))], [("val", f32(M)), ("idx", TensorType((M,), "i32"))], (1, 1, 1), {"VOCAB": V})
    return g


# ---- static partition onto the fused kernels -------------------------------------------------------------------
@dataclass
class KernelPlan:
    """src/fusion.ts:110-117 KernelPlan: what one launch covers.  `kind` names the fused kernel."""
    name: str
    kind: str
    group: list
    args: list     # external tensor names the launch reads / writes, in a fixed order per kind


def _only_consumers(g: Graph, tname: str, nodes) -> bool:
    return all(c in nodes for c in g.t(tname).consumers)


def choosePartition(g: Graph) -> list[list[GraphNode]]:
    """The static counterpart of src/runner.ts:40-49 + src/fusion.ts `explore`: groups of nodes, in schedule order,
    each of which is one fused launch.  Raises ValueError naming the first node that fits no group."""
    used: set[int] = set()
    groups: list[list[GraphNode]] = []
    by_id = {n.id: n for n in g.nodes}

    def consumers(n, port="out"):
        return [c for c in g.t(g.out(n, port)).consumers]

    for n in g.nodes:
        if n.id in used:
            continue
        grp = None
        if n.op in ("embed", "argmax"):
            grp = [n]
        elif n.op == "rmsnorm":
            cons = consumers(n)
            if cons and all(c.op == "gemm" and c.inp("A") == g.out(n) for c in cons):
                grp = [n] + cons
                if len(cons) == 2:   # gate | up feeding one swiglu -> the SwiGLU epilogue
                    sw = [c for c in consumers(cons[0]) if c.op == "swiglu"]
                    if sw and consumers(cons[1]) == sw and len(consumers(cons[0])) == 1:
                        grp = [n] + cons + sw
        elif n.op == "conv1d_decode":
            cons = consumers(n)
            if len(cons) == 1 and cons[0].op == "gdn_delta_rule":
                grp = [n, cons[0]]
        elif n.op == "qnorm":
            # qnorm -> rope (in place) ; knorm -> ropek (in place) ; fa2_attn reads both
            fa = [c for c in consumers(n) if c.op == "fa2_attn"]
            rq = [c for c in consumers(n) if c.op == "rope"]
            if len(fa) == 1 and len(rq) == 1:
                kn = g.t(fa[0].inp("k")).producer
                rk = [c for c in consumers(kn) if c.op == "ropek"] if kn is not None and kn.op == "knorm" else []
                if rk:
                    grp = [n, rq[0], kn, rk[0], fa[0]]
        elif n.op == "gemm":
            cons = consumers(n)
            if len(cons) == 1 and cons[0].op == "cast":
                c2 = consumers(cons[0])
                if len(c2) == 1 and c2[0].op == "add":
                    grp = [n, cons[0], c2[0]]
        if grp is None or any(m.id in used for m in grp):
            raise ValueError(f"node n{n.id} ({n.op}) does not fit a fused kernel of this library")
        for m in grp:
            used.add(m.id)
        groups.append(sorted(grp, key=lambda m: m.id))
    assert len(used) == len(by_id)
    return groups


@dataclass
class CompiledStep:
    graph: Graph
    schedule: list     # KernelPlan, in launch order


def compileStep(g: Graph, partition: list[list[GraphNode]]) -> CompiledStep:
    """src/runner.ts:94-104: groups -> launch plans.  (Nothing is compiled: the kernels are in the library.)"""
    plans = []
    for grp in partition:
        ops_ = [n.op for n in grp]
        if ops_ == ["embed"]:
            kind = "embed"
        elif ops_ == ["argmax"]:
            kind = "argmax"
        elif ops_[0] == "rmsnorm" and ops_[-1] == "swiglu":
            kind = "norm_gemv_swiglu"
        elif ops_[0] == "rmsnorm":
            kind = "norm_gemv"
        elif ops_ == ["conv1d_decode", "gdn_delta_rule"]:
            kind = "gdn"
        elif "fa2_attn" in ops_:
            kind = "attn"
        elif ops_ == ["gemm", "cast", "add"]:
            kind = "gemv_add"
        else:
            raise ValueError(f"group {ops_} has no kernel")
        ext = []
        inside = {p.tensorName for n in grp for p in n.outputs}
        for n in grp:
            for p in n.inputs:
                if p.tensorName not in inside and p.tensorName not in ext:
                    ext.append(p.tensorName)
        for n in grp:
            for p in n.outputs:
                if not _only_consumers(g, p.tensorName, grp) or not g.t(p.tensorName).consumers:
                    ext.append(p.tensorName)
        plans.append(KernelPlan(f"k{len(plans)}_{kind}", kind, grp, ext))
    return CompiledStep(g, plans)


# ---- executor (src/runner.ts:116-162) --------------------------------------------------------------------------
class GraphRunner:
    """Runs a CompiledStep token by token.  `resolve(name)` gives the device pointer of every weight and state tensor
    (the reference's callback, prototypes/decode_graph.ts:111-143); intermediates are allocated here, once."""

    def __init__(self, compiled: CompiledStep, cfg: ModelConfig, resolve: Callable[[str], int], M: int = 1):
        self.c, self.cfg, self.resolve, self.M = compiled, cfg, resolve, M
        R.cu()
        g = compiled.graph
        self.buf: dict[str, R.DeviceBuffer] = {}
        for t in g.tensors.values():
            if t.producer is not None and t.role == "data":
                self.buf[t.name] = R.DeviceBuffer.zeros(max(t.type.nbytes, 16))
        self.ids, self.pos_dev = R.DeviceBuffer.zeros(M * 4), R.DeviceBuffer.zeros(M * 4)
        self.argmax_scratch = R.DeviceBuffer.zeros(ops.argmax_scratch_bytes(M))
        self.split_len, self.attn_warps = ops.attn_plan(cfg.max_len, M, cfg.attn_kv_heads)
        self.attn_scratch = R.DeviceBuffer.zeros(ops.attn_scratch_bytes(M, cfg.attn_q_heads, cfg.head_dim, cfg.max_len, self.split_len))
        self.idx_out, self.val_out = R.DeviceBuffer.zeros(M * 4), R.DeviceBuffer.zeros(M * 4)

    def ptr(self, name: str) -> int:
        b = self.buf.get(name)
        return b.ptr if b is not None else int(self.resolve(name))

    def _launch(self, k: KernelPlan) -> None:
        g, cfg, M = self.c.graph, self.cfg, self.M
        grp = k.group
        if k.kind == "embed":
            n = grp[0]
            ops.embed(self.ptr(n.inp("E")), n.params["H"], self.ids.ptr, M, self.ptr(g.out(n)))
        elif k.kind in ("norm_gemv", "norm_gemv_swiglu"):
            norm, gemms = grp[0], [n for n in grp if n.op == "gemm"]
            K = gemms[0].params["K"]
            if k.kind == "norm_gemv_swiglu":
                sw = grp[-1]
                gate = g.t(sw.inp("g")).producer
                up = g.t(sw.inp("u")).producer
                segs = [ops.gemv_seg(self.ptr(gate.inp("B")), gate.params["N"], self.ptr(g.out(sw)), BK_EPI_SWIGLU,
                                     W2=self.ptr(up.inp("B")))]
            else:
                segs = [ops.gemv_seg(self.ptr(n.inp("B")), n.params["N"], self.ptr(g.out(n)),
                                     BK_EPI_BF16 if n.outputs[0].type.dtype == "bf16" else BK_EPI_F32) for n in gemms]
            ops.gemv(self.ptr(norm.inp("x")), K, M, segs, prologue=BK_PRO_RMSNORM, norm_w=self.ptr(norm.inp("w")), eps=cfg.eps)
        elif k.kind == "gdn":
            conv, gdn = grp
            ops.gdn_step(qkv=self.ptr(conv.inp("qkv")), z=self.ptr(gdn.inp("z")), a=self.ptr(gdn.inp("a_p")), b=self.ptr(gdn.inp("b_p")),
                         conv_w=self.ptr(conv.inp("w")), conv_state_in=self.ptr(conv.inp("state")),
                         conv_state_new=self.ptr(conv.outputs[1].tensorName), A_log=self.ptr(gdn.inp("A_log")),
                         dt_bias=self.ptr(gdn.inp("dt_bias")), norm_w=self.ptr(gdn.inp("norm_w")), S_in=self.ptr(gdn.inp("s_state")),
                         S_new=self.ptr(gdn.outputs[1].tensorName), out=self.ptr(g.out(gdn)), B=M, Hk=gdn.params["LKH"],
                         Hv=gdn.params["LVH"], apply_conv=1)
        elif k.kind == "attn":
            qn, kn, fa = grp[0], next(n for n in grp if n.op == "knorm"), grp[-1]
            ops.attn_decode(qg=self.ptr(fa.inp("qgate")), k=self.ptr(kn.inp("k")), v=self.ptr(fa.inp("v")),
                            q_norm_w=self.ptr(qn.inp("w")), k_norm_w=self.ptr(kn.inp("w")), cos_t=self.ptr("rope_cos"),
                            sin_t=self.ptr("rope_sin"), k_cache=self.ptr(fa.inp("kc_in")), v_cache=self.ptr(fa.inp("vc_in")),
                            pos=self.pos_dev.ptr, out=self.ptr(g.out(fa)), scratch=self.attn_scratch.ptr, B=M, Hq=cfg.attn_q_heads,
                            Hkv=cfg.attn_kv_heads, HD=cfg.head_dim, rot_half=cfg.rot_dim // 2, max_len=cfg.max_len,
                            split_len=self.split_len, max_pos=cfg.max_len - 1, scale=float(1.0 / np.sqrt(np.float32(cfg.head_dim))),
                            fused_norm_rope=1)
        elif k.kind == "gemv_add":
            gm, _, add = grp
            cast_out = g.out(grp[1])
            res = add.inp("b") if add.inp("a") == cast_out else add.inp("a")
            segs = [ops.gemv_seg(self.ptr(gm.inp("B")), gm.params["N"], self.ptr(g.out(add)), BK_EPI_ADD_BF16, residual=self.ptr(res))]
            ops.gemv(self.ptr(gm.inp("A")), gm.params["K"], M, segs, prologue=BK_PRO_BF16)
        elif k.kind == "argmax":
            n = grp[0]
            ops.argmax(self.ptr(n.inp("logits")), n.params["VOCAB"], M, self.idx_out.ptr, self.val_out.ptr, self.argmax_scratch.ptr)

    def step(self, tokens, pos: int):
        """One token per sequence: all launches, sync, read (idx, val) -- src/runner.ts:133-160."""
        R.cuHtoD(self.ids.ptr, np.ascontiguousarray(tokens, np.int32).reshape(self.M))
        R.cuHtoD(self.pos_dev.ptr, np.full((self.M,), pos, np.int32))
        for k in self.c.schedule:
            self._launch(k)
        rc = R.cuSync()
        if rc != 0:
            raise R.BunkerCudaError(rc, R.last_error())
        return self.idx_out.download(np.int32, (self.M,)), self.val_out.download(np.float32, (self.M,))


def runGraphDecode(runner: GraphRunner, prompt: np.ndarray, gen_len: int, onToken: Callable[[int], None]) -> np.ndarray:
    """src/runner.ts:116-162: prompt tokens one at a time through the step, then gen_len-1 greedy steps.  `onToken(pos)` is
    called after every step so that the caller rotates its double-buffered state (decode_graph.ts:145-151)."""
    prompt = np.asarray(prompt, np.int32).reshape(len(prompt), -1)
    out, ids, pos = [], None, 0
    for t in range(prompt.shape[0]):
        ids, _ = runner.step(prompt[t], pos)
        onToken(pos)
        pos += 1
    out.append(ids)
    for _ in range(1, gen_len):
        ids, _ = runner.step(ids, pos)
        onToken(pos)
        pos += 1
        out.append(ids)
    return np.stack(out)


class StateStore:
    """The caller's side of the contract (prototypes/decode_graph.ts:67-151): weights uploaded once, conv and GDN state
    double-buffered and rotated after every token, KV caches single buffers updated in place, rope tables built on
    the host.  `resolve` is what GraphRunner asks for pointers."""

    def __init__(self, g: Graph, cfg: ModelConfig, weights: dict[str, np.ndarray]):
        R.cu()
        self.g = g
        self.w = {}
        for name in g.externals():
            t = g.t(name)
            if t.role == "weight" and name not in ("rope_cos", "rope_sin"):
                src = weights["embed.weight" if name == "lm_head.weight" else name]
                if name == "lm_head.weight" and "embed.weight" in self.w:
                    self.w[name] = self.w["embed.weight"]
                else:
                    self.w[name] = R.DeviceBuffer.from_numpy(np.ascontiguousarray(src))
        cos_t, sin_t = ops.rope_tables(cfg.max_len, cfg.rot_dim, cfg.rope_theta)
        self.w["rope_cos"], self.w["rope_sin"] = R.DeviceBuffer.from_numpy(cos_t), R.DeviceBuffer.from_numpy(sin_t)
        self.state, self.cur = {}, {}
        for t in g.tensors.values():
            if t.role != "state":
                continue
            base = self._clean(t.name)
            if base in self.state:
                continue
            n = max(t.type.nbytes, 16)
            inplace = ".kv_k" in base or ".kv_v" in base or ".s_state" in base   # the GDN state is rewritten in place here
            a = R.DeviceBuffer.zeros(n)
            self.state[base] = [a, a if inplace else R.DeviceBuffer.zeros(n)]
            self.cur[base] = 0

    @staticmethod
    def _clean(name: str) -> str:
        import re
        name = re.sub(r"^n\d+_", "", name)
        return re.sub(r"_(in|new)$", "", name)

    def resolve(self, name: str) -> int:
        if name in self.w:
            return self.w[name].ptr
        base = self._clean(name)
        bufs = self.state[base]
        is_new = name.endswith("_new")
        return bufs[self.cur[base] ^ (1 if is_new else 0)].ptr

    def onToken(self, pos: int) -> None:
        for base in self.cur:
            self.cur[base] ^= 1
