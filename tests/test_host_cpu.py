"""CPU-only: the shared library loads and exports every symbol the header declares; host-side model logic."""
import os
import re

import numpy as np
import pytest

from bunker_b200 import model as M
from bunker_b200 import runtime as R
from bunker_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    inc = os.path.join(ROOT, "include")
    text = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    return sorted(set(re.findall(r"BK_API\s+[\w\s\*]+?\b(bk[A-Z]\w*)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = R.load_library()          # raises if the .so is missing: there is no fallback
    names = header_symbols()
    assert len(names) >= 50
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/*.h but not exported"
    missing = [n for n in names if n not in R.SIGNATURES]
    assert not missing, f"declared but not bound in runtime.SIGNATURES: {missing}"
    extra = [n for n in R.SIGNATURES if n not in names]
    assert not extra, f"bound but not declared in the header: {extra}"


def test_calls_fail_loudly_without_a_gpu_or_init():
    import ctypes as C
    lib = R.load_library()
    out = C.c_uint64()
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present; the uninitialised-state path is covered by the gpu tests")
    assert lib.bkAlloc(16, C.byref(out)) == R.BK_ERR_STATE
    assert b"bkInit" in lib.bkLastError()
    with pytest.raises(R.BunkerCudaError):
        R.cu(0)


def test_struct_layouts_match_the_header():
    import ctypes as C
    assert C.sizeof(R.bkGemvSeg) == 48 and C.sizeof(R.bkGemvArgs) == 40 + 4 * 48
    assert C.sizeof(R.bkGdnArgs) == 15 * 8 + 24 + 8 + 8 and R.bkGdnArgs.out_q8.offset == 144 and R.bkGdnArgs.n_tokens.offset == 152
    assert C.sizeof(R.bkAttnArgs) == 12 * 8 + 8 * 4 + 4 + 4 + 8 + 8 + 8 and R.bkAttnArgs.out_q8.offset == 152
    assert C.sizeof(R.bkModelConfig) == 15 * 4 + 4 + 8


def test_model_specs_and_weight_bytes():
    c3, c4 = M.CONFIG_HYBRID_24L, M.CONFIG_HYBRID_64L
    assert M.weight_bytes(c3) == 1_117_716_480       # 1,987,051,520 parameters x 144/256
    assert M.weight_bytes(c4) == 14_134_763_520
    assert c3.conv_width == 8192 and c3.z_dim == 4096 and c3.qgate_dim == 8192 and c3.kv_dim == 512
    assert [c3.is_full(i) for i in range(8)] == [False, False, False, True] * 2
    names = [n for n, _, _ in M.tensor_specs(c3)]
    assert len(names) == len(set(names))
    assert "model.layers.3.self_attn.q_proj.weight" in names and "model.layers.0.linear_attn.A_log" in names


def test_synth_is_seeded_and_in_range():
    a = M.synth_weights(M.CONFIG_TINY)
    b = M.synth_weights(M.CONFIG_TINY)
    assert all(np.array_equal(a[k], b[k]) for k in a)
    W = a["embed.weight"].reshape(M.CONFIG_TINY.vocab, -1, 144)
    d = W[:, :, 0:4].copy().view(np.float16)
    assert (d >= 0).all() and d.max() < 0.01
    w2, x = synth.gemv_case(8, 512, 2)
    assert w2.shape == (8, 288) and x.shape == (2, 512)


def test_oracle_model_tp_emulation_close_to_single_rank():
    from oracle.model_oracle import OracleModel
    cfg = M.CONFIG_TINY
    w = M.synth_weights(cfg)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, (4, 1)).astype(np.int32)
    a = OracleModel(cfg, w, batch=1, split_len=64)
    b = OracleModel(cfg, w, batch=1, split_len=64, tp=2)
    for t in range(4):
        a.step(prompt[t]); b.step(prompt[t])
    rel = np.abs(a.logits - b.logits).max() / np.abs(a.logits).max()
    assert rel < 2e-2        # different Q8_1 block boundaries never arise (slices are whole superblocks); only sum order differs


def test_staged_image_layout_round_trip():
    """The staged activation layout as documented in the header, built here in numpy from oracle Q8_1 blocks, unpacks to
    the same quants, block scales and d8*sum(q) (host-side helper ops.staged_to_blocks)."""
    from bunker_b200 import ops
    from oracle import oracle as O
    B, K = 3, 512
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (B, K)).astype(np.float32)
    blocks = O.q8_1_quantize(x)                                   # [B, K/32, 36]
    q = blocks[:, :, :32].view(np.int8)
    d8 = O.q8_1_scales(blocks)
    s8 = d8 * q.astype(np.int32).sum(-1).astype(np.float32)
    rw = K // 4 + 8
    words = np.zeros((B, rw), np.uint32)
    qw = np.ascontiguousarray(q).view(np.uint32).reshape(B, K // 32, 8)
    for w in range(8):
        pos = (w & 3) * 2 + (w >> 2)
        words[:, :K // 4].reshape(B, K // 32, 8)[:, :, pos] = qw[:, :, w]
    sc = np.zeros((K // 64, 8, 4), np.float32)
    for b in range(B):
        sc[:, b, 0] = d8[b, 0::2]
        sc[:, b, 1] = d8[b, 1::2] * np.float32(0.0625)
        sc[:, b, 2] = s8[b, 0::2]
        sc[:, b, 3] = s8[b, 1::2]
    img = np.concatenate([words.view(np.uint8).ravel(), sc.view(np.uint8).ravel()])
    q2, d2, s2 = ops.staged_to_blocks(img, K, B)
    assert np.array_equal(q2.reshape(B, K // 32, 32), q)
    assert np.array_equal(d2.view(np.uint32), d8.view(np.uint32))
    assert np.array_equal(s2.view(np.uint32), s8.astype(np.float32).view(np.uint32))


def test_graph_front_end_partitions_onto_fused_kernels():
    """The declarative step graph (src/model.ts shape) falls into exactly the launches of the per-op step: embed, five
    per layer, lm_head, argmax; a graph with a node outside the fused groups is refused by node."""
    from bunker_b200 import graph as G
    cfg = M.CONFIG_HYBRID_24L
    g = G.buildModelGraph(cfg)
    assert len(g.nodes) == 1 + 18 * 17 + 6 * 19 + 3        # embed + GDN layers + attention layers + final norm, lm_head, argmax
    part = G.choosePartition(g)
    assert len(part) == 1 + 24 * 5 + 2
    comp = G.compileStep(g, part)
    kinds = [k.kind for k in comp.schedule]
    assert kinds[:6] == ["embed", "norm_gemv", "gdn", "gemv_add", "norm_gemv_swiglu", "gemv_add"]
    assert kinds[16:21] == ["norm_gemv", "attn", "gemv_add", "norm_gemv_swiglu", "gemv_add"]
    assert kinds[-2:] == ["norm_gemv", "argmax"]
    assert [len(k.group) for k in comp.schedule[1:6]] == [5, 2, 3, 4, 3]
    ext = set(g.externals())
    assert {"token_id", "pos", "embed.weight", "lm_head.weight", "model.layers.0.conv_state_in", "model.layers.3.kv_k_in",
            "rope_cos"} <= ext
    bad = G.Graph()
    x = bad.input("x", G.TensorType((1, 64), "f32"))
    bad.node("swiglu", [("g", x), ("u", x)], [("out", G.TensorType((1, 64), "bf16"))])
    with pytest.raises(ValueError, match="swiglu"):
        G.choosePartition(bad)


def test_typescript_binding_lists_every_export():
    """bunker_b200/ts/bunker_cuda.ts is the bun:ffi side of the boundary (it cannot run here: no bun).  Its symbol
    table must name exactly the exports the headers declare, with pointer-sized handles as u64, never `ptr`."""
    ts = open(os.path.join(ROOT, "bunker_b200", "ts", "bunker_cuda.ts")).read()
    table = ts[ts.index("const SYMBOLS = {"):ts.index("} as const;")]
    bound = dict(re.findall(r"^\s+(bk\w+): \{ args: \[([^\]]*)\]", table, flags=re.M))
    assert sorted(bound) == header_symbols()
    assert bound["bkAlloc"] == '"u64", "ptr"' and bound["bkFree"] == '"u64"' and bound["bkModelFinalize"] == '"u64"'
    for name in ("cuAlloc", "cuHtoD", "cuDtoH", "cuFree", "cuSync", "cuHtoDAsync", "cuDtoHAsync", "cuLaunch", "loadOp",
                 "LoadedKernel", "profGpuReport", "runGraphDecode"):
        assert re.search(rf"export (function|interface|class) {name}\b", ts), name
