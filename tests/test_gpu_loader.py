"""GPU: the loader's Q4_K quantiser against the oracle, bit for bit, and a checkpoint in the reference's naming loaded
into a decode model."""
import os

import numpy as np
import pytest

from bunker_b200 import loader as L
from bunker_b200 import model as M
from bunker_b200 import ops, synth
from bunker_b200 import runtime as R
from oracle import oracle as O
from oracle.model_oracle import OracleModel
from tests.util import assert_same_bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bf16", [False, True])
def test_quantize_q4k_matches_oracle(bk, bf16):
    rng = np.random.default_rng(21)
    N, K = 37, 1024
    x = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    x[0, :256] = 0.0                                   # all-zero superblock
    x[1, :32] = 0.5                                    # constant sub-block
    x[2] = np.abs(x[2])                                # all positive: every min is zero
    x[3] = -np.abs(x[3])                               # all negative
    x[4, ::7] *= 40.0                                  # outliers that dominate their sub-blocks
    x[5] *= 1e-6                                       # scales near the f16 subnormal range
    if bf16:
        xb = synth.f32_to_bf16(x)
        x = synth.bf16_to_f32(xb)
        dx = R.DeviceBuffer.from_numpy(xb)
    else:
        dx = R.DeviceBuffer.from_numpy(x)
    out = R.DeviceBuffer(N * K // 256 * 144)
    ops.quantize_q4k(dx.ptr, N, K, out.ptr, bf16=bf16)
    assert R.cuSync() == 0
    got = out.download(np.uint8, (N, K // 256 * 144))
    assert_same_bits(got, O.q4k_quantize(x), "Q4_K superblocks")
    dx.free(), out.free()


def test_checkpoint_load_matches_host_quantised_model(bk, tmp_path):
    """A bf16 checkpoint with the reference's tensor names (model.language_model.layers.L...., tied embed_tokens) is
    loaded through the device quantiser; the model must decode exactly like one built from the same weights quantised
    on the host by the oracle, and like the oracle itself."""
    cfg = M.CONFIG_TINY.with_(max_len=64)
    rng = np.random.default_rng(33)
    tensors, bf16_names, host = {}, set(), {}
    for name, kind, shape in M.tensor_specs(cfg):
        key = ("model.language_model.embed_tokens.weight" if name == "embed.weight" else
               "model.language_model.norm.weight" if name == "final.norm.weight" else
               "model.language_model." + name[len("model."):])
        if kind == "q4k":
            w = synth.normal_bf16(rng, shape, 0.03)
            tensors[key] = w
            bf16_names.add(key)
            host[name] = O.q4k_quantize(synth.bf16_to_f32(w))
        elif kind == "f32":
            a = (rng.uniform(-2, 0, shape) if name.endswith("A_log") else 1.0 + rng.normal(0, 0.02, shape)).astype(np.float32)
            tensors[key] = a
            host[name] = a
        else:
            w = synth.normal_bf16(rng, shape, 0.3 if name.endswith("conv1d.weight") else 0.02)
            tensors[key] = w.reshape(shape[0], 1, 4) if name.endswith("conv1d.weight") else w   # HF keeps [C, 1, 4]
            bf16_names.add(key)
            host[name] = w
    path = os.path.join(tmp_path, "tiny.safetensors")
    L.write_safetensors(path, tensors, bf16_names)
    gm = L.load_model(cfg, path, batch=1)
    ref = M.DecodeModel(cfg, host, batch=1)
    prompt = rng.integers(0, cfg.vocab, (6, 1)).astype(np.int32)
    a = M.runGraphDecode(gm, prompt, 24)
    b = M.runGraphDecode(ref, prompt, 24)
    assert np.array_equal(a, b)
    assert_same_bits(gm.logits(), ref.logits(), "logits, device-quantised vs host-quantised weights")
    info = gm.info()
    om = OracleModel(cfg, host, batch=1, split_len=info["split_len"], attn_warps=info["attn_warps"])
    assert np.array_equal(a, om.generate(prompt, 24))
    gm.destroy(), ref.destroy()
    # a checkpoint that lacks a tensor is refused by name
    del tensors["model.language_model.norm.weight"]
    L.write_safetensors(path, tensors, bf16_names)
    with pytest.raises(KeyError, match="final.norm.weight"):
        L.load_model(cfg, path)
