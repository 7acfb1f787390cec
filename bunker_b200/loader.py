"""Real-weights loader: a safetensors checkpoint in the reference's naming -> Q4_K model on the device.

Mirrors bunker's loaders: the file format reader of loadWeights (prototypes/decode.ts:64-76: 8-byte little-endian
header length, JSON header with dtype / shape / data_offsets per tensor, then the raw bytes) and the graph-name ->
checkpoint-name rule of safeKey (prototypes/decode_graph.ts:99-109).  bunker uploads the bf16 weights as they are;
here every linear weight is quantised to Q4_K on the device (bkQuantizeQ4K) on its way into the weight slab, one
tensor at a time, so the host never holds more than one tensor and the device never holds the bf16 model.

Tensor parallel: every rank reads the file and cuts its rows / K range out of each tensor BEFORE quantising
(model.shard_plan).  K ranges are whole superblocks and the quantiser works superblock by superblock, so the shard is
bit-identical to the same cut of the quantised full tensor.
"""
from __future__ import annotations

import json
import struct

import numpy as np

from . import model as M
from . import ops
from . import runtime as R

_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2)}


def safetensors_name(graph_name: str, present) -> str | None:
    """Checkpoint name of a graph tensor (safeKey, prototypes/decode_graph.ts:99-109): the tied table and the final
    norm have fixed names, `model.layers.L.x` is looked up as `model.language_model.layers.L.x` first, then as is."""
    if graph_name in ("embed.weight", "lm_head.weight"):
        cand = "model.language_model.embed_tokens.weight"
        return cand if cand in present else None
    if graph_name == "final.norm.weight":
        cand = "model.language_model.norm.weight"
        return cand if cand in present else None
    if graph_name.startswith("model."):
        pre = "model.language_model." + graph_name[len("model."):]
        if pre in present:
            return pre
    return graph_name if graph_name in present else None


def read_header(path: str):
    """-> ({name: {"dtype", "shape", "data_offsets"}}, offset of the data section)"""
    with open(path, "rb") as f:
        (hl,) = struct.unpack("<Q", f.read(8))
        hdr = json.loads(f.read(hl).decode("utf-8"))
    hdr.pop("__metadata__", None)
    return hdr, 8 + hl


def write_safetensors(path: str, tensors: dict[str, np.ndarray], bf16_names=()) -> None:
    """Write a checkpoint: f32 / f16 arrays as they are, uint16 arrays named in bf16_names as BF16."""
    hdr, off, blobs = {}, 0, []
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint16 and name in bf16_names:
            dt = "BF16"
        elif a.dtype == np.float32:
            dt = "F32"
        elif a.dtype == np.float16:
            dt = "F16"
        else:
            raise ValueError(f"{name}: dtype {a.dtype} has no safetensors counterpart here")
        hdr[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    js = json.dumps(hdr, separators=(",", ":")).encode("utf-8")
    js += b" " * (-len(js) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)


def _to_f32(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "F32":
        return a
    if dtype == "F16":
        return a.astype(np.float32)
    return (a.astype(np.uint32) << 16).view(np.float32)


def _to_bf16(a: np.ndarray, dtype: str) -> np.ndarray:
    """bf16 bit patterns (round to nearest even from f32 / f16)."""
    if dtype == "BF16":
        return a
    f = _to_f32(a, dtype)
    u = f.view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def shard_source(cfg: M.ModelConfig, name: str, a: np.ndarray, rank: int, n: int) -> np.ndarray:
    """This rank's part of an unquantised tensor `a` (shaped as tensor_specs gives it), cut as model.shard_plan says."""
    plan = M.shard_plan(cfg, name, rank, n)
    if plan is None:
        return a
    if plan[0] == "rows":
        return np.ascontiguousarray(a[plan[1]])
    return np.ascontiguousarray(a[:, plan[1]:plan[2]])


def load_model(cfg: M.ModelConfig, path: str, batch: int = 1, device: int = 0, step_mode: int = 0,
               tp_rank: int = 0, tp_size: int = 1) -> M.DecodeModel:
    """Build the decode model of `cfg` from the checkpoint at `path`.  Linear weights may be BF16, F16 or F32 and are
    quantised to Q4_K on the device; norm weights, conv taps and dt_bias become bf16, A_log and the GDN norm f32
    (their dtypes in tensor_specs).  With tp_size > 1 this rank loads its shard only (torch.distributed must already
    be initialised, as for DecodeModel).  Raises KeyError for a missing tensor and ValueError for a wrong shape."""
    R.cu(device)
    hdr, data0 = read_header(path)
    full_specs = M.tensor_specs(cfg)
    specs = []   # (name, kind, shape of this rank's shard)
    for name, kind, shape in full_specs:
        probe = shard_source(cfg, name, np.empty(shape, np.bool_), tp_rank, tp_size) if tp_size > 1 else None
        specs.append((name, kind, tuple(probe.shape) if probe is not None else shape))
    full_shape = {name: shape for name, _, shape in full_specs}
    sizes = {}
    for name, kind, shape in specs:
        n = int(np.prod(shape))
        sizes[name] = shape[0] * (shape[1] // 256) * 144 if kind == "q4k" else n * (4 if kind == "f32" else 2)
    offs, total = {}, 0
    for name, _, _ in specs:
        offs[name] = total
        total += (sizes[name] + 255) // 256 * 256
    slab = R.DeviceBuffer(total)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    stage = None
    for name, kind, shape in specs:
        key = safetensors_name(name, hdr)
        if key is None:
            slab.free()
            raise KeyError(f"checkpoint {path} has no tensor for '{name}'")
        ent = hdr[key]
        np_dt, esz = _DTYPES[ent["dtype"]]
        if int(np.prod(ent["shape"])) != int(np.prod(full_shape[name])):
            slab.free()
            raise ValueError(f"{key}: shape {ent['shape']} does not hold the {full_shape[name]} of '{name}'")
        b0, b1 = ent["data_offsets"]
        raw = np.frombuffer(mm[data0 + b0:data0 + b1], dtype=np_dt)
        if tp_size > 1:
            raw = shard_source(cfg, name, raw.reshape(full_shape[name]), tp_rank, tp_size).reshape(-1)
        if kind == "q4k":
            # upload as f32 or bf16 and quantise on the device, straight into the slab
            src = raw.astype(np.float32) if ent["dtype"] == "F16" else raw
            if stage is None or stage.nbytes < src.nbytes:
                if stage is not None:
                    stage.free()
                stage = R.DeviceBuffer(src.nbytes)
            R.cuHtoD(stage.ptr, np.ascontiguousarray(src))
            ops.quantize_q4k(stage.ptr, shape[0], shape[1], slab.ptr + offs[name], bf16=(ent["dtype"] == "BF16"))
            assert R.cuSync() == 0, R.last_error()
        elif kind == "f32":
            R.cuHtoD(slab.ptr + offs[name], np.ascontiguousarray(_to_f32(raw, ent["dtype"])))
        else:
            R.cuHtoD(slab.ptr + offs[name], np.ascontiguousarray(_to_bf16(raw, ent["dtype"])))
    if stage is not None:
        stage.free()
    del mm
    ptrs = {name: (slab.ptr + offs[name], sizes[name]) for name, _, _ in specs}
    return M.DecodeModel.from_device(cfg, ptrs, slab, batch=batch, device=device, step_mode=step_mode, tp_rank=tp_rank,
                                     tp_size=tp_size)
