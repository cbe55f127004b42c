"""Checkpoint directories: config.json + model.safetensors -> a B200Model of the kind the config names.

The safetensors container is read here directly (8-byte little-endian header length, a JSON header name -> dtype / shape /
data_offsets, then the tensor bytes); bfloat16 tensors stay bfloat16 bit patterns (numpy has no such dtype) and cross the C ABI
tagged as AHA_BF16."""
import json
import os
import struct

import numpy as np

from . import _lib as L

_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64, "U8": np.uint8}


def read_safetensors(path):
    """name -> numpy array (bf16 tensors as uint16 bit patterns tagged `_lib.BF16`)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, e = meta["data_offsets"]
        raw = blob[8 + n + a:8 + n + e]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            out[name] = np.frombuffer(raw, np.uint16).reshape(shape).copy().view(L.BF16)
        elif meta["dtype"] in _DTYPES:
            arr = np.frombuffer(raw, _DTYPES[meta["dtype"]]).reshape(shape).copy()
            out[name] = arr.astype(np.float32) if meta["dtype"] == "I32" else arr
        else:
            raise ValueError(f"{path}: tensor '{name}' has unsupported dtype {meta['dtype']}")
    return out


def write_safetensors(path, tensors):
    """The inverse, for synthetic checkpoints: float32 / float16 arrays as they are, `_lib.BF16`-tagged arrays as BF16."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        if isinstance(a, L.BF16):
            dt, raw = "BF16", np.ascontiguousarray(a.view(np.ndarray)).tobytes()
        else:
            a = np.ascontiguousarray(a)
            dt = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.int32): "I32"}[a.dtype]
            raw = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def model_kind(config):
    """Which executor a config.json asks for."""
    arch = config.get("architecture")
    if isinstance(arch, str) and arch.lower() in ("malasun", "gatuzen", "lupolorn", "gomerax"):      # designs of the layered engine: config.json lists the layers
        return arch.lower()
    names = " ".join(config.get("architectures", []) + [config.get("model_type", "")]).lower()
    if "qwen3_asr" in names or "qwen3asr" in names or "thinker_config" in config:
        return "qwen3_asr"
    if "qwen3vl" in names or "qwen3_vl" in names or "vision_config" in config:
        return "qwen3vl"
    if "qwen3" in names:
        return "qwen3"
    raise ValueError("config.json names no architecture this library serves")


def load_model(model_dir, **options):
    """B200Model for the checkpoint in `model_dir`; options go to B200Model (max_ctx, max_prefill, max_seqs, exact_fp32, ...)."""
    from .inference import B200Model
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    eos = options.pop("eos_ids", None)
    if eos is None:
        e = config.get("eos_token_id", [])
        eos = e if isinstance(e, list) else [e]
    return B200Model(model_kind(config), config, weights, eos_ids=eos, **options)
