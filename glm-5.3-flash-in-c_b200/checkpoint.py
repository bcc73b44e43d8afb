"""Checkpoint side of the loader contract: config.json -> Config, safetensors -> named tensors.

Tensor names, dtypes and shapes are the released checkpoint's, as the reference binds them
(src/model/glm53f_bind.c:139-206,311-317; src/io/glm53f_load.c:11-63); the config fields are
the ones the reference's strict reader takes (include/glm53f/glm53f_cfg.h:95-294). The engine
receives tensors by name below the prefix ``model.language_model.`` (``lm_head.weight`` has no
prefix in the checkpoint).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

from . import DT_BF16, DT_F32, DT_FP8, Config

PREFIX = "model.language_model."
_ST_DTYPES = {"F32": (np.float32, DT_F32), "BF16": (np.uint16, DT_BF16), "F8_E4M3": (np.uint8, DT_FP8)}


def read_config(path_or_dict):
    """config.json (a path, or its parsed content) -> (Config, is_mla list, is_dense list, eos ids)."""
    if isinstance(path_or_dict, dict):
        top = path_or_dict
    else:
        with open(path_or_dict) as f:
            top = json.load(f)
    t = top.get("text_config", top)
    q = top.get("quantization_config") or {}
    la = t["linear_attn_config"]
    blk = q.get("weight_block_size") or [0, 0]
    cfg = Config(
        hidden=t["hidden_size"], n_layers=t["num_hidden_layers"], vocab=t["vocab_size"],
        rms_eps=t["rms_norm_eps"], hc_mult=t["hc_mult"], hc_iters=t["hc_sinkhorn_iters"], hc_eps=t["hc_eps"],
        kda_heads=la["num_heads"], kda_head_dim=la["head_dim"], conv_k=la["short_conv_kernel_size"],
        gate_lb=la["gate_lower_bound"], mla_heads=t["num_attention_heads"], q_lora=t["q_lora_rank"],
        kv_lora=t["kv_lora_rank"], qk_nope=t["qk_nope_head_dim"], v_head=t["v_head_dim"],
        index_topk=t["index_topk"], index_kpool=t["index_kpool"], index_heads=t["index_n_heads"],
        index_dim=t["index_head_dim"], n_experts=t["n_routed_experts"], topk=t["num_experts_per_tok"],
        n_shared=t["n_shared_experts"], moe_inter=t["moe_intermediate_size"],
        dense_inter=t["intermediate_size"], routed_scale=t["routed_scaling_factor"],
        norm_topk=1 if t.get("norm_topk_prob", True) else 0, swiglu_limit=t["swiglu_limit"],
        fp8_block_r=blk[0], fp8_block_c=blk[1])
    is_mla = [0 if lt == "linear_attention" else 1 for lt in t["layer_types"]]
    is_dense = [1 if mt == "dense" else 0 for mt in t["mlp_layer_types"]]
    eos = t.get("eos_token_id", [])
    return cfg, is_mla, is_dense, (eos if isinstance(eos, list) else [eos])


def read_safetensors(path: str) -> dict:
    """One .safetensors file -> {full name: (array, dtype code)}; BF16 as uint16 bit patterns,
    FP8 as uint8 codes. Format: 8-byte little-endian header length, JSON header, raw data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        blob = np.fromfile(path, dtype=np.uint8, offset=base)
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _ST_DTYPES:
            raise ValueError(f"{name}: dtype {meta['dtype']} is not part of this architecture")
        npdt, code = _ST_DTYPES[meta["dtype"]]
        a, b = meta["data_offsets"]
        arr = blob[a:b].view(npdt).reshape(meta["shape"])
        out[name] = (arr, code)
    return out


def read_checkpoint(directory: str) -> dict:
    """All shards of a checkpoint directory -> {engine name: (array, dtype, scale or None)}.
    `_scale_inv` grids are attached to their FP8 tensor; conv kernels [n][1][k] become [n][k]."""
    raw = {}
    for fn in sorted(os.listdir(directory)):
        if fn.endswith(".safetensors"):
            raw.update(read_safetensors(os.path.join(directory, fn)))
    out = {}
    for name, (arr, code) in raw.items():
        if name.endswith("_scale_inv"):
            continue
        short = name[len(PREFIX):] if name.startswith(PREFIX) else name
        scale = None
        if code == DT_FP8:
            if name + "_scale_inv" not in raw:
                raise ValueError(f"{name} is FP8 but has no {name}_scale_inv")
            scale = np.ascontiguousarray(raw[name + "_scale_inv"][0], dtype=np.float32)
        if arr.ndim == 3:
            arr = arr.reshape(arr.shape[0], arr.shape[2])
        out[short] = (np.ascontiguousarray(arr), code, scale)
    return out


def write_safetensors(path: str, tensors: dict):
    """{full name: (array, st dtype string)} -> one .safetensors file (fixture generation)."""
    header, chunks, off = {}, [], 0
    for name, (arr, st) in tensors.items():
        b = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": st, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        chunks.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in chunks:
            f.write(b)
