"""Small Taritar configurations for the tests, and folders with weights made so that every mechanism matters.

'wide'   three streams; grouped heads with value heads of their own size, a partial rotation, a score cap, a window that
         keeps first keys; a dense layer, a layer of routed experts (groups, a shared expert), a layer without a
         feed-forward that reads an earlier layer's keys and values under a wider mask of its own, and a layer that sees
         every key, has no cap and no rotation, and routes to one expert without groups or a shared one
'one'    a single stream (all connection tensors of size one); windows no longer than a page, kept keys equal to the
         window and beyond it, one key/value head, heads of 28 elements (held as 32 with zeros behind them)
'odd'    sizes in no step of 4 or 8 (width 50, heads of 10 and 6, feed-forwards of 30, 14 and 10, nine experts), five streams,
         a layer with fewer query heads than the layer whose keys and values it reads
'heads128'  heads of 128 elements, whose prompts of more than 64 tokens run on the tensor-memory attention of pairs of CTAs
'plain'  no streams at all (a plain residual), no logit cap, one expert group kept of one, heads of 12 and 20 elements
"""
from __future__ import annotations

import copy
import json
import os

import torch
from safetensors.torch import save_file


def _att(heads, kv, dim, vdim=None, rot=None, scale=None, cap=None, mask=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim}
    if vdim is not None:
        m["vdim"] = vdim
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if scale is not None:
        m["scale"] = scale
    if cap is not None:
        m["softcap"] = cap
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, limit, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


WIDE = {
    "architecture": "Taritar", "vocab": 200, "width": 64, "max_positions": 400, "streams": 3, "logit_softcap": 9.0,
    "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 16, 24, (8, 500.0), 0.3, 5.0, (40, 5)), "mlp": {"kind": "dense", "ff": 48, "limit": 0.8}},
        {"type": "attention", "mixer": _att(4, 2, 16, 24, (8, 500.0), 0.3, 5.0, (24, 0)),
         "mlp": _moe(8, 2, 24, 1.2, groups=(4, 2), shared=(40, 0.9))},
        {"type": "attention", "mixer": _att(4, 2, 16, 24, (8, 500.0), 0.2, 3.0, (70, 17), kv_from=1), "mlp": None},
        {"type": "attention", "mixer": _att(2, 1, 32), "mlp": _moe(5, 1, 16, 2.5)},
    ],
}

ONE = {
    "architecture": "Taritar", "vocab": 90, "width": 40, "max_positions": 300, "streams": 1, "logit_softcap": 30.0,
    "embedding": {"scale": 0.25}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(2, 1, 28, None, (28, 10000.0), None, 8.0, (16, 16)), "mlp": {"kind": "dense", "ff": 56, "limit": 3.0}},
        {"type": "attention", "mixer": _att(2, 1, 28, None, (28, 10000.0), 0.5, None, (8, 33), kv_from=0),
         "mlp": _moe(6, 3, 8, 0.7, groups=(2, 1), shared=(8, 1.0))},
        {"type": "attention", "mixer": _att(1, 1, 8, 16, (2, 50.0), None, 2.0, (13, 1)), "mlp": {"kind": "dense", "ff": 24, "limit": 1.5}},
    ],
}

PLAIN = {
    "architecture": "Taritar", "vocab": 64, "width": 48, "max_positions": 256,
    "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(3, 3, 12, 20, (6, 100.0), None, 10.0, (20, 3)), "mlp": _moe(4, 2, 16, 1.0, groups=(1, 1))},
        {"type": "attention", "mixer": _att(3, 3, 12, 20, (6, 100.0), None, 10.0, (64, 0), kv_from=0), "mlp": {"kind": "dense", "ff": 32, "limit": 1.0}},
    ],
}

ODD = {
    "architecture": "Taritar", "vocab": 77, "width": 50, "max_positions": 260, "streams": 5, "logit_softcap": 4.0,
    "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(6, 2, 10, 6, (4, 30.0), 0.35, 7.0, (33, 2)), "mlp": _moe(9, 3, 10, 1.1, groups=(3, 2), shared=(14, 0.6))},
        {"type": "attention", "mixer": _att(2, 2, 10, 6, (4, 30.0), 0.35, 7.0, (50, 31), kv_from=0), "mlp": {"kind": "dense", "ff": 30, "limit": 0.9}},
    ],
}

HEADS128 = {
    "architecture": "Taritar", "vocab": 120, "width": 64, "max_positions": 300, "streams": 2, "logit_softcap": 12.0,
    "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 128, None, (64, 10000.0), 0.08, 6.0, (40, 5)), "mlp": {"kind": "dense", "ff": 40, "limit": 1.0}},
        {"type": "attention", "mixer": _att(4, 2, 128, None, (64, 10000.0), 0.08, 6.0, (23, 18), kv_from=0), "mlp": None},
    ],
}

CONFIGS = {"wide": WIDE, "one": ONE, "plain": PLAIN, "odd": ODD, "heads128": HEADS128}
SEEDS = {"wide": 21, "one": 22, "plain": 23, "odd": 24, "heads128": 25}


def write_folder(folder: str, name: str, dtype=torch.bfloat16) -> str:
    """config.json and model.safetensors.  Matrices N(0, 0.1) and position rows N(0, 0.3); gains around 1; connection
    weights that keep the streams apart (in and out around 0.8, mix the identity plus noise); routers and shared gates
    large enough that the choice of experts is no close call."""
    from wllm_b200.weights import random_tensors
    cfg = copy.deepcopy(CONFIGS[name])
    tensors = random_tensors(cfg, SEEDS[name], dtype=torch.float32, std=0.1, vector_std=0.3)
    g = torch.Generator().manual_seed(SEEDS[name] + 1000)
    for key, t in tensors.items():
        if key.endswith((".in", ".out")):
            tensors[key] = 0.8 + 0.4 * torch.randn(t.shape, generator=g)
        elif key.endswith(".mix"):
            tensors[key] = torch.eye(t.shape[0]) + 0.3 * torch.randn(t.shape, generator=g)
        elif key.endswith((".router", ".sg")):
            tensors[key] = torch.randn(t.shape, generator=g) * 0.8
        elif key == "pos":
            tensors[key] = torch.randn(t.shape, generator=g) * 0.3
        elif t.dim() == 1:
            tensors[key] = 1.0 + t
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
