"""Small Pesanex configurations for the tests, as config.json dictionaries, and folders of seeded weights for them.

They differ from one another in every size and option: which mixers there are and in which order, feed-forward or none
behind each kind of mixer, a loop (none; one that repeats two layers three times; one that runs once), grouped and
ungrouped query heads, key and value sizes that differ and that are equal, rotation over a part of a head, over all
of it and none, decays far from 1, tau of 1, odd vocabularies, eps.
"""
import copy
import json
import os

import torch
from safetensors.torch import save_file

ROT_A = {"dims": 16, "base": 10000.0}

MIX = {
    "architecture": "Pesanex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 160},
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "rot": ROT_A},
                   "right": {"heads": 3, "dim": 24, "vdim": 40, "tau": 4.0, "rank": 8}}},
        {"type": "retention", "mlp": {"kind": "dense", "ff": 72},
         "mixer": {"heads": 2, "dim": 24, "vdim": 48, "decay": [0.9, 0.995], "rot": {"dims": 8, "base": 500.0}}},
        {"type": "gla", "mlp": None, "mixer": {"heads": 2, "dim": 40, "vdim": 24, "tau": 8.0, "rank": 4}},
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

PLAIN = {
    "architecture": "Pesanex", "vocab": 300, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "retention", "mlp": None, "mixer": {"heads": 4, "dim": 16, "vdim": 16, "decay": [0.5, 0.8, 0.97, 1.0]}},
        {"type": "parallel", "mlp": None,
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.5, "rot": {"dims": 64, "base": 100.0}},
                   "right": {"heads": 1, "dim": 32, "vdim": 32, "tau": 1.0, "rank": 16}}},
        {"type": "gla", "mlp": {"kind": "dense", "ff": 128}, "mixer": {"heads": 4, "dim": 8, "vdim": 32, "tau": 2.0, "rank": 2}},
    ],
}

ONCE = {   # a loop that runs its layers once, a left mixer without rotation, one head everywhere
    "architecture": "Pesanex", "vocab": 97, "width": 48, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "gla", "mlp": None, "mixer": {"heads": 1, "dim": 48, "vdim": 16, "tau": 16.0, "rank": 3}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 40},
         "mixer": {"left": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 48, "scale": 1.0},
                   "right": {"heads": 2, "dim": 16, "vdim": 8, "tau": 3.0, "rank": 5}}},
    ],
    "loop": {"start": 0, "stop": 2, "times": 1},
}

ODD = {    # sizes that are multiples of little: a width and a feed-forward that are no multiples of 8, key sizes that are no
           # multiples of 4 or 16, three query heads on one key/value head, a loop over the first layer alone
    "architecture": "Pesanex", "vocab": 77, "width": 100, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "gla", "mlp": {"kind": "dense", "ff": 50}, "mixer": {"heads": 3, "dim": 18, "vdim": 12, "tau": 5.0, "rank": 3}},
        {"type": "retention", "mlp": None,
         "mixer": {"heads": 2, "dim": 20, "vdim": 36, "decay": [0.75, 0.98], "rot": {"dims": 10, "base": 77.0}}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 36},
         "mixer": {"left": {"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 8, "scale": 0.3, "rot": {"dims": 12, "base": 1000.0}},
                   "right": {"heads": 1, "dim": 70, "vdim": 66, "tau": 2.5, "rank": 7}}},
    ],
    "loop": {"start": 0, "stop": 1, "times": 2},
}

CONFIGS = {"mix": MIX, "plain": PLAIN, "once": ONCE, "odd": ODD}
SEEDS = {"mix": 5, "plain": 9, "once": 13, "odd": 17}


def write_folder(folder: str, name: str, dtype=torch.bfloat16) -> str:
    """config.json and model.safetensors of a test configuration.  Matrices N(0, 0.08); gains around 1; the numbers
    that random weights would leave near zero are spread so that they matter: sinks over [-2, 4], decay biases over
    [-3, 5] (decays from 0.5 to nearly 1)."""
    from wllm_b200.weights import random_tensors
    cfg = copy.deepcopy(CONFIGS[name])
    tensors = random_tensors(cfg, SEEDS[name], dtype=torch.float32, std=0.08, vector_std=0.3)
    g = torch.Generator().manual_seed(SEEDS[name] + 1000)
    for key, t in tensors.items():
        if key.endswith(".sink"):
            tensors[key] = torch.rand(t.shape, generator=g) * 6.0 - 2.0
        elif key.endswith(".a2.b"):
            tensors[key] = torch.rand(t.shape, generator=g) * 8.0 - 3.0
        elif t.dim() == 1:
            tensors[key] = 1.0 + t               # gains
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
