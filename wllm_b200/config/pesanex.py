"""Pesanex configuration, read from its own config.json keys.

    architecture   "Pesanex"
    vocab, width   sizes of the vocabulary and of the residual stream
    norm.eps       the eps of every norm of the model (layer norms, unit and gained root-mean-square norms)
    layers[i]      {"type": "retention" | "gla" | "parallel", "mixer": sizes of the mixer, "mlp": {"kind": "dense",
                   "ff": n} or null}
    loop           {"start", "stop", "times"}: layers start .. stop-1 run `times` times in a row with the same weights
                   (every pass with a cache and state of its own), then the rest follow; absent: every layer once

Mixer sizes: retention {heads, dim, vdim, decay: [one per head], rot: {dims, base} or absent}; gla {heads, dim, vdim,
tau, and optionally rank, else the checkpoint's shapes give it}; parallel {left: {heads, kv_heads, dim, vdim, scale,
rot}, right: a gla mixer}.  Whatever a config.json leaves out does not exist: no rotation without `rot`, every layer
once without `loop`.  Positions have no upper bound.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .base import ConfigError, ConfigReader

MIXER_TYPES = ("retention", "gla", "parallel")


def _rot(r: ConfigReader, raw: dict, dim: int, where: str):
    rot = raw.get("rot")
    if rot is None:
        return None
    if not isinstance(rot, dict):
        r.complain(f"{where}.rot must be an object")
        return None
    sub = ConfigReader(rot, where + ".rot")
    dims, base = sub.integer("dims", minimum=0), sub.number("base")
    r.problems.extend(f"{where}.rot: {p}" for p in sub.problems)
    if dims is not None and (dims % 2 or dims > dim):
        r.complain(f"{where}.rot.dims = {dims}: even and at most dim {dim}")
    return {"dims": dims, "base": base}


def _linear_sizes(r: ConfigReader, raw, where: str) -> dict:
    if not isinstance(raw, dict):
        r.complain(f"{where} must be an object")
        return {}
    sub = ConfigReader(raw, where)
    out = {"heads": sub.integer("heads"), "dim": sub.integer("dim"), "vdim": sub.integer("vdim")}
    r.problems.extend(f"{where}: {p}" for p in sub.problems)
    return out


def _check_layer(r: ConfigReader, i: int, layer) -> dict:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
        r.complain(f"{where}.type must be one of {', '.join(MIXER_TYPES)}")
        return {}
    kind, m = layer["type"], layer.get("mixer")
    out = {"type": kind, "mixer": {}, "mlp": None}

    def gla(raw, where):
        sizes = _linear_sizes(r, raw, where)
        sub = ConfigReader(raw if isinstance(raw, dict) else {}, where)
        sizes["tau"] = sub.number("tau")
        rank = sub.optional_integer("rank")
        if rank is not None:
            sizes["rank"] = rank
        r.problems.extend(f"{where}: {p}" for p in sub.problems)
        return sizes
    if kind == "retention":
        sizes = _linear_sizes(r, m, where + ".mixer")
        decay = (m or {}).get("decay") if isinstance(m, dict) else None
        if not isinstance(decay, list) or len(decay) != sizes.get("heads") or \
                not all(isinstance(a, (int, float)) and not isinstance(a, bool) for a in decay):
            r.complain(f"{where}.mixer.decay must list one number per head")
            decay = []
        sizes["decay"] = [float(a) for a in decay]
        rot = _rot(r, m if isinstance(m, dict) else {}, sizes.get("dim") or 0, where + ".mixer")
        if rot is not None:
            sizes["rot"] = rot
        out["mixer"] = sizes
    elif kind == "gla":
        out["mixer"] = gla(m, where + ".mixer")
    else:
        if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
            r.complain(f"{where}.mixer must hold 'left' and 'right'")
            return out
        left = _linear_sizes(r, m["left"], where + ".mixer.left")
        sub = ConfigReader(m["left"], where + ".mixer.left")
        left["kv_heads"] = sub.integer("kv_heads", default=left.get("heads"))
        left["scale"] = sub.number("scale", default=(float(left["dim"]) ** -0.5 if left.get("dim") else None))
        r.problems.extend(f"{where}.mixer.left: {p}" for p in sub.problems)
        if left.get("heads") and left.get("kv_heads") and left["heads"] % left["kv_heads"]:
            r.complain(f"{where}.mixer.left: {left['heads']} heads are no multiple of {left['kv_heads']} kv_heads")
        rot = _rot(r, m["left"], left.get("dim") or 0, where + ".mixer.left")
        if rot is not None:
            left["rot"] = rot
        out["mixer"] = {"left": left, "right": gla(m["right"], where + ".mixer.right")}
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            r.complain(f"{where}.mlp.kind must be 'dense' (or mlp null)")
        else:
            sub = ConfigReader(mlp, where + ".mlp")
            out["mlp"] = {"kind": "dense", "ff": sub.integer("ff")}
            r.problems.extend(f"{where}.mlp: {p}" for p in sub.problems)
    return out


@dataclass(frozen=True)
class PesanexConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple           # of checked layer dictionaries (see the module's text)
    loop: tuple | None      # (start, stop, times)

    architecture = "Pesanex"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "PesanexConfig":
        r = ConfigReader(raw, where)
        vocab, width = r.integer("vocab"), r.integer("width")
        norm = raw.get("norm")
        eps = None
        if not isinstance(norm, dict):
            r.complain("missing object 'norm' with key 'eps'")
        else:
            sub = ConfigReader(norm, "norm")
            eps = sub.number("eps")
            r.problems.extend(f"norm: {p}" for p in sub.problems)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            r.complain("'layers' must be a list with at least one layer")
            layers = []
        checked = tuple(_check_layer(r, i, layer) for i, layer in enumerate(layers))
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                r.complain("'loop' must be an object")
                loop = None
            else:
                sub = ConfigReader(loop, "loop")
                start, stop, times = sub.integer("start", minimum=0), sub.integer("stop", minimum=0), sub.integer("times", minimum=1)
                r.problems.extend(f"loop: {p}" for p in sub.problems)
                loop = (start, stop, times)
                if None not in loop and not 0 <= start <= stop <= len(layers):
                    r.complain(f"loop: 0 <= start <= stop <= {len(layers)} layers")
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, layers=checked, loop=loop)

    def order(self) -> list:
        """The layers in the order in which they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d
