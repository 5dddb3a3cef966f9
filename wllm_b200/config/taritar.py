"""Taritar configuration, read from its own config.json keys.

    architecture     "Taritar"
    vocab, width     sizes of the vocabulary and of the residual stream
    max_positions    rows of the learned position table `pos` (a sequence holds no more tokens)
    embedding.scale  factor on the token's embedding row
    streams          copies of the residual stream that the layers read and write through learned weights
                     (absent: one plain residual stream and no such weights)
    norm.eps         the eps of every root-mean-square norm
    logit_softcap    c: logits become c * tanh(logits / c) (absent: as they are)
    layers[i]        {"type": "attention", "mixer": {...}, "mlp": {...} or null}

Mixer: heads, kv_heads (default heads), dim, vdim (default dim), scale (default dim^-1/2), softcap (absent: none),
rot {dims, base} (absent: no rotation), mask {size, keep_first} (absent: every earlier key is seen; keep_first
defaults to 0), kv_from: j (the layer has no key and value projections and reads layer j's cache).
mlp: {"kind": "dense", "ff", "limit"} or {"kind": "moe", "expert": {ff, limit}, "router": {experts, top, groups:
{count, keep} (absent: one group)}, "shared": {ff, limit} (absent: no shared expert)}.
Whatever a config.json leaves out does not exist.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .base import ConfigError, ConfigReader


def _sub(r: ConfigReader, raw, where: str):
    if not isinstance(raw, dict):
        r.complain(f"{where} must be an object")
        return None
    return ConfigReader(raw, where)


def _take(r: ConfigReader, sub: ConfigReader) -> None:
    r.problems.extend(f"{sub.where}: {p}" for p in sub.problems)
    sub.problems = []


def _gated(r: ConfigReader, raw, where: str) -> dict:
    sub = _sub(r, raw, where)
    if sub is None:
        return {}
    out = {"ff": sub.integer("ff"), "limit": sub.number("limit")}
    _take(r, sub)
    return out


def _mixer(r: ConfigReader, raw, where: str, index: int) -> dict:
    sub = _sub(r, raw, where)
    if sub is None:
        return {}
    heads, dim = sub.integer("heads"), sub.integer("dim")
    out = {"heads": heads, "kv_heads": sub.integer("kv_heads", default=heads), "dim": dim,
           "vdim": sub.integer("vdim", default=dim),
           "scale": sub.number("scale", default=(float(dim) ** -0.5 if dim else None))}
    cap = sub.number("softcap", default=None)
    if cap is not None:
        out["softcap"] = cap
    src = sub.optional_integer("kv_from")
    if src is not None:
        if not 0 <= src < index:
            r.complain(f"{where}.kv_from = {src}: an earlier layer")
        out["kv_from"] = src
    _take(r, sub)
    if heads and out["kv_heads"] and heads % out["kv_heads"]:
        r.complain(f"{where}: {heads} heads are no multiple of {out['kv_heads']} kv_heads")
    if raw.get("rot") is not None:
        rot = _sub(r, raw["rot"], where + ".rot")
        if rot is not None:
            dims, base = rot.integer("dims", minimum=0), rot.number("base")
            _take(r, rot)
            if dims is not None and dim and (dims % 2 or dims > dim):
                r.complain(f"{where}.rot.dims = {dims}: even and at most dim {dim}")
            out["rot"] = {"dims": dims, "base": base}
    if raw.get("mask") is not None:
        mask = _sub(r, raw["mask"], where + ".mask")
        if mask is not None:
            out["mask"] = {"size": mask.integer("size"), "keep_first": mask.integer("keep_first", default=0, minimum=0)}
            _take(r, mask)
    return out


def _mlp(r: ConfigReader, raw, where: str):
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") not in ("dense", "moe"):
        r.complain(f"{where}.kind must be 'dense' or 'moe' (or mlp null)")
        return None
    if raw["kind"] == "dense":
        return {"kind": "dense", **_gated(r, raw, where)}
    out = {"kind": "moe", "expert": _gated(r, raw.get("expert"), where + ".expert")}
    router = _sub(r, raw.get("router"), where + ".router")
    if router is not None:
        experts, top = router.integer("experts"), router.integer("top")
        out["router"] = {"experts": experts, "top": top}
        _take(r, router)
        count = keep = 1
        if raw["router"].get("groups") is not None:
            groups = _sub(r, raw["router"]["groups"], where + ".router.groups")
            if groups is not None:
                count, keep = groups.integer("count"), groups.integer("keep")
                _take(r, groups)
                out["router"]["groups"] = {"count": count, "keep": keep}
        if None not in (experts, top, count, keep):
            if experts % count:
                r.complain(f"{where}.router: {experts} experts do not form {count} equal groups")
            elif keep > count or top > keep * (experts // count):
                r.complain(f"{where}.router: top {top} of {keep} groups of {experts // count} experts, out of {count} groups")
    if raw.get("shared") is not None:
        out["shared"] = _gated(r, raw["shared"], where + ".shared")
    return out


@dataclass(frozen=True)
class TaritarConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    streams: int | None
    eps: float
    logit_softcap: float | None
    layers: tuple            # of checked layer dictionaries (see the module's text)

    architecture = "Taritar"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "TaritarConfig":
        r = ConfigReader(raw, where)
        vocab, width, max_positions = r.integer("vocab"), r.integer("width"), r.integer("max_positions")
        streams = r.integer("streams", default=None)
        cap = r.number("logit_softcap", default=None)
        eps = scale = None
        norm = _sub(r, raw.get("norm"), "norm")
        if norm is not None:
            eps = norm.number("eps")
            _take(r, norm)
        emb = _sub(r, raw.get("embedding"), "embedding")
        if emb is not None:
            scale = emb.number("scale", default=1.0)
            _take(r, emb)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            r.complain("'layers' must be a list with at least one layer")
            layers = []
        checked = []
        for i, layer in enumerate(layers):
            here = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") != "attention":
                r.complain(f"{here}.type must be 'attention'")
                checked.append({})
                continue
            one = {"type": "attention", "mixer": _mixer(r, layer.get("mixer"), here + ".mixer", i),
                   "mlp": _mlp(r, layer.get("mlp"), here + ".mlp")}
            src = one["mixer"].get("kv_from")
            if src is not None and src < len(checked) and checked[src]:
                theirs = checked[src].get("mixer", {})
                if theirs.get("kv_from") is not None:
                    r.complain(f"{here}.mixer.kv_from = {src}: that layer has no keys and values of its own")
                for key in ("kv_heads", "dim", "vdim", "rot"):
                    if theirs.get(key) != one["mixer"].get(key):
                        r.complain(f"{here}.mixer.{key} differs from layer {src}'s, whose keys and values it reads")
            checked.append(one)
        r.finish()
        return cls(vocab=vocab, width=width, max_positions=max_positions, embedding_scale=scale, streams=streams, eps=eps,
                   logit_softcap=cap, layers=tuple(checked))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
             "norm": {"eps": self.eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d


__all__ = ["TaritarConfig", "ConfigError"]
