"""Taritar in plain, slow PyTorch: the statement the engine is held against.

One function per mechanism, whole sequences only, no cache, no batching, nothing shared with the package.  `cfg` is
the raw config.json dictionary, `w` maps tensor names to tensors; everything runs in the type of the weights it is
given (the tests pass float32 or float64 copies).

    embedding       x[p] = embed[token] * embedding.scale + pos[p]
    streams         s copies of x; sublayer q of a layer reads u = sum_s in[s] x_s, and with y = sublayer(norm(u))
                    every stream becomes x_t' = sum_s mix[s, t] x_s + out[t] y; the model's output is sum_s x_s
    attention       grouped heads, rotary turn of the pairs (2i, 2i+1) over the first rot.dims elements of a head,
                    score = cap * tanh(scale * q.k / cap), key j visible to i when j <= i and (i - j < size or
                    j < keep_first), softmax, output projection; a layer with kv_from reads that layer's keys, values
    feed-forward    g = min(gate h, limit), u = clamp(up h, +-limit), down(g * sigmoid(1.702 g) * (u + 1))
    experts         softmax over all router logits; groups of neighbouring experts are ranked by their best score and
                    only the best `keep` groups stay; the `top` best experts of those are run and weighted by their
                    scores as they are; a shared expert is added, times sigmoid(sg . h)
    head            final norm, logits = head x, then cap * tanh(logits / cap)
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def embed(cfg, w, tokens):
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    return w["embed"][ids] * cfg["embedding"]["scale"] + w["pos"][pos]


def rotate_interleaved(x, positions, dims, base):
    """x: [n, heads, dim]; the pairs (2i, 2i+1), i < dims/2, turn by positions * base^(-2i/dims)."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).to(x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(n, size, keep_first):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def _rot(m):
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    return rot["dims"], rot["base"]


def keys_values(m, w, p, h):
    """Rotated keys [n, G, dim] and values [n, G, vdim] of the layer with prefix p from its input h."""
    n, G = h.shape[0], m.get("kv_heads", m["heads"])
    k = (h @ w[p + "k"].T).view(n, G, m["dim"])
    v = (h @ w[p + "v"].T).view(n, G, m.get("vdim", m["dim"]))
    return rotate_interleaved(k, torch.arange(n), *_rot(m)), v


def attention(m, w, p, h, kv):
    """m: the mixer's sizes; kv: (keys, values) as keys_values returns them (this layer's or another's)."""
    n, H, G = h.shape[0], m["heads"], m.get("kv_heads", m["heads"])
    q = rotate_interleaved((h @ w[p + "q"].T).view(n, H, m["dim"]), torch.arange(n), *_rot(m))
    k, v = kv
    mask = visible(n, m["mask"]["size"], m["mask"].get("keep_first", 0)) if m.get("mask") else visible(n, n, 0)
    scale = m["scale"] if m.get("scale") is not None else m["dim"] ** -0.5
    heads = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        s = s.masked_fill(~mask, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def capped_glu(w, p, h, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def route(scores, top, groups, keep):
    """scores [n, E] -> chosen experts [n, top] (indices): the best `top` among the experts of the best `keep` groups."""
    n, E = scores.shape
    per = E // groups
    best = scores.view(n, groups, per).max(-1).values
    kept = torch.topk(best, keep, dim=-1).indices
    allowed = torch.zeros(n, groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = scores.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    return torch.topk(masked, top, dim=-1).indices


def experts(mlp, w, p, h):
    r = mlp["router"]
    scores = torch.softmax((h.float() @ w[p + "router"].float().T), dim=-1)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen = route(scores, r["top"], groups["count"], groups["keep"])
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        rows, col = torch.nonzero(chosen == e, as_tuple=True)
        if rows.numel():
            y = capped_glu(w, f"{p}e{e}.", h[rows], mlp["expert"]["limit"])
            out[rows] += scores[rows, e].to(h.dtype)[:, None] * y
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)
        out = out + gate * capped_glu(w, p + "shared.", h, mlp["shared"]["limit"])
    return out


def feed_forward(mlp, w, p, h):
    if mlp["kind"] == "dense":
        return capped_glu(w, p, h, mlp["limit"])
    return experts(mlp, w, p, h)


def hyper_step(streams, w, p, sublayer):
    """streams [s, n, width]; p names the tensors in/out/mix of this sublayer's connections."""
    u = torch.einsum("s,snw->nw", w[p + "in"], streams)
    y = sublayer(u)
    return torch.einsum("st,snw->tnw", w[p + "mix"], streams) + w[p + "out"][:, None, None] * y[None]


def forward(cfg, w, tokens, layers_out=None):
    """Logits [n, vocab] of one whole sequence; `layers_out` (a list) receives the sum of the streams after each layer."""
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, tokens)
    bare = cfg.get("streams") is None                  # one plain residual: x <- x + sublayer(norm(x))
    if bare:
        w = dict(w)
        for i, layer in enumerate(cfg["layers"]):
            for q in ("hc1.", "hc2."):
                w[f"l{i}.{q}in"], w[f"l{i}.{q}out"], w[f"l{i}.{q}mix"] = x.new_ones(1), x.new_ones(1), x.new_ones(1, 1)
    streams = x[None].repeat(1 if bare else cfg["streams"], 1, 1)
    cache = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]

        def mixer(u, p=p, m=m, i=i):
            h = rms_norm(u, w[p + "norm1"], eps)
            if m.get("kv_from") is None:
                cache[i] = keys_values(m, w, p + "mix.", h)
            return attention(m, w, p + "mix.", h, cache[m["kv_from"] if m.get("kv_from") is not None else i])
        streams = hyper_step(streams, w, p + "hc1.", mixer)
        if layer.get("mlp") is not None:
            streams = hyper_step(streams, w, p + "hc2.",
                                 lambda u, p=p, layer=layer: feed_forward(layer["mlp"], w, p + "mlp.", rms_norm(u, w[p + "norm2"], eps)))
        if layers_out is not None:
            layers_out.append(streams.sum(0))
    x = rms_norm(streams.sum(0), w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
