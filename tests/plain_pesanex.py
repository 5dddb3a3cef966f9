"""Pesanex, stated plainly: whole sequences, no cache, no batching, one function per mechanism.

Everything is computed in the element type of the weights handed in (float64 in the tests), token by
token where the design is a recurrence, with sums written out as they are defined.  Nothing here is
shared with the engine.  `cfg` is the config.json dictionary of the design:

    width, vocab, norm.eps, layers[i] = {type, mixer, mlp}, loop = {start, stop, times}

Mechanisms:
    layer_norm          (x - mean) / sqrt(var + eps) * w
    unit_rms            x / sqrt(mean(x^2) + eps)
    rotate_half         rotary turn of the first `dims` elements of a head, pairs (i, i + dims/2)
    decayed_outer_scan  S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
    retention           fixed decay per head, rotary q and k, unit-RMS heads, SiLU gate
    gated_linear        decay per key channel from a low-rank map, RMS-normed heads, SiLU gate
    sink_attention      grouped causal softmax attention with unit-RMS q and k and a sink in the denominator
    parallel            mean of the two mixers' outputs, each RMS-normed over the width
    dense_relu          down(relu(gate x) * up x)
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, w, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def rotate_half(x, positions, dims, base):
    """x: [T, heads, dim]; the first `dims` elements of every head turn by position * base^(-2i/dims)."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]          # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def decayed_outer_scan(q, k, v, decay, state=None):
    """q, k: [T, heads, dim]; v: [T, heads, vdim]; decay: [T, heads, dim] (per key channel).
    Returns (o [T, heads, vdim], final state [heads, dim, vdim])."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out), S


def retention(h, w, p, m, eps, positions=None):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half(q, pos, rot["dims"], rot["base"])
    k = rotate_half(k, pos, rot["dims"], rot["base"]) * D ** -0.5
    decay = torch.tensor(m["decay"], dtype=h.dtype)[None, :, None].expand(T, H, D)
    o, _ = decayed_outer_scan(q, k, v, decay)
    o = unit_rms(o, eps).reshape(T, H * V)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def gated_linear(h, w, p, m, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z) ** (1.0 / m["tau"])
    o, _ = decayed_outer_scan(q, k, v, alpha.view(T, H, D))
    o = (unit_rms(o, eps) * w[p + "norm"]).reshape(T, H * V)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def sink_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = unit_rms(rotate_half(q, pos, rot["dims"], rot["base"]), eps)
    k = unit_rms(rotate_half(k, pos, rot["dims"], rot["base"]), eps)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, head]) * m["scale"]
            top = max(float(s.max()), float(w[p + "sink"][head]))
            e = torch.exp(s - top)
            denom = e.sum() + math.exp(float(w[p + "sink"][head]) - top)
            out[i, head] = (e[:, None] * v[: i + 1, g]).sum(0) / denom
    return out.reshape(T, H * V) @ w[p + "o"].T


def parallel(h, w, p, m, eps):
    left = sink_attention(h, w, p + "left.", m["left"], eps)
    right = gated_linear(h, w, p + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * w[p + "left.out"] + unit_rms(right, eps) * w[p + "right.out"])


def dense_relu(h, w, p):
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


MIXERS = {"retention": retention, "gla": gated_linear, "parallel": parallel}


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + \
        list(range(loop["stop"], n))


def forward(ids, w, cfg, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out` (a list) receives the residual after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids)]
    for i in layer_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        y = MIXERS[L["type"]](layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
        x = x + layer_norm(y, w[p + "norm1b"], eps)
        if L.get("mlp"):
            y = dense_relu(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + layer_norm(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x)
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
