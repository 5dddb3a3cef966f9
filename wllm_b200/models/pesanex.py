"""Pesanex as a plan of parts.

Every layer is a 'sandwich' block: a layer norm (gain, no bias) in front of and behind each sublayer.  The mixer is one
of three: retention (linear attention with one fixed decay per head and rotary q and k), gated linear attention
(decay per key channel from a low-rank map of the input), or the two side by side: softmax attention with grouped
heads, unit-norm q and k, a score scale of its own and a sink per head, beside a gated linear attention, their
outputs root-mean-square normed and averaged.  A layer may have a dense feed-forward with a ReLU gate, or none.  A
run of layers may be repeated with the same weights; every pass has its own cache and state.  Untied head, embedding
unscaled, no limit on positions.

Checkpoint names: embed, head, final.norm; layer i: l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.* (q k v g o, norm,
a1 a2 a2.b, sink, left.* right.* left.out right.out), l<i>.mlp.gate / up / down.
"""
from __future__ import annotations

from ..config.pesanex import PesanexConfig
from ..config.registry import register_architecture
from ..parts import LayerRun, ModelPlan, spec

NO_POSITION_LIMIT = 1 << 30


def _rope(rot, dim: int):
    if not rot or not rot.get("dims"):
        return None
    return spec("rope", theta=rot["base"], head_dim=dim, rotary_dim=rot["dims"], exact_table=True)


def _names(p: str, keys) -> dict:
    return {k + "_proj": p + k for k in keys}


def _retention(p: str, m: dict, eps: float):
    return spec("linear_attention", num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], eps=eps,
                k_scale=float(m["dim"]) ** -0.5, position=_rope(m.get("rot"), m["dim"]),
                decay={"kind": "per_head", "values": list(m["decay"])}, head_norm_weight=None, **_names(p, "qkvgo"))


def _gla(p: str, m: dict, eps: float):
    decay = {"kind": "low_rank", "down": p + "a1", "up": p + "a2", "bias": p + "a2.b", "tau": m["tau"]}
    if m.get("rank") is not None:
        decay["rank"] = m["rank"]
    return spec("linear_attention", num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], eps=eps,
                q_scale=float(m["dim"]) ** -0.5, position=None, decay=decay, head_norm_weight=p + "norm",
                **_names(p, "qkvgo"))


def _sink_attention(p: str, m: dict, eps: float):
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    return spec("attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                window=None, scale=m["scale"], sink=p + "sink", qk_unit_norm_eps=eps,
                position=spec("rope", theta=rot["base"], head_dim=m["dim"], rotary_dim=rot["dims"], exact_table=True),
                **_names(p, "qkvo"))


def _mixer(p: str, layer: dict, eps: float):
    kind, m = layer["type"], layer["mixer"]
    if kind == "retention":
        return _retention(p, m, eps)
    if kind == "gla":
        return _gla(p, m, eps)
    return spec("parallel_mean", left=_sink_attention(p + "left.", m["left"], eps), right=_gla(p + "right.", m["right"], eps),
                left_out=p + "left.out", right_out=p + "right.out", eps=eps)


@register_architecture("Pesanex", PesanexConfig)
def pesanex_plan(cfg: PesanexConfig) -> ModelPlan:
    def norm(name):
        return spec("layernorm", weight=name, eps=cfg.eps)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        options = dict(norm_in=norm(p + "norm1"), mixer=_mixer(p + "mix.", layer, cfg.eps), norm_mixer_out=norm(p + "norm1b"))
        if layer["mlp"] is not None:
            options.update(norm_post=norm(p + "norm2"), norm_ff_out=norm(p + "norm2b"),
                           feed_forward=spec("gated_dense", intermediate_size=layer["mlp"]["ff"], activation="relu",
                                             gate_proj=p + "mlp.gate", up_proj=p + "mlp.up", down_proj=p + "mlp.down"))
        blocks.append(spec("sandwich", **options))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=NO_POSITION_LIMIT,
        embedding=spec("scaled_embedding", weight="embed", vocab_size=cfg.vocab, scale=1.0),
        blocks=blocks, final_norm=norm("final.norm"),
        head=spec("logits_head", tied=False, weight="head", vocab_size=cfg.vocab),
        runs=[LayerRun(i) for i in cfg.order()],
    )
