"""Taritar as a plan of parts.

Every layer is a pre-norm block of root-mean-square norms around an attention mixer and a feed-forward, but the
residual is kept as several streams that each sublayer reads and writes through learned weights ('hyper_connected'
blocks with 'hyper_rmsnorm' norms; one plain stream when the configuration names no streams).  The attention has grouped
heads, a rotary turn of interleaved pairs over the first part of a head, a score scale of its own, a tanh cap on the
scores and a window that also keeps a sequence's first keys; a layer may read an earlier layer's keys and values instead
of projecting its own.  The feed-forward is a gated unit with clamped inputs, dense or as routed experts (softmax
scores, choice limited to the best groups of experts, a shared expert behind a sigmoid gate).  The embedding is scaled
and a learned position row is added; the head is untied and its logits pass a tanh cap.

Checkpoint names: embed, pos, head, final.norm; layer i: l<i>.norm1 / norm2, l<i>.hc1.* / hc2.* (in, out, mix),
l<i>.mix.q / k / v / o, l<i>.mlp.gate / up / down, or l<i>.mlp.router, l<i>.mlp.e<j>.gate / up / down and
l<i>.mlp.shared.gate / up / down / sg.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.taritar import TaritarConfig
from ..parts import LayerRun, ModelPlan, spec

GLU_SLOPE = 1.702        # y = g * sigmoid(GLU_SLOPE * g) * (u + 1) in every gated unit of the design


def _attention(p: str, m: dict):
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    mask = m.get("mask") or {}
    shared = m.get("kv_from") is not None
    names = {"q_proj": p + "q", "o_proj": p + "o"}
    if not shared:
        names.update(k_proj=p + "k", v_proj=p + "v")
    return spec("attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                window=mask.get("size"), keep_first=mask.get("keep_first", 0), scale=m["scale"], softcap=m.get("softcap"),
                reads_other_cache=shared,
                position=spec("rope", theta=rot["base"], head_dim=m["dim"], rotary_dim=rot["dims"], exact_table=True,
                              pairing="interleaved"), **names)


def _gated(p: str, sizes: dict):
    return dict(intermediate_size=sizes["ff"], activation="capped_swish", limit=sizes["limit"], slope=GLU_SLOPE,
                gate_proj=p + "gate", up_proj=p + "up", down_proj=p + "down")


def _feed_forward(p: str, mlp: dict):
    if mlp["kind"] == "dense":
        return spec("gated_dense", **_gated(p, mlp))
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    shared = None
    if mlp.get("shared") is not None:
        shared = dict(_gated(p + "shared.", mlp["shared"]), gate_weight=p + "shared.sg")
    return spec("routed_experts", num_experts=router["experts"], top=router["top"], groups=groups["count"],
                groups_kept=groups["keep"], router=p + "router", expert_prefix=p + "e", shared=shared,
                **{k: v for k, v in _gated(p, mlp["expert"]).items() if not k.endswith("_proj")})


@register_architecture("Taritar", TaritarConfig)
def taritar_plan(cfg: TaritarConfig) -> ModelPlan:
    S = cfg.streams

    def norm(name, connections=None):
        if S is None:
            return spec("rmsnorm", weight=name, eps=cfg.eps)
        return spec("hyper_rmsnorm", weight=name, eps=cfg.eps, streams=S, connections=connections)
    blocks, runs = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        options = dict(norm_in=norm(p + "norm1", p + "hc1."), mixer=_attention(p + "mix.", layer["mixer"]))
        if layer["mlp"] is not None:
            options.update(norm_post=norm(p + "norm2", p + "hc2."), feed_forward=_feed_forward(p + "mlp.", layer["mlp"]))
        blocks.append(spec("pre_norm" if S is None else "hyper_connected", **options))
        runs.append(LayerRun(i, cache_from=layer["mixer"].get("kv_from")))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=spec("scaled_embedding", weight="embed", vocab_size=cfg.vocab, scale=cfg.embedding_scale,
                       position_table="pos", max_positions=cfg.max_positions),
        blocks=blocks, final_norm=norm("final.norm"),
        head=spec("logits_head", tied=False, weight="head", vocab_size=cfg.vocab, softcap=cfg.logit_softcap),
        runs=runs,
    )
