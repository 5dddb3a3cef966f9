"""A residual of several streams that sublayers read and write through learned weights (hyper-connections).

Instead of one residual x there are S streams x_1 .. x_S, all equal to the embedding's output at first.  A sublayer
with connection weights in [S], out [S] and mix [S, S] (indexed [from, to]) reads u = sum_s in[s] x_s through its
norm, and with its output y every stream becomes x_t <- sum_s mix[s, t] x_s + out[t] y, all from the old streams.
The model's last norm reads the plain sum of the streams.

'hyper_rmsnorm' (NORMS)   the norm in front of a sublayer together with that sublayer's connection weights.  It folds
                          the update that the sublayer before left pending into the streams, forms u and norms it, in
                          one kernel (csrc/hyper_connections.cu).  spec options: weight, eps, streams, connections
                          (prefix of the checkpoint names <prefix>in / out / mix; None: no weights, u is the plain sum:
                          the norm in front of the head).
'hyper_connected' (BLOCKS) pre-norm arrangement over such a residual.  spec options: norm_in, mixer, and norm_post,
                          feed_forward (both or neither).

The streams live in `residual.streams` [S, n, hidden] (32-bit); `residual.stream` stays the embedding's output.  A
pending update is a `StreamUpdate` on `residual.pending`; only norms of this kind can read it.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheRef, ParamSpec, Residual, branch_pair


class StreamUpdate:
    """A sublayer's output (a tensor, `Partials`, or something with `materialize`) and the connection it joins the
    streams through."""

    def __init__(self, branch, connection: "HyperRMSNorm"):
        self.branch, self.connection = branch, connection


@NORMS.register("hyper_rmsnorm")
class HyperRMSNorm:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.weight_name, self.eps, self.S = spec.weight, float(spec.eps), int(spec.streams)
        self.prefix = spec.options.get("connections")
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.weight = self.w_in = self.w_out = self.w_mix = None

    def param_specs(self):
        out = [ParamSpec(self.weight_name, (self.hidden_size,), "vector")]
        if self.prefix is not None:
            out += [ParamSpec(self.prefix + "in", (self.S,), "vector"), ParamSpec(self.prefix + "out", (self.S,), "vector"),
                    ParamSpec(self.prefix + "mix", (self.S, self.S), "vector")]
        return out

    def load(self, fetch):
        self.weight = fetch(self.weight_name).to(torch.float32).contiguous()
        if self.prefix is not None:
            self.w_in, self.w_out, self.w_mix = (fetch(self.prefix + k).to(torch.float32).contiguous() for k in ("in", "out", "mix"))

    def __call__(self, residual: Residual, ctx) -> torch.Tensor:
        out = ctx.buffer("normed", (residual.stream.shape[0], self.hidden_size), self.model_dtype)
        self._run(residual, ctx, out, None)
        residual.pending = None
        return out

    def rows(self, residual: Residual, rows: torch.Tensor, ctx) -> torch.Tensor:
        out = torch.empty((rows.shape[0], self.hidden_size), dtype=self.model_dtype, device=rows.device)
        self._run(residual, ctx, out, rows)
        return out

    def _run(self, residual: Residual, ctx, out, rows) -> None:
        n = residual.stream.shape[0]
        streams = getattr(residual, "streams", None)
        pending = residual.pending
        if pending is not None and not isinstance(pending, StreamUpdate):
            raise TypeError("a residual of several streams takes a sublayer's output through its connection (StreamUpdate)")
        if streams is None:
            # the model's first norm: every stream is the embedding's output, read from there and spread by the kernel
            src, dst = residual.stream, ctx.buffer("streams", (self.S, n, self.hidden_size), torch.float32)
            if rows is None:
                residual.streams = dst
        else:
            src = dst = streams
        branch, mix, w_out = None, None, None
        if pending is not None:
            branch = pending.branch.materialize(ctx) if hasattr(pending.branch, "materialize") else pending.branch
            branch, mix, w_out = branch_pair(branch), pending.connection.w_mix, pending.connection.w_out
        ops.hyper_norm(src, dst, self.S, branch, mix, w_out, self.w_in, self.weight, self.eps, out, rows)


@BLOCKS.register("hyper_connected")
class HyperConnectedBlock:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.norm_in = NORMS.build(spec.norm_in, **kw)
        self.mixer = MIXERS.build(spec.mixer, **kw)
        self.feed_forward = None
        if spec.options.get("feed_forward") is not None:
            self.norm_post = NORMS.build(spec.norm_post, **kw)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, **kw)
        for norm in [self.norm_in] + ([self.norm_post] if self.feed_forward is not None else []):
            if not isinstance(norm, HyperRMSNorm) or norm.prefix is None:
                raise TypeError("a hyper_connected block needs hyper_rmsnorm norms with connection weights")

    def parts(self):
        return [self.norm_in, self.mixer] + ([] if self.feed_forward is None else [self.norm_post, self.feed_forward])

    def cache_need(self):
        return self.mixer.cache_need()

    def __call__(self, residual: Residual, ctx, cache: CacheRef) -> None:
        residual.pending = StreamUpdate(self.mixer(self.norm_in(residual, ctx), ctx, cache), self.norm_in)
        if self.feed_forward is not None:
            residual.pending = StreamUpdate(self.feed_forward(self.norm_post(residual, ctx), ctx), self.norm_post)
