"""Hyper-connections: a residual of several parallel streams in place of the single residual sum.

The residual of a token is ``streams`` vectors x_1 .. x_S side by side (a row of [S * D], 32-bit), all equal to the
embedding at the start (``TokenEmbedding(copies=S)``).  Every sublayer (a mixer or a feed-forward) has a
``HyperConnection`` with three learned tensors:

    read    u = sum_s in[s] x_s                          the sublayer runs on norm(u)
    write   x_t <- sum_s mix[s, t] x_s + out[t] * y      all streams at once from the old ones; y the sublayer's result

The arrangement "hyper" wires a layer this way.  One kernel pass over a token's row does the write of one sublayer and
the read and norm of the next, also across layers: a layer leaves its last write to the next layer's first read
(``ctx.carry``), so a layer is one pass per sublayer; the pass after a routed feed-forward also takes the weighted sum
over the token's experts.  The model's last norm sees the plain sum of the streams (``StreamSumNorm``); it takes the last
layer's write along for the tokens whose logits are wanted, and no others.
"""
from __future__ import annotations

import torch

from .base import Join, Norm, ParamSpec, register_part
from .block import _branch


def _norm_args(norm):
    """(gamma, beta or None, eps) of a LayerNorm or a plain-weight RMS norm part."""
    beta = getattr(norm, "bias", None)
    if beta is None and getattr(norm, "unit_offset", False):
        return norm.gamma, None, norm.eps
    return norm.weight, beta, norm.eps


class HyperConnection(Join):
    takes_pairs = True          # a routed feed-forward may leave the weighted sum over a token's experts to this pass

    def __init__(self, hidden_size: int, streams: int):
        self.hidden_size, self.streams = int(hidden_size), int(streams)
        if self.streams < 1:
            raise ValueError("HyperConnection: at least one stream")

    def param_specs(self):
        S = self.streams
        return {"read": ParamSpec((S,), "vector"), "write": ParamSpec((S,), "vector"), "mix": ParamSpec((S, S), "vector")}

    def kernel_limits(self, dtype: str):
        from .. import ops
        if self.streams > ops.HYPER_MAX_STREAMS:
            return [f"hyper-connections: {self.streams} streams; the kernel takes up to {ops.HYPER_MAX_STREAMS}"]
        return []

    def read_norm(self, x, norm, ctx):
        """h = norm(sum_s read[s] x_s) in the activation dtype."""
        gamma, beta, eps = _norm_args(norm)
        h = ctx.ws.buf("norm_out", x.shape[0], self.hidden_size, self.rt.act_dtype)
        self.rt.ops.hyper_step(x, self.streams, in_weights=self.read, gamma=gamma, beta=beta, eps=eps, h=h)
        return h

    def forward(self, y, x, ctx, then=None, pairs=None):
        """The write of this sublayer's result y into the streams x; with ``then`` = (the next sublayer's
        HyperConnection, its norm) also that sublayer's read and norm of the new streams, which comes back.
        ``pairs`` = (results per (token, choice), weights, top) of a routed feed-forward: their weighted sum is part of
        the result (y may then be None)."""
        if then is None:
            self.rt.ops.hyper_step(x, self.streams, y=y, mix=self.mix, out_weights=self.write, pairs=pairs)
            return None
        nxt, norm = then
        gamma, beta, eps = _norm_args(norm)
        h = ctx.ws.buf("norm_out", x.shape[0], self.hidden_size, self.rt.act_dtype)
        self.rt.ops.hyper_step(x, self.streams, y=y, mix=self.mix, out_weights=self.write, in_weights=nxt.read, gamma=gamma,
                               beta=beta, eps=eps, h=h, pairs=pairs)
        return h


register_part("join", "hyper_connection", HyperConnection)


class StreamSumNorm(Norm):
    """LayerNorm (weight and bias) of the sum of a residual's streams: what the head reads."""

    def __init__(self, hidden_size: int, eps: float, streams: int):
        self.hidden_size, self.eps, self.streams = int(hidden_size), float(eps), int(streams)

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), "vector"), "bias": ParamSpec((self.hidden_size,), "vector")}

    def forward(self, x, ctx, rows=None, lazy=False):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buf("norm_out", n, self.hidden_size, self.rt.act_dtype)
        left = _take_carry(ctx, x)
        if left is None:
            self.rt.ops.hyper_step(x, self.streams, gamma=self.weight, beta=self.bias, eps=self.eps, rows=rows, h=out)
        else:       # the last layer's write on the way, for the rows that are read (all of them when rows is None)
            join, y, pairs = left
            self.rt.ops.hyper_step(x, self.streams, y=y, mix=join.mix, out_weights=join.write, pairs=pairs, gamma=self.weight,
                                   beta=self.bias, eps=self.eps, rows=rows, h=out)
        return out

    def stream_sum(self, x, ctx):
        """The plain sum of the streams, [T, D] 32-bit (what a single-stream model calls its residual).  A write that
        the last layer left open is made first, for all tokens."""
        out = ctx.ws.buf("stream_sum", x.shape[0], self.hidden_size, torch.float32)
        left = _take_carry(ctx, x)
        if left is None:
            self.rt.ops.hyper_step(x, self.streams, sum_out=out)
        else:
            join, y, pairs = left
            self.rt.ops.hyper_step(x, self.streams, y=y, mix=join.mix, out_weights=join.write, pairs=pairs, sum_out=out)
        return out


register_part("norm", "stream_sum_layernorm", StreamSumNorm)


def _leave(ctx, x, join, y, pairs) -> None:
    """A layer's last write stays open: whoever reads the streams next (the next layer, the model's last norm, or
    ``StreamSumNorm.stream_sum``) makes it in the same pass.  y and the experts' results live in workspace buffers that
    nothing touches before that read.  A context without a ``carry`` slot gets the write at once."""
    if not hasattr(ctx, "carry"):
        join.forward(y, x, ctx, pairs=pairs)
        return
    if ctx.carry is not None:
        raise RuntimeError("hyper arrangement: a write is still open")
    ctx.carry = (x, join, y, pairs)


def _take_carry(ctx, x):
    """(join, y, pairs) of the write that was left open on these streams, or None."""
    left = getattr(ctx, "carry", None)
    if left is None:
        return None
    if left[0] is not x and left[0].data_ptr() != x.data_ptr():
        raise RuntimeError("hyper arrangement: the open write belongs to other streams")
    ctx.carry = None
    return left[1:]


def hyper(layer, x, ctx, cache):
    """x: the streams [T, S * D].  Mixer, then feed-forward (if the layer has one), each read from and written to all
    streams through its HyperConnection (``LayerSpec.mixer_join`` / ``ff_join``)."""
    if layer.mixer_join is None or (layer.ff is not None and layer.ff_join is None):
        raise RuntimeError("hyper arrangement: a sublayer has no HyperConnection")
    D = layer.mixer_join.hidden_size
    y = ctx.ws.buf("branch_out", x.shape[0], D, torch.float32)
    left = _take_carry(ctx, x)
    if left is None:
        h = layer.mixer_join.read_norm(x, layer.mixer_norm, ctx)
    else:           # the layer before left its last write open: one pass makes it and this layer's first read
        join, y_left, pairs = left
        h = join.forward(y_left, x, ctx, then=(layer.mixer_join, layer.mixer_norm), pairs=pairs)
    _branch(layer.mixer, y, h, ctx, cache)
    if layer.ff is None:
        _leave(ctx, x, layer.mixer_join, y, None)
        return x
    h = layer.mixer_join.forward(y, x, ctx, then=(layer.ff_join, layer.ff_norm))
    if hasattr(layer.ff, "forward_pairs"):
        shared, pairs = layer.ff.forward_pairs(h, ctx, y)
        _leave(ctx, x, layer.ff_join, y if shared else None, pairs)
    else:
        _branch(layer.ff, y, h, ctx)
        _leave(ctx, x, layer.ff_join, y, None)
    return x


register_part("arrangement", "hyper", lambda: hyper)
