"""Joins: how a branch's result reaches the residual stream when that is more than a sum.

``NormScaleJoin``: x += rms_norm(y, w) * s, the branch's result normed once more (plain weights, eps inside the
root) and multiplied column by column by a learned scale before it is added; all 32-bit, one kernel.

``PostNormJoin``: x <- rms_norm(alpha * x + y, w), the block that norms after the sum; the new x also comes back in the
activation dtype for the branch that reads it next; all 32-bit, one kernel.
"""
from __future__ import annotations

from .base import Join, ParamSpec, register_part


class NormScaleJoin(Join):
    norms_next = True       # forward(..., then_norm=) also norms the new x for the next branch
    takes_pairs = True      # forward(..., pairs=) takes the weighted sum over a routed feed-forward's choices itself

    def __init__(self, hidden_size: int, eps: float, scaled: bool = True):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.scaled = bool(scaled)
        self.scale = None

    def param_specs(self):
        p = {"weight": ParamSpec((self.hidden_size,), "vector")}
        if self.scaled:
            p["scale"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def forward(self, y, x, ctx, pairs=None, then_norm=None):
        """x += n(y [+ the weighted pairs], w) * s.  ``pairs``: (results [T * top, D], weights [T, top], top) of a routed
        feed-forward whose weighted sum has not been taken yet (y may then be None).  ``then_norm``: an RMS norm that the
        next branch applies to the new x; its result comes back (one kernel does both), else None."""
        ops = self.rt.ops
        kw = {}
        if pairs is not None:
            kw.update(pairs=pairs[0], pair_weights=pairs[1], top=pairs[2])
        h = None
        if then_norm is not None:
            h = ctx.ws.buf("norm_out", x.shape[0], self.hidden_size, self.rt.act_dtype)
            kw.update(next_weight=then_norm.weight, next_eps=then_norm.eps, next_offset=1.0 if then_norm.unit_offset else 0.0,
                      next_out=h)
        ops.norm_scale_add(y, self.weight, self.scale, x, self.eps, **kw)
        return h


register_part("join", "norm_scale", NormScaleJoin)


class PostNormJoin(Join):
    takes_pairs = True      # forward(..., pairs=) takes the weighted sum over a routed feed-forward's choices itself

    def __init__(self, hidden_size: int, eps: float, alpha: float = 1.0):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.alpha = float(alpha)

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), "vector")}

    def forward(self, y, x, ctx, pairs=None):
        """x <- n(alpha * x + y [+ the weighted pairs], w) in place; returns the new x as the products read it: x itself
        on the 32-bit path, a copy in the activation dtype otherwise.  ``pairs``: (results [T * top, D], weights [T, top],
        top) of a routed feed-forward whose weighted sum has not been taken yet (y may then be None); y None and no pairs:
        the norm of alpha * x alone."""
        import torch
        kw = {}
        if pairs is not None:
            kw.update(pairs=pairs[0], pair_weights=pairs[1], top=pairs[2])
        h = None
        if self.rt.act_dtype != torch.float32:
            h = ctx.ws.buf("post_norm_out", x.shape[0], self.hidden_size, self.rt.act_dtype)
        self.rt.ops.post_norm(x, self.weight, self.eps, self.alpha, y=y, h=h, **kw)
        return x if h is None else h


register_part("join", "post_norm", PostNormJoin)
