"""A routed feed-forward: a mixture of small gated experts, of which each token uses a few.

Router logits z = W_r h (32-bit), scores s = softmax(z) over all experts.  Experts form ``groups`` equal groups of
neighbours; a group's score is its largest score and only experts of the best ``keep`` groups can be chosen
(``groups`` = 1: no restriction).  The ``top`` experts with the largest scores are chosen, their weights are their
scores divided by their sum (+ 1e-20), and the output is the weighted sum of the chosen experts' outputs, each
W_down (act(W_gate h) * (W_up h)) without biases; a shared expert of the same form (``shared_size``, or None) runs
for every token and is added.

Variants, all constructor constants.  ``router_bias``: the logits get a trained offset per expert.
``selection`` "softmax_top": no softmax over all experts; the ``top`` largest logits are chosen and weighted by the
softmax over those alone (no groups).  ``activation`` "swiglu_clamp": an expert is W_down (g * sigmoid(alpha * g) *
(u + 1)) with g = min(W_gate h, limit) and u = clamp(W_up h, -limit, limit); the shared expert has a limit of its own
(``shared_limit``).  ``selection`` "sigmoid": the scores are sigmoid(z), expert by expert; ``group_sum`` 2: a group's
score is the sum of its two largest scores; ``weight_scale``: a factor on the weights.  ``activation`` "relu_sq": an
expert has no gate, W_down relu(W_up h)^2.

Nothing is read back by the host: a kernel routes and orders the (token, choice) pairs by expert, and the experts'
products run over that order with a grid that depends on the number of pairs only, so the step can be captured in a
CUDA graph.  The experts' matrices are stacked at bind: [E, 2F, D] (gate rows, then up rows) and [E, D, F].
"""
from __future__ import annotations

from typing import Optional

from .base import FeedForward, ParamSpec, register_part


class MoEFeedForward(FeedForward):
    can_overwrite = True

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, groups: int = 1, keep: int = 1,
                 shared_size: Optional[int] = None, activation: str = "silu", router_bias: bool = False,
                 selection: str = "softmax_all", limit: float = 0.0, alpha: float = 1.0,
                 shared_limit: Optional[float] = None, group_sum: int = 1, weight_scale: float = 1.0):
        self.hidden_size, self.num_experts, self.top = int(hidden_size), int(num_experts), int(top)
        self.expert_size, self.groups, self.keep = int(expert_size), int(groups), int(keep)
        self.shared_size = None if shared_size is None else int(shared_size)
        if activation not in ("silu", "swiglu_clamp", "relu_sq"):
            raise ValueError(f"MoEFeedForward: the experts' activation is silu, swiglu_clamp or relu_sq, got {activation!r}")
        self.activation = activation
        self.gated = activation != "relu_sq"
        if not self.gated and self.shared_size is not None:
            raise ValueError("MoEFeedForward: experts without a gate come without a shared expert")
        self.group_sum, self.weight_scale = int(group_sum), float(weight_scale)
        if self.group_sum not in (1, 2):
            raise ValueError(f"MoEFeedForward: a group's score is its largest score or the sum of its two largest, got {group_sum!r}")
        self.limit, self.alpha = float(limit), float(alpha)
        self.shared_limit = self.limit if shared_limit is None else float(shared_limit)
        if activation == "swiglu_clamp" and not (self.limit > 0 and self.shared_limit > 0):
            raise ValueError("MoEFeedForward: the clamped activation needs positive limits")
        self.has_router_bias = bool(router_bias)
        if selection not in ("softmax_all", "softmax_top", "sigmoid"):
            raise ValueError(f"MoEFeedForward: selection is softmax_all, softmax_top or sigmoid, got {selection!r}")
        if selection == "softmax_top" and self.groups != 1:
            raise ValueError("MoEFeedForward: the softmax over the chosen logits takes no groups")
        self.selection = selection
        self.router_bias = None
        if self.num_experts % self.groups or not (1 <= self.keep <= self.groups):
            raise ValueError(f"MoEFeedForward: {self.num_experts} experts in {self.groups} groups, {self.keep} kept")
        if not (1 <= self.top <= self.keep * (self.num_experts // self.groups)):
            raise ValueError(f"MoEFeedForward: top {self.top} of {self.keep} groups of {self.num_experts // self.groups}")

    def param_specs(self):
        D, F = self.hidden_size, self.expert_size
        p = {"router": ParamSpec((self.num_experts, D), "matrix")}
        if self.has_router_bias:
            p["router_bias"] = ParamSpec((self.num_experts,), "vector")
        for e in range(self.num_experts):
            if self.gated:
                p[f"expert{e}.gate"] = ParamSpec((F, D), "matrix")
            p[f"expert{e}.up"] = ParamSpec((F, D), "matrix")
            p[f"expert{e}.down"] = ParamSpec((D, F), "matrix")
        if self.shared_size is not None:
            p["shared.gate"] = ParamSpec((self.shared_size, D), "matrix")
            p["shared.up"] = ParamSpec((self.shared_size, D), "matrix")
            p["shared.down"] = ParamSpec((D, self.shared_size), "matrix")
        return p

    def kernel_limits(self, dtype: str):
        from .. import ops
        if self.num_experts > ops.MOE_MAX_EXPERTS or self.groups > 64:
            return [f"routed feed-forward: {self.num_experts} experts in {self.groups} groups; the router kernel takes "
                    f"{ops.MOE_MAX_EXPERTS} experts in up to 64 groups"]
        return []

    def bind(self, params, rt) -> None:
        import torch
        self.rt = rt
        if not params:
            return
        E = self.num_experts
        self.router = params["router"]
        self.router_bias = params.get("router_bias")
        if self.gated:
            self.w_first = torch.stack([torch.cat([params[f"expert{e}.gate"], params[f"expert{e}.up"]], 0) for e in range(E)]).contiguous()
        else:
            self.w_first = torch.stack([params[f"expert{e}.up"] for e in range(E)]).contiguous()
        self.w_second = torch.stack([params[f"expert{e}.down"] for e in range(E)]).contiguous()
        if self.shared_size is not None:
            self.shared_first = torch.cat([params["shared.gate"], params["shared.up"]], 0).contiguous()
            self.shared_down = params["shared.down"]

    def _experts(self, h, ctx):
        """Route, order, and run the chosen experts: (results per (token, choice) [T * top, D] 32-bit, weights [T, top])."""
        import torch
        ops = self.rt.ops
        T, top, E = h.shape[0], self.top, self.num_experts
        idx = ctx.ws.buf("moe_idx", T, top, torch.int32)
        wts = ctx.ws.buf("moe_weights", T, top, torch.float32)
        order = ctx.ws.buf("moe_order", T, top, torch.int32)
        offsets = ctx.ws.buf("moe_offsets", 1, E + 1, torch.int32)
        ops.moe_route(h, self.router, idx, wts, offsets, order, top=top, groups=self.groups, keep=self.keep,
                      bias=self.router_bias, mode=self.selection, group_sum=self.group_sum, weight_scale=self.weight_scale)
        mid = ctx.ws.buf("moe_mid", T * top, self.expert_size, self.rt.act_dtype)
        ops.moe_grouped(h, self.w_first, mid, offsets, order, top=top, first=True, act=self.activation, limit=self.limit,
                        alpha=self.alpha)
        pair_out = ctx.ws.buf("moe_pair_out", T * top, self.hidden_size, torch.float32)
        ops.moe_grouped(mid, self.w_second, pair_out, offsets, order, top=top, first=False)
        return pair_out, wts

    def _shared(self, h, ctx, out, accumulate):
        ops = self.rt.ops
        T = h.shape[0]
        gu = ctx.ws.buf("ff_gate_up", T, 2 * self.shared_size, self.rt.act_dtype)
        ops.linear(h, self.shared_first, None, out=gu)
        smid = ctx.ws.buf("ff_mid", T, self.shared_size, self.rt.act_dtype)
        ops.gated_act(gu, smid, self.activation, limit=self.shared_limit, alpha=self.alpha)
        ops.linear(smid, self.shared_down, None, out=out, accumulate=accumulate)

    def forward_pairs(self, h, ctx, y):
        """For a join that takes the weighted sum itself: the shared expert's result goes to y (if there is one), the
        chosen experts' results stay apart.  Returns (whether y was written, (results, weights, top))."""
        if isinstance(h, self.rt.ops.NormedInput):
            h = h.materialize()
        pair_out, wts = self._experts(h, ctx)
        if self.shared_size is not None:
            self._shared(h, ctx, y, False)
        return self.shared_size is not None, (pair_out, wts, self.top)

    def forward(self, h, ctx, out_accum, accumulate: bool = True):
        ops = self.rt.ops
        if isinstance(h, ops.NormedInput):
            h = h.materialize()
        pair_out, wts = self._experts(h, ctx)
        if self.shared_size is not None:
            self._shared(h, ctx, out_accum, accumulate)
            accumulate = True
        ops.moe_combine(pair_out, wts, out_accum, top=self.top, accumulate=accumulate)


register_part("feed_forward", "moe", MoEFeedForward)
