"""Dense feed-forward: x += act(h @ W_fc^T + b_fc) @ W_proj^T + b_proj.

As in the reference the bias and the activation ride in the first product's
epilogue (src/kernels/linear.cu:48-66) and the bias and the residual sum in
the second's (src/kernels/linear.cu:28-46; src/model/gpt2_model.cu:345-363).
Activations: "gelu_tanh" (src/kernels/gemm.cu:17-20) and "gelu_erf".
"""
from __future__ import annotations

from .base import FeedForward, ParamSpec, register_part

ACTIVATIONS = ("gelu_tanh", "gelu_erf")


class MLP(FeedForward):
    accepts_lazy_norm = True

    def __init__(self, hidden_size: int, inner_size: int, activation: str, bias: bool = True):
        if activation not in ACTIVATIONS:
            raise ValueError(f"MLP activation must be one of {ACTIVATIONS}, got {activation!r}")
        self.hidden_size = int(hidden_size)
        self.inner_size = int(inner_size)
        self.activation = activation
        self.has_bias = bool(bias)
        self.fc_bias = None
        self.proj_bias = None

    def param_specs(self):
        p = {"fc_weight": ParamSpec((self.inner_size, self.hidden_size), "matrix"),
             "proj_weight": ParamSpec((self.hidden_size, self.inner_size), "matrix")}
        if self.has_bias:
            p["fc_bias"] = ParamSpec((self.inner_size,), "vector")
            p["proj_bias"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def forward(self, h, ctx, out_accum):
        ops = self.rt.ops
        mid = ctx.ws.buf("ff_mid", h.shape[0], self.inner_size, self.rt.act_dtype)
        ops.linear(h, self.fc_weight, self.fc_bias, out=mid, act=self.activation)
        ops.linear(mid, self.proj_weight, self.proj_bias, out=out_accum, accumulate=True)


register_part("feed_forward", "mlp", MLP)


GATE_ACTIVATIONS = ("relu", "silu", "gelu_tanh", "gelu_erf")


class GatedMLP(FeedForward):
    """x += W_down (act(W_gate h) * (W_up h)), no biases.  The gate and the up matrix are stacked into one
    [2F, D] matrix when the weights are bound, so both come from one product; a small kernel applies the
    activation and multiplies the halves; the down-projection adds into the residual in its epilogue."""

    def __init__(self, hidden_size: int, inner_size: int, activation: str = "silu"):
        if activation not in GATE_ACTIVATIONS:
            raise ValueError(f"GatedMLP activation must be one of {GATE_ACTIVATIONS}, got {activation!r}")
        self.hidden_size = int(hidden_size)
        self.inner_size = int(inner_size)
        self.activation = activation

    def param_specs(self):
        return {"gate_weight": ParamSpec((self.inner_size, self.hidden_size), "matrix"),
                "up_weight": ParamSpec((self.inner_size, self.hidden_size), "matrix"),
                "down_weight": ParamSpec((self.hidden_size, self.inner_size), "matrix")}

    def bind(self, params, rt) -> None:
        import torch
        super().bind(params, rt)
        if "gate_weight" in params:
            self.gate_up_weight = torch.cat([self.gate_weight, self.up_weight], 0).contiguous()
            self.gate_weight = self.gate_up_weight[:self.inner_size]
            self.up_weight = self.gate_up_weight[self.inner_size:]

    accepts_lazy_norm = True
    can_overwrite = True                # forward(..., accumulate=False) writes the result instead of adding it

    def project(self, h, ctx):
        """The first half: gate | up of h (a tensor or a norm not yet evaluated).  It only reads; an arrangement whose
        branches all read the same x calls it before any branch adds to x."""
        gu = ctx.ws.buf("ff_gate_up", h.shape[0], 2 * self.inner_size, self.rt.act_dtype)
        self.rt.ops.linear(h, self.gate_up_weight, None, out=gu)
        return gu

    def finish(self, gu, ctx, out_accum, accumulate: bool = True):
        ops = self.rt.ops
        mid = ctx.ws.buf("ff_mid", gu.shape[0], self.inner_size, self.rt.act_dtype)
        ops.gated_act(gu, mid, self.activation)
        ops.linear(mid, self.down_weight, None, out=out_accum, accumulate=accumulate)

    def forward(self, h, ctx, out_accum, accumulate: bool = True):
        self.finish(self.project(h, ctx), ctx, out_accum, accumulate)


register_part("feed_forward", "gated_mlp", GatedMLP)
