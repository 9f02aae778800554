"""A recurrent mixer with a decay that depends on the token (RWKV-style time mixing).

With h the mixer's input and h' the previous token's h (zeros before the first token of a sequence), each of the five
projections reads its own mix m_s = h + (h' - h) * mu_s, s in (r, k, v, g, w).  r, k, v = W_r m_r, W_k m_k, W_v m_v are
``num_heads`` heads of ``head_dim`` entries, the gate is silu(W_g m_g), and the decay per head and key channel is

    w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))                        W_w1 [rank, hidden], W_w2 [heads * dim, rank]

Per head, with a state S [dim, dim] that starts at zero:

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          S_t = diag(w_t) S_(t-1) + k_t v_t^T

(the bonus u counts for the current token only).  Each head's o_t is divided by its root mean square (eps inside the
root); the joined heads are multiplied by a weight per channel and by the gate, then W_o.  The request's state is S of
every head and the last row of h, both 32-bit, in one row of the cache manager's state arena; the decay (tanh and both
exponentials), the update, o, the norm and the gate are 32-bit whatever the engine's dtype.
"""
from __future__ import annotations

from ..cache.manager import StateNeed
from .base import Mixer, ParamSpec, register_part

MIXES = ("r", "k", "v", "g", "w")


class WKVMixer(Mixer):
    can_overwrite = True                # forward(..., accumulate=False) writes the result instead of adding it

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, norm_eps: float, decay_rank=None):
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        # None: the rank of the decay's two matrices is whatever the checkpoint stores
        self.decay_rank, self.norm_eps = (None if decay_rank is None else int(decay_rank)), float(norm_eps)
        self.inner = self.num_heads * self.head_dim
        self.s_floats = self.num_heads * self.head_dim * self.head_dim
        self.state_floats = self.s_floats + self.hidden_size

    def param_specs(self):
        D, N = self.hidden_size, self.inner
        p = {f"mu_{s}": ParamSpec((D,), "vector") for s in MIXES}
        p.update({"r_weight": ParamSpec((N, D), "matrix"), "k_weight": ParamSpec((N, D), "matrix"),
                  "v_weight": ParamSpec((N, D), "matrix"), "g_weight": ParamSpec((N, D), "matrix"),
                  "w1_weight": ParamSpec((self.decay_rank, D), "matrix"), "w2_weight": ParamSpec((N, self.decay_rank), "matrix"),
                  "w0": ParamSpec((N,), "vector"), "u": ParamSpec((self.num_heads, self.head_dim), "vector"),
                  "norm_weight": ParamSpec((N,), "vector"), "out_weight": ParamSpec((D, N), "matrix")})
        return p

    def kernel_limits(self, dtype: str):
        from .. import ops
        out = []
        if self.head_dim > ops.WKV_MAX_DIM:
            out.append(f"wkv: heads of {self.head_dim} entries; the kernel takes {ops.WKV_MAX_DIM}")
        if self.decay_rank is not None and self.decay_rank * 64 + 17 * 1024 > 96 * 1024:
            out.append(f"wkv: a decay of rank {self.decay_rank} does not fit the shared memory of the recurrence kernel")
        return out

    def cache_need(self):
        return StateNeed((self.state_floats,), "float32")

    def bind(self, params, rt) -> None:
        import torch
        super().bind(params, rt)
        if "mu_r" in params:
            self.mu = torch.stack([params[f"mu_{s}"] for s in MIXES]).contiguous()
            self.u_flat = self.u.reshape(-1).contiguous()
            self.rank = int(self.w1_weight.shape[0])
            if self.w2_weight.shape[1] != self.rank or self.rank * 64 + 17 * 1024 > 96 * 1024:
                raise ValueError(f"wkv: the decay's matrices have ranks {self.rank} and {self.w2_weight.shape[1]} "
                                 f"(equal, and at most {(96 - 17) * 1024 // 64})")

    def forward(self, h, ctx, cache, out_accum, accumulate: bool = True):
        import torch
        ops = self.rt.ops
        if isinstance(h, ops.NormedInput):
            h = h.materialize()
        T, D, N = h.shape[0], self.hidden_size, self.inner
        act = self.rt.act_dtype
        mixes = ctx.ws.buf("wkv_mixes", len(MIXES) * T, D, act).view(len(MIXES), T, D)
        ops.wkv_shift(h, self.mu, cache.state, self.s_floats, ctx, mixes)
        r = ctx.ws.buf("wkv_r", T, N, act)
        k = ctx.ws.buf("wkv_k", T, N, act)
        v = ctx.ws.buf("wkv_v", T, N, act)
        g = ctx.ws.buf("wkv_g", T, N, act)
        low = ctx.ws.buf("wkv_low", T, -(-self.rank // 8) * 8, act)[:, :self.rank]     # rows stay 16-byte aligned
        ops.linear(mixes[0], self.r_weight, None, out=r)
        ops.linear(mixes[1], self.k_weight, None, out=k)
        ops.linear(mixes[2], self.v_weight, None, out=v)
        ops.linear(mixes[3], self.g_weight, None, out=g)
        ops.linear(mixes[4], self.w1_weight, None, out=low)
        mid = ctx.ws.buf("mix_core", T, N, act)
        if getattr(ctx, "decode_only", False) and ops.wkv_step_ok(self.head_dim, self.rank):
            # single tokens: decay, update, output, norm and gate in one launch
            ops.wkv_step(r, k, v, low, self.w2_weight, self.w0, self.u_flat, g, self.norm_weight, h, cache.state, self.s_floats,
                         ctx, mid, heads=self.num_heads, eps=self.norm_eps, write_state=cache.write)
            ops.linear(mid, self.out_weight, None, out=out_accum, accumulate=accumulate)
            return
        dec = ctx.ws.buf("wkv_decay", T, N, torch.float32)
        ops.wkv_decay(low, self.w2_weight, self.w0, dec)
        raw = ctx.ws.buf("wkv_raw", T, N, torch.float32)
        ops.wkv_scan(r, k, v, dec, self.u_flat, h, cache.state, self.s_floats, ctx, raw, heads=self.num_heads,
                     write_state=cache.write)
        ops.wkv_finish(raw, g, self.norm_weight, mid, heads=self.num_heads, eps=self.norm_eps)
        ops.linear(mid, self.out_weight, None, out=out_accum, accumulate=accumulate)


register_part("mixer", "wkv", WKVMixer)
