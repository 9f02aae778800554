"""Causal multi-head attention over the paged cache.

One fused projection gives Q | K | V (column thirds, head h = columns
h*dh..h*dh+dh-1 of its third: src/kernels/prefill/flashattention.cu:60-64,
100-111); keys and values of the step's tokens go to their page slots before
attention (src/kernels/prefill/append_kv.cu:28-46); every query at absolute
position p attends to cached positions <= p of its own request with
score = (q.k)*scale and a 32-bit softmax (src/kernels/prefill/flashattention.cu:
129-168, src/kernels/decode/paged_attention.cu:60-120, without the latter's
+1e-6 on the denominator); the output projection adds its bias and the
residual in its epilogue (src/model/gpt2_model.cu:326-334).

Unlike the reference's prefill kernel, which reads the step's own QKV buffer
and therefore needs the whole prompt at once (src/model/gpt2_model.cu:307-324),
every query here reads the cache, so a prompt can be cut anywhere.
"""
from __future__ import annotations

from typing import Optional

from ..cache.manager import PagedNeed
from .base import Mixer, ParamSpec, register_part
from .projected import ProjectedMixer


class Attention(Mixer):
    accepts_lazy_norm = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, scale: float,
                 num_kv_heads: Optional[int] = None, window: Optional[int] = None, bias: bool = True):
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads if num_kv_heads is not None else num_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.has_bias = bool(bias)
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_bias = None
        self.out_bias = None
        self.positions = None

    def param_specs(self):
        p = {"qkv_weight": ParamSpec((self.q_size + 2 * self.kv_size, self.hidden_size), "matrix"),
             "out_weight": ParamSpec((self.hidden_size, self.q_size), "matrix")}
        if self.has_bias:
            p["qkv_bias"] = ParamSpec((self.q_size + 2 * self.kv_size,), "vector")
            p["out_bias"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def kernel_limits(self, dtype: str):
        # every attention kernel of the library works on head sizes that are multiples of 16 from 16 to 256
        # (16-byte pieces of a key row per lane; mma tiles of 16): anything else has no kernel
        if self.head_dim % 16 != 0 or not (16 <= self.head_dim <= 256):
            return [f"attention: head size {self.head_dim} (hidden size {self.hidden_size} over {self.num_heads} heads) "
                    f"is not a multiple of 16 between 16 and 256, the sizes the attention kernels take"]
        return []

    def cache_need(self):
        return PagedNeed(kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window)

    def forward(self, h, ctx, cache, out_accum):
        ops = self.rt.ops
        T = h.shape[0]
        gv = ctx.groups[cache.group]
        rotates = self.positions is not None and getattr(self.positions, "acts_on_qk", False)
        if cache.write and not rotates:
            # keys and values go to their page slots from the projection itself
            q = ops.linear_qkv_cache(h, self.qkv_weight, self.qkv_bias,
                                     ctx.ws.buf("q", T, self.q_size, self.rt.act_dtype), cache.k_pages,
                                     cache.v_pages, gv.slot_mapping, ctx.ws)
        else:
            qkv = ctx.ws.buf("qkv", T, self.q_size + 2 * self.kv_size, self.rt.act_dtype)
            ops.linear(h, self.qkv_weight, self.qkv_bias, out=qkv)
            q = qkv[:, :self.q_size]
            k = qkv[:, self.q_size:self.q_size + self.kv_size]
            v = qkv[:, self.q_size + self.kv_size:]
            if rotates:
                self.positions.apply_qk(q, k, ctx)
            if cache.write:
                ops.kv_write(k, v, cache.k_pages, cache.v_pages, gv.slot_mapping)
        att = ctx.ws.buf("attn_out", T, self.q_size, self.rt.act_dtype)
        ops.paged_attention(q, cache.k_pages, cache.v_pages, gv.block_table, ctx, att,
                            num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                            head_dim=self.head_dim, scale=self.scale, window=self.window)
        ops.linear(att, self.out_weight, self.out_bias, out=out_accum, accumulate=True)


register_part("mixer", "attention", Attention)


class DistanceBiasAttention(ProjectedMixer):
    """Causal softmax attention with grouped key/value heads, key and value heads of different sizes, no
    rotation, and two ways in which positions enter the scores:

    * a query temperature: the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
      (``q_temp_coef`` = 0: none);
    * a distance penalty per head: r1_h * ln(1 + r2_h * (i - j)) is taken off the score of query i and key j,
      with r1, r2 learned per head (``log_distance_bias`` False: none).

    Both are functions of one integer, so they are tabulated once when the weights are bound (in float64, kept
    in float32): a factor per position and a bias per head and distance; the attention kernels look them up.
    """

    in_names = ("q_weight", "k_weight", "v_weight")
    out_name = "out_weight"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float,
                 max_positions: int, q_temp_coef: float = 0.0, q_temp_every: int = 1, log_distance_bias: bool = True,
                 window: Optional[int] = None):
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale = float(scale)
        self.max_positions = int(max_positions)
        self.q_temp_coef, self.q_temp_every = float(q_temp_coef), int(q_temp_every)
        self.log_distance_bias = bool(log_distance_bias)
        self.window = None if window is None else int(window)
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if self.q_temp_every < 1:
            raise ValueError("q_temp_every must be at least 1")
        self.q_size = self.num_heads * self.head_dim
        self.k_size = self.num_kv_heads * self.head_dim
        self.v_size = self.num_kv_heads * self.v_head_dim
        self.k_row = -(-self.head_dim // 8) * 8        # a key row in the pages: padded to 16-byte pieces, the padding zero
        self.dist_bias = None
        self.q_scale = None

    def param_specs(self):
        p = {"q_weight": ParamSpec((self.q_size, self.hidden_size), "matrix"),
             "k_weight": ParamSpec((self.k_size, self.hidden_size), "matrix"),
             "v_weight": ParamSpec((self.v_size, self.hidden_size), "matrix"),
             "out_weight": ParamSpec((self.hidden_size, self.num_heads * self.v_head_dim), "matrix")}
        if self.log_distance_bias:
            p["r1"] = ParamSpec((self.num_heads,), "vector")
            p["r2"] = ParamSpec((self.num_heads,), "vector")
        return p

    def kernel_limits(self, dtype: str):
        out = []
        if not (1 <= self.head_dim <= 256):
            out.append(f"distance-bias attention: key size {self.head_dim} is not between 1 and 256")
        if not (1 <= self.v_head_dim <= 256):
            out.append(f"distance-bias attention: value size {self.v_head_dim} is not between 1 and 256")
        return out

    def cache_need(self):
        return PagedNeed(kv_heads=self.num_kv_heads, head_dim=self.k_row, window=self.window,
                         v_head_dim=None if self.v_head_dim == self.k_row else self.v_head_dim)

    def bind(self, params, rt) -> None:
        import torch
        super().bind(params, rt)
        if not params:
            return
        n = self.max_positions
        if self.log_distance_bias:
            d = torch.arange(n, dtype=torch.float64)[None, :]
            r1 = self.r1.detach().double().cpu()[:, None]
            r2 = self.r2.detach().double().cpu()[:, None]
            self.dist_bias = (-r1 * torch.log1p(r2 * d)).float().contiguous().to(rt.device)
        if self.q_temp_coef != 0.0:
            steps = torch.div(torch.arange(n, dtype=torch.int64) + 1, self.q_temp_every, rounding_mode="floor").double()
            self.q_scale = (1.0 + self.q_temp_coef * torch.log(steps + 1.0)).float().contiguous().to(rt.device)

    def core(self, proj, ctx, cache, out, out_scale: float = 1.0) -> None:
        ops = self.rt.ops
        gv = ctx.groups[cache.group]
        q = proj[:, :self.q_size]
        if cache.write:
            ops.paged_write_kv(proj[:, self.q_size:self.q_size + self.k_size], proj[:, self.q_size + self.k_size:],
                               cache.k_pages, cache.v_pages, gv.slot_mapping)
        ops.biased_attention(q, cache.k_pages, cache.v_pages, gv.block_table, ctx, out, num_heads=self.num_heads,
                             num_kv_heads=self.num_kv_heads, scale=self.scale, dist_bias=self.dist_bias,
                             q_scale=self.q_scale, out_scale=out_scale, window=self.window)


register_part("mixer", "distance_bias_attention", DistanceBiasAttention)


class RotaryAttention(ProjectedMixer):
    """Causal softmax attention with grouped key/value heads and key and value heads of different sizes, in which
    queries and keys are normed and rotated before the scores are taken:

    * ``qk_norm``: an RMS norm over the WHOLE query projection of a token (all heads at once) and another over the whole
      key projection, each with a plain weight vector of that length and ``norm_eps`` inside the root;
    * a rotation of the first ``rot_dims`` entries of every query and key head by position * base^(-2i / rot_dims);
      ``rot_interleaved``: entry 2i pairs with 2i + 1, otherwise entry i with i + rot_dims / 2;
    * score = (q . k) * scale over the keys j <= i that the mask leaves: all of them, the last ``window``, or (``chunk``)
      those of the query's own block, block b being positions [b * chunk, (b + 1) * chunk) of the request;
    * ``sink``: a trained scalar s_h per head; exp(s_h) is one more term of the softmax's denominator and of nothing else,
      so part of a head's weight can go nowhere.

    Further options, all constructor constants.  ``head_norm`` (instead of ``qk_norm``): after the rotation every query
    head and every key head is divided by its own root mean square (no weights).  ``rot_scaling``: the frequencies'
    scaling (``parts.rotary``).  ``bias``: the three projections have biases.  ``softcap`` c: the scaled product s becomes
    c * tanh(s / c).  ``distance_slopes``: slope_h * (i - j) is taken off the score of query i and key j (after the cap),
    slope_h = 2^(-8 (h + 1) / H).  ``value_mix``: "first": the values of the step's tokens are also kept in a buffer of
    the step (``value_mix_key`` names it) for later layers; "mix": the values become (1 - lambda) v + lambda v_first
    before they are cached, v_first that buffer's rows of the same tokens and lambda a trained scalar (``v_mix``; a
    "first" layer has the tensor too and does not use it).

    The keys are cached normed and rotated (rows padded to 16-byte pieces), so a cached token is never touched again.
    With a chunk mask the pages of finished blocks go back to the pool as the request moves on.
    """

    in_names = ("q_weight", "k_weight", "v_weight")
    out_name = "out_weight"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float,
                 norm_eps: float = 1e-6, qk_norm: bool = True, rot_dims: int = 0, rot_base: float = 10000.0,
                 rot_interleaved: bool = True, window: Optional[int] = None, chunk: Optional[int] = None, sink: bool = False,
                 head_norm: bool = False, rot_scaling: Optional[dict] = None, bias: bool = False,
                 softcap: Optional[float] = None, distance_slopes: bool = False, value_mix: Optional[str] = None,
                 value_mix_key: str = "v_first"):
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.qk_norm = bool(qk_norm)
        self.head_norm = bool(head_norm)
        if self.qk_norm and self.head_norm:
            raise ValueError("rotary attention: a norm over the whole projection or one per head, not both")
        self.rot_scaling = None if rot_scaling is None else dict(rot_scaling)
        self.has_bias = bool(bias)
        self.softcap = None if softcap is None else float(softcap)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"rotary attention: the cap on the scores must be positive, got {softcap!r}")
        self.distance_slopes = bool(distance_slopes)
        if value_mix not in (None, "first", "mix"):
            raise ValueError(f"rotary attention: value_mix is None, 'first' or 'mix', got {value_mix!r}")
        self.value_mix, self.value_mix_key = value_mix, str(value_mix_key)
        self.rot_dims, self.rot_base, self.rot_interleaved = int(rot_dims), float(rot_base), bool(rot_interleaved)
        self.window = None if window is None else int(window)
        self.chunk = None if chunk is None else int(chunk)
        self.has_sink = bool(sink)
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.head_dim:
            raise ValueError(f"rot_dims={rot_dims} must be even and at most head_dim={head_dim}")
        if (self.window is not None and self.window < 1) or (self.chunk is not None and self.chunk < 1):
            raise ValueError("window and chunk must be positive")
        self.q_size = self.num_heads * self.head_dim
        self.k_size = self.num_kv_heads * self.head_dim
        self.v_size = self.num_kv_heads * self.v_head_dim
        self.k_row = -(-self.head_dim // 8) * 8        # a key row in the pages: padded to 16-byte pieces, the padding zero
        self.q_norm = self.k_norm = self.sink = self.freq = self.slopes = self.v_mix = None

    def param_specs(self):
        p = {"q_weight": ParamSpec((self.q_size, self.hidden_size), "matrix"),
             "k_weight": ParamSpec((self.k_size, self.hidden_size), "matrix"),
             "v_weight": ParamSpec((self.v_size, self.hidden_size), "matrix"),
             "out_weight": ParamSpec((self.hidden_size, self.num_heads * self.v_head_dim), "matrix")}
        if self.has_bias:
            p["q_bias"] = ParamSpec((self.q_size,), "vector")
            p["k_bias"] = ParamSpec((self.k_size,), "vector")
            p["v_bias"] = ParamSpec((self.v_size,), "vector")
        if self.value_mix is not None:
            p["v_mix"] = ParamSpec((), "vector")
        if self.qk_norm:
            p["q_norm"] = ParamSpec((self.q_size,), "vector")
            p["k_norm"] = ParamSpec((self.k_size,), "vector")
        if self.has_sink:
            p["sink"] = ParamSpec((self.num_heads,), "vector")
        return p

    def kernel_limits(self, dtype: str):
        out = []
        if not (1 <= self.head_dim <= 256):
            out.append(f"rotary attention: key size {self.head_dim} is not between 1 and 256")
        if not (1 <= self.v_head_dim <= 256):
            out.append(f"rotary attention: value size {self.v_head_dim} is not between 1 and 256")
        if (self.q_size + self.k_size) * 4 * (2 if self.head_norm else 1) > 200 * 1024:
            out.append(f"rotary attention: a token's {self.q_size} + {self.k_size} query and key entries do not fit the "
                       f"shared memory of the kernel that norms and rotates them")
        return out

    def cache_need(self):
        return PagedNeed(kv_heads=self.num_kv_heads, head_dim=self.k_row, window=self.window, chunk=self.chunk,
                         v_head_dim=None if self.v_head_dim == self.k_row else self.v_head_dim)

    def bind(self, params, rt) -> None:
        import torch
        from .rotary import rotary_table
        super().bind(params, rt)
        if not params:
            return
        if self.rot_dims:
            f, _ = rotary_table(self.rot_dims, self.rot_base, self.rot_scaling)   # float64 -> float32; the kernel takes position * f in 32-bit
            self.freq = torch.tensor(f, dtype=torch.float64).float().contiguous().to(rt.device)
        if self.has_bias:
            self.in_bias = torch.cat([self.q_bias, self.k_bias, self.v_bias]).contiguous()
        if self.distance_slopes:
            H = self.num_heads
            self.slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64).float().to(rt.device)
        if self.value_mix is not None:
            self.v_mix = self.v_mix.reshape(1).contiguous()

    def core(self, proj, ctx, cache, out, out_scale: float = 1.0) -> None:
        ops = self.rt.ops
        gv = ctx.groups[cache.group]
        T = proj.shape[0]
        q = ctx.ws.buf("attn_q", T, self.q_size, self.rt.act_dtype)
        mix = {}
        if self.value_mix is not None:
            # the first value-mixing layer's values of the step's tokens live in a buffer of the step under a name of
            # their own: nothing else writes it between that layer and the ones that mix them in
            kept = ctx.ws.buf("values_" + self.value_mix_key, T, self.v_size, self.rt.act_dtype)
            mix = dict(v_keep=kept) if self.value_mix == "first" else dict(v_first=kept, v_lambda=self.v_mix)
        ops.qk_norm_rope(proj, 0, self.q_size, self.q_size + self.k_size, ctx, q, cache.k_pages, cache.v_pages,
                         gv.slot_mapping if cache.write else None, heads=self.num_heads, kv_heads=self.num_kv_heads,
                         head_dim=self.head_dim, v_head_dim=self.v_head_dim, q_norm=self.q_norm, k_norm=self.k_norm,
                         eps=self.norm_eps, freq=self.freq, rot_dims=self.rot_dims, interleaved=self.rot_interleaved,
                         head_norm=self.head_norm, **mix)
        ops.biased_attention(q, cache.k_pages, cache.v_pages, gv.block_table, ctx, out, num_heads=self.num_heads,
                             num_kv_heads=self.num_kv_heads, scale=self.scale, out_scale=out_scale, window=self.window,
                             chunk=self.chunk, sink=self.sink, softcap=self.softcap or 0.0, slopes=self.slopes)


register_part("mixer", "rotary_attention", RotaryAttention)
