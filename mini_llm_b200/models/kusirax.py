"""Kusirax: configuration -> model description.

A decoder without a position table and with a 32-bit residual that is normed AFTER every sum: the embedded rows are
RMS-normed, then every layer is x <- norm1(alpha * x + mixer(x)), x <- norm2(alpha * x + ff(x)) (arrangement
"post_norm", joins ``parts.join.PostNormJoin``); the branches read x itself.  Three mixers, in any order:

* "wkv": ``parts.wkv.WKVMixer``, a recurrence with a matrix state per head, a decay per channel from a low-rank
  projection of the token, and token-shifted inputs;
* "attention": ``parts.attention.RotaryAttention`` with grouped heads, a rotation of the first entries of every head in
  half-split pairs (frequencies scaled by wavelength), then a unit RMS norm per head on queries and keys;
* "attention_2": the same part without rotation: biases on the three projections, a unit RMS norm per head, scores
  capped by c * tanh(. / c), a distance penalty slope_h * (i - j) and a chunk mask.

Attention layers whose configuration says ``v_mix`` mix their values with those of the first such layer,
(1 - lambda) v + lambda v_first, before they are cached.  The feed-forward is gated and dense (the tanh form of gelu),
a mixture of experts without gates (W_down relu(W_up h)^2) chosen by sigmoid scores inside the best groups (a group's
score: the sum of its two largest) with weights normed over the chosen and scaled, or absent.  The head is the embedding
table.

Tensor names: embed, embed.norm, final.norm; l<i>.norm1, l<i>.norm2; wkv: l<i>.mix.mu.{r,k,v,g,w}, l<i>.mix.{r,k,v,g,
w1,w2,w0,u,norm,o}; attention: l<i>.mix.{q,k,v,o,vmix} and, with biases, l<i>.mix.{q,k,v}.b; l<i>.mlp.{gate,up,down} or
l<i>.mlp.router, l<i>.mlp.e<k>.{up,down}; matrices are stored [out, in].
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.kusirax import DenseSizes, KusiraxConfig, WKVSizes
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, WeightRef

GROUP_SUM = 2           # the design scores a group of experts by the sum of this many of its largest scores


def build_kusirax_spec(cfg: KusiraxConfig) -> ModelSpec:
    D = cfg.width
    std = 1.0 / math.sqrt(D)

    def join(name):
        return PartSpec("post_norm", dict(hidden_size=D, eps=cfg.norm_eps, alpha=cfg.postln_alpha),
                        {"weight": WeightRef((name,), init=("uniform", 0.5, 1.5))})

    layers, ignored = [], []
    first_mix = None
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        s = lay.mixer
        if isinstance(s, WKVSizes):
            N = s.heads * s.dim
            w = {f"mu_{c}": WeightRef((f"{m}mu.{c}",), init=("uniform", 0.0, 1.0)) for c in "rkvgw"}
            w.update({"r_weight": WeightRef((m + "r",), init=("normal", std)),
                      "k_weight": WeightRef((m + "k",), init=("normal", std)),
                      "v_weight": WeightRef((m + "v",), init=("normal", std)),
                      "g_weight": WeightRef((m + "g",), init=("normal", std)),
                      "w1_weight": WeightRef((m + "w1",), init=("normal", std)),
                      "w2_weight": WeightRef((m + "w2",), init=("normal", 0.5)),
                      "w0": WeightRef((m + "w0",), init=("uniform", -4.0, 0.5)),
                      "u": WeightRef((m + "u",), init=("normal", 0.5)),
                      "norm_weight": WeightRef((m + "norm",), init=("uniform", 0.5, 1.5)),
                      "out_weight": WeightRef((m + "o",), init=("normal", 1.0 / math.sqrt(N)))})
            mixer = PartSpec("wkv", dict(hidden_size=D, num_heads=s.heads, head_dim=s.dim, norm_eps=cfg.norm_eps,
                                         decay_rank=s.decay_rank), w)
        else:
            biased = lay.type == "attention_2"
            value_mix = None
            if s.v_mix:
                value_mix = "first" if first_mix is None else "mix"
                first_mix = i if first_mix is None else first_mix
            w = {"q_weight": WeightRef((m + "q",), init=("normal", std)),
                 "k_weight": WeightRef((m + "k",), init=("normal", std)),
                 "v_weight": WeightRef((m + "v",), init=("normal", std)),
                 "out_weight": WeightRef((m + "o",), init=("normal", 1.0 / math.sqrt(s.heads * s.vdim)))}
            if biased:
                for c in "qkv":
                    w[c + "_bias"] = WeightRef((f"{m}{c}.b",), init=("normal", 0.3))
            if value_mix is not None:
                w["v_mix"] = WeightRef((m + "vmix",), init=("uniform", 0.2, 0.8))
            else:
                ignored.append(rf"^l{i}\.mix\.vmix$")
            mixer = PartSpec("rotary_attention",
                             dict(hidden_size=D, num_heads=s.heads, num_kv_heads=s.kv_heads, head_dim=s.dim, v_head_dim=s.vdim,
                                  scale=s.scale, norm_eps=cfg.norm_eps, qk_norm=False, head_norm=True, rot_dims=s.rot_dims,
                                  rot_base=s.rot_base, rot_interleaved=False, rot_scaling=s.rot_scaling, chunk=s.chunk,
                                  bias=biased, softcap=s.softcap, distance_slopes=biased, value_mix=value_mix), w)
        ff = None
        f = lay.mlp
        if isinstance(f, DenseSizes):
            ff = PartSpec("gated_mlp", dict(hidden_size=D, inner_size=f.ff, activation="gelu_tanh"),
                          {"gate_weight": WeightRef((p + "mlp.gate",), init=("normal", std)),
                           "up_weight": WeightRef((p + "mlp.up",), init=("normal", std)),
                           "down_weight": WeightRef((p + "mlp.down",), init=("normal", 1.0 / math.sqrt(f.ff)))})
        elif f is not None:
            w = {"router": WeightRef((p + "mlp.router",), init=("normal", 2.0 * std))}
            for e in range(f.experts):
                w[f"expert{e}.up"] = WeightRef((f"{p}mlp.e{e}.up",), init=("normal", std))
                w[f"expert{e}.down"] = WeightRef((f"{p}mlp.e{e}.down",), init=("normal", 1.0 / math.sqrt(f.expert_ff)))
            ff = PartSpec("moe", dict(hidden_size=D, num_experts=f.experts, top=f.top, expert_size=f.expert_ff, groups=f.groups,
                                      keep=f.keep, activation="relu_sq", selection="sigmoid", group_sum=GROUP_SUM,
                                      weight_scale=f.scale), w)
        else:
            ignored.append(rf"^l{i}\.norm2$")        # a layer without a feed-forward has no use for it
        layers.append(LayerSpec(mixer=mixer, ff=ff, mixer_norm=None, ff_norm=None, arrangement="post_norm",
                                mixer_join=join(p + "norm1"), ff_join=join(p + "norm2") if ff is not None else None))
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                     embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab, norm_eps=cfg.norm_eps),
                                        {"table": WeightRef(("embed",), init=("normal", 1.0)),
                                         "norm_weight": WeightRef(("embed.norm",), init=("uniform", 0.5, 1.5))}),
                     positions=PartSpec("none", {}, {}),
                     layers=layers,
                     final_norm=PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.norm_eps),
                                         {"weight": WeightRef(("final.norm",), init=("uniform", 0.5, 1.5))}),
                     head=PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab), {}),
                     max_positions=cfg.max_positions, eos_token_id=cfg.eos_token_id, ignored_tensors=ignored)


register_architecture("Kusirax", KusiraxConfig, build_kusirax_spec, replace=True)
