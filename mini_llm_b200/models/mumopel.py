"""Mumopel: configuration -> model description.

A decoder without a position table (positions enter through the rotation inside attention) and a 32-bit residual.
Every layer is pre-norm, x <- x + attention(norm1(x)), x <- x + ff(norm2(x)), with LayerNorms that have a weight and a
bias; with ``streams`` in the configuration the residual is that many streams and every sublayer reads and writes them
through a hyper-connection (``parts.hyper``; arrangement "hyper"), otherwise the plain sum (arrangement "pre_norm").
The mixer is ``parts.attention.RotaryAttention``: grouped heads, an RMS norm over the whole query and the whole key
projection, a rotation of the first entries of every head in interleaved pairs, a block mask (block b is the request's
positions [b * size, (b + 1) * size)) and a sink per head in the softmax.  The feed-forward is a gated dense one (silu), a mixture of clamped gated experts
chosen by the largest router logits (with a bias) and weighted by the softmax over the chosen logits, plus a shared
expert, or absent.  A stretch of the layers may run several times in a row with the same tensors, each pass with a cache
of its own.  The head is the embedding table; the logits may be capped by c * tanh(. / c).

Tensor names: embed, final.norm(.b); l<i>.norm1(.b), l<i>.norm2(.b); l<i>.mix.{q,k,v,o,q.norm,k.norm,sink};
l<i>.mlp.{gate,up,down} or l<i>.mlp.{router,router.b}, l<i>.mlp.e<k>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down};
l<i>.hc1.{in,out,mix}, l<i>.hc2.{in,out,mix}; matrices are stored [out, in], mix [from, to].
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.mumopel import DenseSizes, MumopelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, WeightRef

SIGMOID_SLOPE = 1.702       # the design's constant in an expert's gate, g * sigmoid(1.702 g)


def build_mumopel_spec(cfg: MumopelConfig) -> ModelSpec:
    D = cfg.width
    S = cfg.streams
    std = 1.0 / math.sqrt(D)

    def norm(name):
        return PartSpec("layernorm", dict(hidden_size=D, eps=cfg.norm_eps),
                        {"weight": WeightRef((name,), init=("uniform", 0.5, 1.5)),
                         "bias": WeightRef((name + ".b",), init=("normal", 0.1))})

    def connection(prefix):
        return PartSpec("hyper_connection", dict(hidden_size=D, streams=S),
                        {"read": WeightRef((prefix + ".in",), init=("uniform", 0.2, 0.8)),
                         "write": WeightRef((prefix + ".out",), init=("uniform", 0.3, 1.0)),
                         "mix": WeightRef((prefix + ".mix",), init=("uniform", 0.0, 0.6))})

    layers, ignored = [], []
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        s = lay.mixer
        mixer = PartSpec("rotary_attention",
                         dict(hidden_size=D, num_heads=s.heads, num_kv_heads=s.kv_heads, head_dim=s.dim, v_head_dim=s.vdim,
                              scale=s.scale, norm_eps=cfg.norm_eps, qk_norm=True, rot_dims=s.rot_dims, rot_base=s.rot_base,
                              rot_interleaved=True, chunk=s.chunk, sink=True),
                         {"q_weight": WeightRef((m + "q",), init=("normal", std)),
                          "k_weight": WeightRef((m + "k",), init=("normal", std)),
                          "v_weight": WeightRef((m + "v",), init=("normal", std)),
                          "out_weight": WeightRef((m + "o",), init=("normal", 1.0 / math.sqrt(s.heads * s.vdim))),
                          "q_norm": WeightRef((m + "q.norm",), init=("uniform", 0.5, 1.5)),
                          "k_norm": WeightRef((m + "k.norm",), init=("uniform", 0.5, 1.5)),
                          "sink": WeightRef((m + "sink",), init=("normal", 1.0))})
        ff = ff_norm = None
        f = lay.mlp
        if isinstance(f, DenseSizes):
            ff = PartSpec("gated_mlp", dict(hidden_size=D, inner_size=f.ff, activation="silu"),
                          {"gate_weight": WeightRef((p + "mlp.gate",), init=("normal", std)),
                           "up_weight": WeightRef((p + "mlp.up",), init=("normal", std)),
                           "down_weight": WeightRef((p + "mlp.down",), init=("normal", 1.0 / math.sqrt(f.ff)))})
        elif f is not None:
            w = {"router": WeightRef((p + "mlp.router",), init=("normal", 2.0 * std)),
                 "router_bias": WeightRef((p + "mlp.router.b",), init=("normal", 0.5))}
            for e in range(f.experts):
                w[f"expert{e}.gate"] = WeightRef((f"{p}mlp.e{e}.gate",), init=("normal", std))
                w[f"expert{e}.up"] = WeightRef((f"{p}mlp.e{e}.up",), init=("normal", std))
                w[f"expert{e}.down"] = WeightRef((f"{p}mlp.e{e}.down",), init=("normal", 1.0 / math.sqrt(f.expert_ff)))
            if f.shared_ff is not None:
                w["shared.gate"] = WeightRef((p + "mlp.shared.gate",), init=("normal", std))
                w["shared.up"] = WeightRef((p + "mlp.shared.up",), init=("normal", std))
                w["shared.down"] = WeightRef((p + "mlp.shared.down",), init=("normal", 1.0 / math.sqrt(f.shared_ff)))
            ff = PartSpec("moe", dict(hidden_size=D, num_experts=f.experts, top=f.top, expert_size=f.expert_ff,
                                      shared_size=f.shared_ff, activation="swiglu_clamp", router_bias=True,
                                      selection="softmax_top", limit=f.expert_limit, alpha=SIGMOID_SLOPE,
                                      shared_limit=f.shared_limit), w)
        if ff is not None:
            ff_norm = norm(p + "norm2")
        else:
            ignored.append(rf"^l{i}\.(norm2|norm2\.b|hc2\.(in|out|mix))$")     # a layer without a feed-forward has no use for them
        if S is None:
            layers.append(LayerSpec(mixer=mixer, ff=ff, mixer_norm=norm(p + "norm1"), ff_norm=ff_norm, arrangement="pre_norm"))
        else:
            layers.append(LayerSpec(mixer=mixer, ff=ff, mixer_norm=norm(p + "norm1"), ff_norm=ff_norm, arrangement="hyper",
                                    mixer_join=connection(p + "hc1"),
                                    ff_join=connection(p + "hc2") if ff is not None else None))
    # a layer's first run keeps the layer's own cache; every further run of a looped layer gets one of its own
    seen = set()
    schedule = []
    for li in cfg.layer_order():
        schedule.append(ScheduleEntry(li, private_cache=li in seen))
        seen.add(li)
    if S is None:
        final = norm("final.norm")
    else:
        final = PartSpec("stream_sum_layernorm", dict(hidden_size=D, eps=cfg.norm_eps, streams=S),
                         {"weight": WeightRef(("final.norm",), init=("uniform", 0.5, 1.5)),
                          "bias": WeightRef(("final.norm.b",), init=("normal", 0.1))})
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                     embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab, copies=S or 1),
                                        {"table": WeightRef(("embed",), init=("normal", 1.0))}),
                     positions=PartSpec("none", {}, {}),
                     layers=layers, final_norm=final,
                     head=PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab, softcap=cfg.logit_softcap), {}),
                     schedule=schedule, max_positions=cfg.max_positions, eos_token_id=cfg.eos_token_id,
                     ignored_tensors=ignored)


register_architecture("Mumopel", MumopelConfig, build_mumopel_spec, replace=True)
