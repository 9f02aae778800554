"""KusiraxConfig: the keys of a Kusirax config.json, typed and checked.

A Kusirax model is a list of layers, each with a mixer of one of three kinds ("wkv": a recurrence with a decay that
depends on the token; "attention": rotary softmax attention; "attention_2": softmax attention with biases, capped
scores, a linear distance penalty and a chunk mask) and a feed-forward that is dense, a mixture of experts, or absent.
Nothing is assumed equal between layers: every size and constant is read per entry.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig
from .finuvik import _int, _num

LAYER_TYPES = ("wkv", "attention", "attention_2")
FF_KINDS = ("dense", "moe")


@dataclass
class WKVSizes:
    heads: int
    dim: int                        # entries of r, k and v per head; the state of a head is dim x dim
    decay_rank: Optional[int] = None    # rank of the decay's two matrices; None: as the checkpoint stores them


@dataclass
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int                        # query / key entries per head
    vdim: int                       # value entries per head
    scale: float                    # factor on q.k, as given
    v_mix: bool = False             # the layer's values are mixed with the first such layer's
    rot_dims: int = 0               # how many of the first entries of a head turn (0: no rotation)
    rot_base: float = 10000.0
    rot_scaling: Optional[Dict[str, float]] = None      # factor, low, high, original
    softcap: Optional[float] = None
    chunk: Optional[int] = None     # size of the blocks of the mask (None: plain causal)


@dataclass
class DenseSizes:
    ff: int


@dataclass
class MoESizes:
    experts: int
    top: int
    expert_ff: int
    scale: float = 1.0
    groups: int = 1
    keep: int = 1


@dataclass
class KusiraxLayer:
    type: str
    mixer: Any                      # WKVSizes | AttentionSizes
    mlp: Any = None                 # DenseSizes | MoESizes | None


@dataclass
class KusiraxConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    postln_alpha: float = 1.0
    layers: List[KusiraxLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    max_positions: Optional[int] = None
    raw: Dict[str, Any] = field(default_factory=dict, repr=False)

    @staticmethod
    def _wkv(m: dict, where: str) -> WKVSizes:
        rank = m.get("decay_rank")
        return WKVSizes(heads=_int(m, "heads", where), dim=_int(m, "dim", where),
                        decay_rank=None if rank is None else _int(m, "decay_rank", where))

    @staticmethod
    def _attention(m: dict, where: str, kind: str) -> AttentionSizes:
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: heads={heads} is not a multiple of kv_heads={kv}")
        dim = _int(m, "dim", where)
        a = AttentionSizes(heads=heads, kv_heads=kv, dim=dim, vdim=_int(m, "vdim", where), scale=_num(m, "scale", where),
                           v_mix=bool(m.get("v_mix", False)))
        if kind == "attention":
            rot = m.get("rot")
            if rot is not None:
                if not isinstance(rot, dict):
                    raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims', or null")
                a.rot_dims = _int(rot, "dims", where + ".rot", minimum=0)
                if a.rot_dims % 2 or a.rot_dims > dim:
                    raise ConfigError(f"config.json: {where}.rot.dims={a.rot_dims} must be even and at most dim={dim}")
                a.rot_base = _num(rot, "base", where + ".rot")
                if a.rot_dims and a.rot_base <= 1.0:
                    raise ConfigError(f"config.json: {where}.rot.base must be greater than 1")
                sc = rot.get("scaling")
                if sc is not None:
                    if not isinstance(sc, dict):
                        raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
                    a.rot_scaling = {k: _num(sc, k, where + ".rot.scaling") for k in ("factor", "low", "high", "original")}
                    if not (a.rot_scaling["high"] > a.rot_scaling["low"] > 0 and a.rot_scaling["factor"] > 0
                            and a.rot_scaling["original"] > 0):
                        raise ConfigError(f"config.json: {where}.rot.scaling needs high > low > 0 and positive factor and original")
        else:
            cap = m.get("softcap")
            if cap is not None:
                a.softcap = _num(m, "softcap", where)
                if not a.softcap > 0:
                    raise ConfigError(f"config.json: {where}.softcap must be positive")
            mask = m.get("mask")
            if mask is not None:
                if not isinstance(mask, dict):
                    raise ConfigError(f"config.json: {where}.mask must be an object with 'size', or null")
                a.chunk = _int(mask, "size", where + ".mask")
        return a

    @staticmethod
    def _mlp(mlp: dict, where: str):
        kind = mlp.get("kind")
        if kind not in FF_KINDS:
            raise ConfigError(f"config.json: {where}.kind must be one of {FF_KINDS}, got {kind!r}")
        if kind == "dense":
            return DenseSizes(ff=_int(mlp, "ff", where))
        r, ex = mlp.get("router"), mlp.get("expert")
        if not isinstance(r, dict) or not isinstance(ex, dict):
            raise ConfigError(f"config.json: {where} must have 'router' and 'expert' objects")
        experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
        groups, keep = 1, 1
        g = r.get("groups")
        if g is not None:
            if not isinstance(g, dict):
                raise ConfigError(f"config.json: {where}.router.groups must be an object with 'count' and 'keep', or null")
            groups, keep = _int(g, "count", where + ".router.groups"), _int(g, "keep", where + ".router.groups")
        if experts % groups or keep > groups:
            raise ConfigError(f"config.json: {where}.router: {experts} experts in {groups} groups, {keep} kept")
        if top > keep * (experts // groups):
            raise ConfigError(f"config.json: {where}.router: top={top} of {keep} groups of {experts // groups} experts")
        scale = _num(r, "scale", where + ".router") if r.get("scale") is not None else 1.0
        return MoESizes(experts=experts, top=top, expert_ff=_int(ex, "ff", where + ".expert"), scale=scale, groups=groups,
                        keep=keep)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KusiraxConfig":
        for key in ("vocab", "width", "norm", "layers", "postln_alpha"):
            if d.get(key) is None:
                raise ConfigError(f"config.json: missing required key {key!r}")
        if not isinstance(d["norm"], dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(d["norm"], "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[KusiraxLayer] = []
        first_mix = None
        for i, e in enumerate(d["layers"]):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = e.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {LAYER_TYPES}, got {kind!r}")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            mixer = cls._wkv(m, where + ".mixer") if kind == "wkv" else cls._attention(m, where + ".mixer", kind)
            if kind != "wkv" and mixer.v_mix:
                if first_mix is None:
                    first_mix = (i, mixer.kv_heads * mixer.vdim)
                elif first_mix[1] != mixer.kv_heads * mixer.vdim:
                    raise ConfigError(f"config.json: {where}.mixer mixes its {mixer.kv_heads * mixer.vdim} values per token with "
                                      f"the {first_mix[1]} of layers[{first_mix[0]}]")
            mlp = e.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}.mlp must be an object or null")
            layers.append(KusiraxLayer(type=kind, mixer=mixer, mlp=cls._mlp(mlp, where + ".mlp") if mlp is not None else None))
        vocab = _int(d, "vocab", "config")
        eos = d.get("eos_token_id")
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int) or not (0 <= eos < vocab)):
            raise ConfigError(f"config.json: eos_token_id {eos!r} is not a token of the vocabulary")
        mp = d.get("max_positions")
        if mp is not None:
            mp = _int(d, "max_positions", "config")
        cfg = cls(vocab=vocab, width=_int(d, "width", "config"), norm_eps=eps, postln_alpha=_num(d, "postln_alpha", "config"),
                  layers=layers, eos_token_id=eos, max_positions=mp, raw=copy.deepcopy(d))
        cfg.architecture = "Kusirax"
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = copy.deepcopy(self.raw)
        d["architecture"] = "Kusirax"
        return d
