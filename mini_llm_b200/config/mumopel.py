"""MumopelConfig: the keys of a Mumopel config.json, typed and checked.

A Mumopel model is a list of attention layers, each with its own sizes and constants and a feed-forward that is dense,
a mixture of experts, or absent.  A stretch of the layers may run several times in a row with the same tensors
(``loop``), and the residual may be several streams with learned mixing (``streams``).  Nothing is assumed equal between
layers: every size is read per entry.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig
from .finuvik import _int, _num

LAYER_TYPES = ("attention",)
FF_KINDS = ("dense", "moe")


@dataclass
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int                        # query / key entries per head
    vdim: int                       # value entries per head
    scale: float                    # factor on q.k, as given
    rot_dims: int = 0               # how many of the first entries of a head turn (0: no rotation)
    rot_base: float = 10000.0
    chunk: Optional[int] = None     # size of the blocks of the mask (None: plain causal)


@dataclass
class DenseSizes:
    ff: int


@dataclass
class MoESizes:
    experts: int
    top: int
    expert_ff: int
    expert_limit: float
    shared_ff: Optional[int] = None
    shared_limit: Optional[float] = None


@dataclass
class MumopelLayer:
    type: str
    mixer: AttentionSizes
    mlp: Any = None                 # DenseSizes | MoESizes | None


@dataclass
class Loop:
    start: int
    stop: int
    times: int


@dataclass
class MumopelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    layers: List[MumopelLayer] = field(default_factory=list)
    loop: Optional[Loop] = None
    streams: Optional[int] = None           # None: a single residual with the plain sum
    logit_softcap: Optional[float] = None
    eos_token_id: Optional[int] = None
    max_positions: Optional[int] = None
    raw: Dict[str, Any] = field(default_factory=dict, repr=False)

    @staticmethod
    def _attention(m: dict, where: str) -> AttentionSizes:
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: heads={heads} is not a multiple of kv_heads={kv}")
        dim = _int(m, "dim", where)
        rot = m.get("rot")
        dims, base = 0, 10000.0
        if rot is not None:
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims', or null")
            dims = _int(rot, "dims", where + ".rot", minimum=0)
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even and at most dim={dim}")
            base = _num(rot, "base", where + ".rot")
            if dims and base <= 1.0:
                raise ConfigError(f"config.json: {where}.rot.base must be greater than 1")
        mask = m.get("mask")
        chunk = None
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"config.json: {where}.mask must be an object with 'size', or null")
            chunk = _int(mask, "size", where + ".mask")
        return AttentionSizes(heads=heads, kv_heads=kv, dim=dim, vdim=_int(m, "vdim", where), scale=_num(m, "scale", where),
                              rot_dims=dims, rot_base=base, chunk=chunk)

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
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: top={top} of {experts} experts")
        limit = _num(ex, "limit", where + ".expert")
        if not limit > 0:
            raise ConfigError(f"config.json: {where}.expert.limit must be positive")
        shared = mlp.get("shared")
        sff = slim = None
        if shared is not None:
            if not isinstance(shared, dict):
                raise ConfigError(f"config.json: {where}.shared must be an object or null")
            sff, slim = _int(shared, "ff", where + ".shared"), _num(shared, "limit", where + ".shared")
            if not slim > 0:
                raise ConfigError(f"config.json: {where}.shared.limit must be positive")
        return MoESizes(experts=experts, top=top, expert_ff=_int(ex, "ff", where + ".expert"), expert_limit=limit,
                        shared_ff=sff, shared_limit=slim)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MumopelConfig":
        for key in ("vocab", "width", "norm", "layers"):
            if d.get(key) is None:
                raise ConfigError(f"config.json: missing required key {key!r}")
        if not isinstance(d["norm"], dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(d["norm"], "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[MumopelLayer] = []
        for i, e in enumerate(d["layers"]):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            if e.get("type") not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {LAYER_TYPES}, got {e.get('type')!r}")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            mlp = e.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}.mlp must be an object or null")
            layers.append(MumopelLayer(type=e["type"], mixer=cls._attention(m, where + ".mixer"),
                                       mlp=cls._mlp(mlp, where + ".mlp") if mlp is not None else None))
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times', or null")
            loop = Loop(start=_int(loop, "start", "loop", minimum=0), stop=_int(loop, "stop", "loop", minimum=0),
                        times=_int(loop, "times", "loop"))
            if not (loop.start < loop.stop <= len(layers)):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} is no stretch of the {len(layers)} layers")
        streams = d.get("streams")
        if streams is not None:
            streams = _int(d, "streams", "config")
        cap = d.get("logit_softcap")
        if cap is not None:
            cap = _num(d, "logit_softcap", "config")
            if not cap > 0:
                raise ConfigError(f"config.json: logit_softcap must be positive, got {cap!r}")
        vocab = _int(d, "vocab", "config")
        eos = d.get("eos_token_id")
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int) or not (0 <= eos < vocab)):
            raise ConfigError(f"config.json: eos_token_id {eos!r} is not a token of the vocabulary")
        mp = d.get("max_positions")
        if mp is not None:
            mp = _int(d, "max_positions", "config")
        cfg = cls(vocab=vocab, width=_int(d, "width", "config"), norm_eps=eps, layers=layers, loop=loop, streams=streams,
                  logit_softcap=cap, eos_token_id=eos, max_positions=mp, raw=copy.deepcopy(d))
        cfg.architecture = "Mumopel"
        return cfg

    def layer_order(self) -> List[int]:
        """The layers in the order they run: the looped stretch as a whole, ``times`` times in a row."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        lp = self.loop
        return list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))

    def to_dict(self) -> Dict[str, Any]:
        d = copy.deepcopy(self.raw)
        d["architecture"] = "Mumopel"
        return d
