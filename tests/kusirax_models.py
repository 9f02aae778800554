"""Small Kusirax configurations and weights for the tests: models that differ from each other in every size and
option, with weights that make faults show."""
from __future__ import annotations

import math

import torch


def wkv(heads, dim, rank):
    return dict(type="wkv", mixer=dict(heads=heads, dim=dim), rank=rank)


def attn(heads, kv_heads, dim, vdim, scale, rot, scaling=None, v_mix=False):
    """rot: (dims, base); scaling: (factor, low, high, original) or None."""
    r = dict(dims=rot[0], base=rot[1])
    if scaling is not None:
        r["scaling"] = dict(factor=scaling[0], low=scaling[1], high=scaling[2], original=scaling[3])
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=r, v_mix=v_mix))


def attn2(heads, kv_heads, dim, vdim, scale, chunk, cap, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if chunk is not None:
        m["mask"] = dict(size=chunk)
    if cap is not None:
        m["softcap"] = cap
    return dict(type="attention_2", mixer=m)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, scale, groups=None):
    """groups: (count, keep) or None."""
    r = dict(experts=experts, top=top, scale=scale)
    if groups is not None:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", router=r, expert=dict(ff=ff))


def layer(mix, mlp):
    """The ``rank`` of a wkv entry is not a key of config.json (the decay's matrices give it): it stays beside it."""
    out = dict(type=mix["type"], mixer=dict(mix["mixer"]), mlp=mlp)
    if "rank" in mix:
        out["_rank"] = mix["rank"]
    return out


def config(width, vocab, eps, alpha, layers):
    return dict(architecture="Kusirax", width=width, vocab=vocab, norm=dict(eps=eps), postln_alpha=alpha, layers=layers)


def ranks(cfg):
    return {i: l["_rank"] for i, l in enumerate(cfg["layers"]) if "_rank" in l}


def clean(cfg):
    """The configuration as config.json holds it."""
    c = dict(cfg)
    c["layers"] = [{k: v for k, v in l.items() if k != "_rank"} for l in cfg["layers"]]
    return c


# A: the first value-mixing layer is an attention_2: six heads over two key/value heads, keys of 20 (rows padded to 24 in
# the pages) and values of 12, blocks of 24 (one and a half pages), capped scores, six experts in three groups of which two
# are kept.  Then a recurrence of three heads of 16 with a decay of rank 5; a rotary attention that mixes its values (one
# key/value head of 24 values against the first layer's two of 12: the same 24 numbers per token), 8 of 16 entries turning
# with scaled frequencies, no feed-forward; a recurrence of one head of 40 (no multiple of 32) with rank 3 and one expert
# per token.
CFG_A = config(64, 97, 1e-5, 2.0, [
    layer(attn2(6, 2, 20, 12, 0.9, 24, 5.0, v_mix=True), moe(6, 3, 24, 1.7, groups=(3, 2))),
    layer(wkv(3, 16, 5), dense(72)),
    layer(attn(2, 1, 16, 24, 0.7, (8, 100.0), scaling=(4.0, 1.0, 4.0, 32), v_mix=True), None),
    layer(wkv(1, 40, 3), moe(4, 1, 16, 1.0)),
])
# B: starts with a recurrence of two heads of 64 (rank 16).  A rotary attention of sizes the tensor-core kernel takes (32 /
# 32) whose heads turn whole, without scaling and without value mixing, ten experts in two groups of which one is kept.
# An attention_2 of eight heads over two with values three times as wide as keys, blocks of 100, no cap, the only
# value-mixing layer.  An attention_2 of one head of 64, blocks of 7, a tight cap.  A recurrence of five heads of 8.
CFG_B = config(96, 211, 1e-6, 3.5, [
    layer(wkv(2, 64, 16), dense(40)),
    layer(attn(4, 4, 32, 32, 0.4, (32, 10000.0)), moe(10, 4, 16, 1.9, groups=(2, 1))),
    layer(attn2(8, 2, 16, 48, 0.8, 100, None, v_mix=True), dense(56)),
    layer(attn2(1, 1, 64, 16, 0.5, 7, 2.0), moe(3, 3, 8, 0.8)),
    layer(wkv(5, 8, 2), None),
])
CONFIGS = {"A": CFG_A, "B": CFG_B}
PAGE = {"A": 16, "B": 8}


def make_tensors(cfg, seed):
    """Scales that give a peaked softmax (single keys carry weight), decays from nearly none to nearly all within one
    head, bonuses of both signs, routers that decide clearly, mixing factors away from 0 and 1, norm weights away
    from 1."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def normal(*shape, std):
        return torch.empty(shape).normal_(0.0, std, generator=g)

    def uniform(*shape, lo, hi):
        return torch.empty(shape).uniform_(lo, hi, generator=g)

    t = {"embed": normal(cfg["vocab"], D, std=0.8), "embed.norm": uniform(D, lo=0.5, hi=1.5),
         "final.norm": uniform(D, lo=0.5, hi=1.5)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        t[p + "norm1"] = uniform(D, lo=0.5, hi=1.5)
        if lay["type"] == "wkv":
            N, R = m["heads"] * m["dim"], lay["_rank"]
            for c in "rkvgw":
                t[f"{p}mix.mu.{c}"] = uniform(D, lo=0.0, hi=1.0)
                if c != "w":
                    t[f"{p}mix.{c}"] = normal(N, D, std=1.0 / math.sqrt(D))
            t[p + "mix.w1"] = normal(R, D, std=1.5 / math.sqrt(D))
            t[p + "mix.w2"] = normal(N, R, std=0.8)
            t[p + "mix.w0"] = uniform(N, lo=-5.0, hi=0.8)
            t[p + "mix.u"] = normal(m["heads"], m["dim"], std=0.7)
            t[p + "mix.norm"] = uniform(N, lo=0.5, hi=1.5)
            t[p + "mix.o"] = normal(D, N, std=1.0 / math.sqrt(N))
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"] = normal(H * dk, D, std=1.0 / math.sqrt(D))
            t[p + "mix.k"] = normal(G * dk, D, std=1.0 / math.sqrt(D))
            t[p + "mix.v"] = normal(G * dv, D, std=1.5 / math.sqrt(D))
            t[p + "mix.o"] = normal(D, H * dv, std=1.0 / math.sqrt(H * dv))
            if lay["type"] == "attention_2":
                for c in "qkv":
                    t[f"{p}mix.{c}.b"] = normal(t[f"{p}mix.{c}"].shape[0], std=0.4)
            if m.get("v_mix"):
                t[p + "mix.vmix"] = uniform(lo=0.25, hi=0.75)
        f = lay.get("mlp")
        if not f:
            continue
        t[p + "norm2"] = uniform(D, lo=0.5, hi=1.5)
        if f["kind"] == "dense":
            t[p + "mlp.gate"] = normal(f["ff"], D, std=1.2 / math.sqrt(D))
            t[p + "mlp.up"] = normal(f["ff"], D, std=1.2 / math.sqrt(D))
            t[p + "mlp.down"] = normal(D, f["ff"], std=1.0 / math.sqrt(f["ff"]))
            continue
        E, F = f["router"]["experts"], f["expert"]["ff"]
        t[p + "mlp.router"] = normal(E, D, std=3.0 / math.sqrt(D))
        for e in range(E):
            t[f"{p}mlp.e{e}.up"] = normal(F, D, std=1.2 / math.sqrt(D))
            t[f"{p}mlp.e{e}.down"] = normal(D, F, std=1.0 / math.sqrt(F))
    return {k: v.to(torch.bfloat16).float() for k, v in t.items()}
