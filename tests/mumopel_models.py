"""Small Mumopel configurations and weights for the tests: models that differ from each other in every size and
option, with weights that make faults show."""
from __future__ import annotations

import math

import torch


def attn(heads, kv_heads, dim, vdim, scale, rot=None, chunk=None):
    """rot: (dims, base) or None; chunk: block size of the mask or None."""
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if rot is not None:
        m["rot"] = dict(dims=rot[0], base=rot[1])
    if chunk is not None:
        m["mask"] = dict(size=chunk)
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit, shared=None):
    """shared: (ff, limit) or None."""
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit),
                shared=dict(ff=shared[0], limit=shared[1]) if shared else None)


def layer(mixer, mlp):
    return dict(type="attention", mixer=mixer, mlp=mlp)


def config(width, vocab, eps, layers, streams=None, loop=None, cap=None):
    c = dict(architecture="Mumopel", width=width, vocab=vocab, norm=dict(eps=eps), layers=layers)
    if streams is not None:
        c["streams"] = streams
    if loop is not None:
        c["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    if cap is not None:
        c["logit_softcap"] = cap
    return c


# R: two streams; layers 0 and 1 run twice in a row; capped logits.  Layer 0: six heads over two key/value heads, keys of
# 20 (rows padded to 24 in the pages) and values of 12, 8 of the 20 entries turn, blocks of 24 (one and a half pages), five
# experts of which two, a shared expert with another limit.  Layer 1: as many key/value heads as heads, all 16 entries turn,
# blocks of 37, a dense feed-forward.  Layer 2: one key/value head, no rotation, no mask, no feed-forward.
CFG_R = config(64, 97, 1e-5, [
    layer(attn(6, 2, 20, 12, 0.45, rot=(8, 100.0), chunk=24), moe(5, 2, 24, 0.7, shared=(40, 1.5))),
    layer(attn(2, 2, 16, 16, 0.6, rot=(16, 20.0), chunk=37), dense(72)),
    layer(attn(4, 1, 8, 24, 0.8), None),
], streams=2, loop=(0, 2, 2), cap=8.0)
# S: a single residual with the plain sum, no loop, no cap.  Layer 0: sizes the tensor-core attention takes (32 / 32), blocks
# of 64 (a key tile of that kernel), one expert per token and no shared expert.  Layer 1: eight heads over two, values
# three times as wide as keys, only 4 entries turn, blocks of 100.  Layer 2: one head of 64 that turns whole, blocks of 7,
# every expert for every token.
CFG_S = config(96, 211, 1e-6, [
    layer(attn(3, 3, 32, 32, 0.35, rot=(16, 30000.0), chunk=64), moe(4, 1, 16, 2.0)),
    layer(attn(8, 2, 16, 48, 0.5, rot=(4, 7.0), chunk=100), dense(40)),
    layer(attn(1, 1, 64, 16, 0.25, rot=(64, 1000.0), chunk=7), moe(3, 3, 8, 0.5, shared=(8, 0.5))),
])
CONFIGS = {"R": CFG_R, "S": CFG_S}
PAGE = {"R": 16, "S": 8}


def make_tensors(cfg, seed):
    """Norm weights of both signs on queries and keys and scales that give a peaked softmax (single keys carry weight),
    sinks from far below to above the usual scores, routers that decide clearly with biases that matter, expert limits
    that are reached often, stream weights away from 0 and 1 and a mixing matrix far from the identity."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    S = cfg.get("streams")

    def normal(*shape, std):
        return torch.empty(*shape).normal_(0.0, std, generator=g)

    def uniform(*shape, lo, hi):
        return torch.empty(*shape).uniform_(lo, hi, generator=g)

    def sign(*shape):
        return (torch.rand(*shape, generator=g) < 0.5).float() * 2.0 - 1.0

    t = {"embed": normal(cfg["vocab"], D, std=0.8), "final.norm": uniform(D, lo=0.5, hi=1.5), "final.norm.b": normal(D, std=0.2)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = uniform(D, lo=0.5, hi=1.5)
        t[p + "norm1.b"] = normal(D, std=0.2)
        t[p + "mix.q"] = normal(H * dk, D, std=1.0 / math.sqrt(D))
        t[p + "mix.k"] = normal(G * dk, D, std=1.0 / math.sqrt(D))
        t[p + "mix.v"] = normal(G * dv, D, std=1.5 / math.sqrt(D))
        t[p + "mix.q.norm"] = uniform(H * dk, lo=0.6, hi=1.8) * sign(H * dk)
        t[p + "mix.k.norm"] = uniform(G * dk, lo=0.6, hi=1.8) * sign(G * dk)
        t[p + "mix.sink"] = normal(H, std=2.0)
        t[p + "mix.o"] = normal(D, H * dv, std=1.0 / math.sqrt(H * dv))
        if S is not None:
            for q in ("hc1", "hc2") if lay.get("mlp") else ("hc1",):
                t[f"{p}{q}.in"] = uniform(S, lo=0.3, hi=0.9)
                t[f"{p}{q}.out"] = uniform(S, lo=0.4, hi=1.1) * sign(S)
                t[f"{p}{q}.mix"] = 0.7 * torch.eye(S) + uniform(S, S, lo=-0.25, hi=0.3)
        f = lay.get("mlp")
        if not f:
            continue
        t[p + "norm2"] = uniform(D, lo=0.5, hi=1.5)
        t[p + "norm2.b"] = normal(D, std=0.2)
        if f["kind"] == "dense":
            t[p + "mlp.gate"] = normal(f["ff"], D, std=1.2 / math.sqrt(D))
            t[p + "mlp.up"] = normal(f["ff"], D, std=1.2 / math.sqrt(D))
            t[p + "mlp.down"] = normal(D, f["ff"], std=1.0 / math.sqrt(f["ff"]))
            continue
        E = f["router"]["experts"]
        t[p + "mlp.router"] = normal(E, D, std=3.0 / math.sqrt(D))
        t[p + "mlp.router.b"] = normal(E, std=1.0)
        names = [f"e{e}" for e in range(E)]
        sizes = [f["expert"]["ff"]] * E
        if f.get("shared"):
            names.append("shared")
            sizes.append(f["shared"]["ff"])
        for n, F in zip(names, sizes):
            t[f"{p}mlp.{n}.gate"] = normal(F, D, std=1.2 / math.sqrt(D))
            t[f"{p}mlp.{n}.up"] = normal(F, D, std=1.2 / math.sqrt(D))
            t[f"{p}mlp.{n}.down"] = normal(D, F, std=1.0 / math.sqrt(F))
    return {k: v.to(torch.bfloat16).float() for k, v in t.items()}
