"""A plain, slow statement of the Mumopel design: whole sequences, no cache, float64.

One function per mechanism, written from the design's equations; it shares no code with
the package.  ``tensors`` maps checkpoint names to torch tensors, ``cfg`` is the parsed
config.json.  ``store`` rounds the values that the engine hands from kernel to kernel in
its activation dtype (identity for the 32-bit path).

Notation: D width, T tokens, p position (from 0), S residual streams.  Attention: H query
heads over G key/value heads, dk query/key size, dv value size, C the chunk of the mask.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F64 = torch.float64


def _keep(x):
    return x


def to_bf16(x):
    return x.to(torch.bfloat16).to(F64)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean of the squared deviations."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------------- rotation
def rotate_pairs(x, positions, dims: int, base: float):
    """x [..., T, d]: entries (2i, 2i + 1) of the first ``dims`` turn by p * base^(-2i/dims); the rest pass.
    The angle is taken in 32-bit: frequency and position as float32, their product rounded to float32."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    f = (float(base) ** (-2.0 * i / dims)).to(torch.float32)
    a = (positions.to(torch.float32)[:, None] * f[None, :]).to(F64)
    cos, sin = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------- attention
def visible(T: int, chunk: Optional[int]):
    """mask[i, j]: query i sees key j: j <= i, and both in the same block of ``chunk`` positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if chunk:
        m = m & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return m


def sink_softmax(s, mask, sink):
    """s [H, T, T] scores, sink [H]: p_ij = exp(s_ij) / (exp(sink_h) + sum over visible j' of exp(s_ij'))."""
    s = s.masked_fill(~mask[None], float("-inf"))
    if sink is None:
        return torch.softmax(s, -1)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, store: Callable = _keep):
    """h [T, D] -> [T, D]."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ w["q"].t())
    k = store(h @ w["k"].t())
    v = store(h @ w["v"].t())
    # one norm over the whole projection, before the heads are split
    q = rms_unit(q, eps) * w["q.norm"]
    k = rms_unit(k, eps) * w["k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    q = rotate_pairs(q.view(T, H, dk).transpose(0, 1), pos, rot["dims"], rot["base"])      # [H, T, dk]
    k = rotate_pairs(k.view(T, G, dk).transpose(0, 1), pos, rot["dims"], rot["base"])      # [G, T, dk]
    q, k = store(q), store(k)
    v = v.view(T, G, dv).transpose(0, 1)
    rep = H // G
    kh = k.repeat_interleave(rep, 0)
    vh = v.repeat_interleave(rep, 0)
    s = torch.einsum("hid,hjd->hij", q, kh) * m["scale"]
    mask = visible(T, (m.get("mask") or {}).get("size"))
    p = sink_softmax(s, mask, w.get("sink"))
    o = torch.einsum("hij,hjd->ihd", p, vh).reshape(T, H * dv)
    return store(o) @ w["o"].t()


# ------------------------------------------------------------------------------------------- feed-forward
def dense_ff(h, w: Dict[str, torch.Tensor], store: Callable = _keep):
    """W_down (silu(W_gate h) * (W_up h))."""
    g = store(h @ w["gate"].t())
    u = store(h @ w["up"].t())
    return store(g * torch.sigmoid(g) * u) @ w["down"].t()


def clamped_expert(h, w: Dict[str, torch.Tensor], limit: float, store: Callable = _keep, fused: bool = False):
    """W_down y with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g sigmoid(1.702 g) (u + 1).
    ``fused``: the engine applies the activation to the 32-bit sums of the first product (no rounding between)."""
    g = h @ w["gate"].t()
    u = h @ w["up"].t()
    if not fused:
        g, u = store(g), store(u)
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    return store(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].t()


def route(h, router, bias, top: int):
    """(indices [T, top], weights [T, top]): the ``top`` largest of W_router h + b (the lowest index among equals),
    weighted by the softmax over those ``top`` logits alone."""
    z = h @ router.t() + bias
    vals, idx = [], []
    zz = z.clone()
    for _ in range(top):
        mx = zz.max(-1, keepdim=True).values
        best = (zz == mx).to(torch.int64).argmax(-1)          # the first index that reaches the maximum
        idx.append(best)
        vals.append(zz.gather(-1, best[:, None])[:, 0])
        zz.scatter_(-1, best[:, None], float("-inf"))
    idx = torch.stack(idx, -1)
    vals = torch.stack(vals, -1)
    return idx, torch.softmax(vals, -1)


def moe_ff(h, w: Dict[str, torch.Tensor], f: dict, store: Callable = _keep):
    """h [T, D]; ``w`` holds "router", "router.b", "e<k>.gate|up|down" and, with a shared expert, "shared.*"."""
    T, D = h.shape
    r = f["router"]
    idx, wt = route(h, w["router"], w["router.b"], r["top"])
    out = torch.zeros(T, D, dtype=F64)
    for t in range(T):
        for k in range(r["top"]):
            e = int(idx[t, k])
            ew = {n: w[f"e{e}.{n}"] for n in ("gate", "up", "down")}
            out[t] += wt[t, k] * clamped_expert(h[t:t + 1], ew, f["expert"]["limit"], store, fused=True)[0]
    if f.get("shared"):
        sw = {n: w[f"shared.{n}"] for n in ("gate", "up", "down")}
        out = out + clamped_expert(h, sw, f["shared"]["limit"], store)
    return out


# ------------------------------------------------------------------------------------------- the model
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def layer_order(cfg: dict) -> List[int]:
    """The layers in the order they run: the looped stretch repeated as a whole."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer(streams, y_fn, hc: Optional[Dict[str, torch.Tensor]], norm_w, norm_b, eps, store):
    """One sublayer on the residual: plain (x += f(norm(x))) for a single stream without mixing tensors, else
    u = sum_s in_s x_s; y = f(norm(u)); x_t <- sum_s mix[s, t] x_s + out_t y for all t at once."""
    if hc is None:
        x = streams[0]
        return [x + y_fn(store(layer_norm(x, norm_w, norm_b, eps)))]
    S = len(streams)
    u = sum(hc["in"][s] * streams[s] for s in range(S))
    y = y_fn(store(layer_norm(u, norm_w, norm_b, eps)))
    return [sum(hc["mix"][s, t] * streams[s] for s in range(S)) + hc["out"][t] * y for t in range(S)]


def forward(tensors: Dict[str, torch.Tensor], cfg: dict, tokens, store: Callable = _keep, trace: Optional[list] = None):
    """Logits [T, vocab] of one sequence from position 0.  ``trace``: gets the residual (sum of the streams) after
    every run of a layer."""
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams")
    embed = tensors["embed"].to(F64)
    x0 = embed[torch.as_tensor(tokens, dtype=torch.long)]
    streams = [x0.clone() for _ in range(S or 1)]
    for li in layer_order(cfg):
        lay = cfg["layers"][li]
        w = sub(tensors, f"l{li}.")
        mw = sub(w, "mix.")
        hc1 = sub(w, "hc1.") if S else None
        streams = sublayer(streams, lambda h: attention(h, mw, lay["mixer"], eps, store), hc1, w["norm1"], w["norm1.b"],
                           eps, store)
        f = lay.get("mlp")
        if f:
            fw = sub(w, "mlp.")
            hc2 = sub(w, "hc2.") if S else None
            if f["kind"] == "dense":
                fn = lambda h: dense_ff(h, fw, store)
            else:
                fn = lambda h: moe_ff(h, fw, f, store)
            streams = sublayer(streams, fn, hc2, w["norm2"], w["norm2.b"], eps, store)
        if trace is not None:
            trace.append(sum(streams))
    x = sum(streams)
    y = store(layer_norm(x, tensors["final.norm"].to(F64), tensors["final.norm.b"].to(F64), eps))
    logits = y @ embed.t()
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def greedy(tensors, cfg, prompt, n_new: int, store: Callable = _keep):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(tensors, cfg, toks, store)[-1].argmax()))
    return toks[len(prompt):]
