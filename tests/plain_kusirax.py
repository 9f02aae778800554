"""A plain, slow statement of the Kusirax design: whole sequences, no cache, float64.

One function per mechanism, written from the design's equations; it shares no code with
the package.  ``tensors`` maps checkpoint names to torch tensors, ``cfg`` is the parsed
config.json.  ``store`` rounds the values that the engine hands from kernel to kernel in
its activation dtype (identity for the 32-bit path).

Notation: D width, T tokens, p position (from 0).  Attention: H query heads over G key/value
heads, dk query/key size, dv value size, C the chunk of the mask.  Recurrence: Hr heads of n
channels, a state S [n, n] per head.
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


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------------------- rotation
def frequencies(dims: int, base: float, scaling: Optional[dict]):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` (factor, low, high, original) the slow ones are divided by
    factor: a wavelength l = 2 pi / f below original/high keeps f, above original/low gets f / factor, and between the
    two the mix (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling is None:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for n in range(f.numel()):
        l = 2.0 * math.pi / float(f[n])
        if l < orig / high:
            continue
        if l > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / l - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate_half(x, positions, dims: int, freq):
    """x [..., T, d]: entry i of the first ``dims`` pairs with entry i + dims/2; the pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p * f_i.  The angle is taken in 32-bit: frequency and position as
    float32, their product rounded to float32."""
    if dims == 0:
        return x
    half = dims // 2
    a = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(F64)
    cos, sin = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------- attention
def visible(T: int, chunk: Optional[int]):
    """mask[i, j]: query i sees key j: j <= i, and (with a chunk) both in the same block of ``chunk`` positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if chunk:
        m = m & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return m


def slopes(H: int):
    """slope_h = 2^(-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F64)


def mix_values(v, v_first, lam):
    """(1 - lambda) v + lambda v_first."""
    return (1.0 - lam) * v + lam * v_first


def attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, kind: str, v_first=None, store: Callable = _keep):
    """h [T, D] -> ([T, D], the values as they are cached [T, G * dv]).  ``kind`` "attention": rotation, no biases;
    "attention_2": biases, capped scores, a distance penalty and a chunk mask.  ``v_first``: the values of the first
    value-mixing layer (None: this layer is the first, or does not mix)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if kind == "attention_2":
        q, k, v = q + w["q.b"], k + w["k.b"], v + w["v.b"]
    q, k, v = store(q), store(k), store(v)
    if m.get("v_mix") and v_first is not None:
        v = store(mix_values(v, v_first, w["vmix"]))
    q = q.view(T, H, dk).transpose(0, 1)
    k = k.view(T, G, dk).transpose(0, 1)
    if kind == "attention":
        rot = m["rot"]
        f = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_half(q, pos, rot["dims"], f), rotate_half(k, pos, rot["dims"], f)
    q, k = store(rms_unit(q, eps)), store(rms_unit(k, eps))
    vh = v.view(T, G, dv).transpose(0, 1)
    k = k.repeat_interleave(H // G, 0)
    vh = vh.repeat_interleave(H // G, 0)
    s = (q @ k.transpose(1, 2)) * m["scale"]
    chunk = None
    if kind == "attention_2":
        cap = m.get("softcap")
        if cap:
            s = cap * torch.tanh(s / cap)
        dist = (pos[:, None] - pos[None, :]).to(F64)
        s = s - slopes(H)[:, None, None] * dist[None]
        chunk = (m.get("mask") or {}).get("size")
    s = s.masked_fill(~visible(T, chunk)[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = store((p @ vh).transpose(0, 1).reshape(T, H * dv))
    return o @ w["o"].T, v


# ------------------------------------------------------------------------------------------- recurrence
def token_shift(h, mu, h_before=None):
    """h + (h' - h) * mu with h' the row before (``h_before``, or zeros, before the first)."""
    first = torch.zeros_like(h[:1]) if h_before is None else h_before[None]
    prev = torch.cat([first, h[:-1]], 0)
    return h + (prev - h) * mu


def decay(xw, w1, w2, w0, store: Callable = _keep):
    """exp(-exp(W2 tanh(W1 xw) + w0)) per channel.  Only the first product's result is handed on in the activation
    dtype; from the tanh on everything belongs to the recurrence and stays exact."""
    low = torch.tanh(store(xw @ w1.T))
    return torch.exp(-torch.exp(low @ w2.T + w0))


def wkv_scan(r, k, v, w, u, S0=None):
    """Per head: o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T.  r, k, v, w [T, Hr, n], u
    [Hr, n]; returns (o [T, Hr, n], S [Hr, n, n])."""
    T, Hr, n = r.shape
    S = torch.zeros(Hr, n, n, dtype=F64) if S0 is None else S0.clone()
    out = torch.zeros(T, Hr, n, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t][:, :, None] * S + kv
    return out, S


def wkv(h, w: Dict[str, torch.Tensor], m: dict, eps: float, store: Callable = _keep):
    """h [T, D] -> [T, D]."""
    T = h.shape[0]
    Hr, n = m["heads"], m["dim"]
    mixes = {s: store(token_shift(h, w["mu." + s])) for s in "rkvgw"}
    r = store(mixes["r"] @ w["r"].T).view(T, Hr, n)
    k = store(mixes["k"] @ w["k"].T).view(T, Hr, n)
    v = store(mixes["v"] @ w["v"].T).view(T, Hr, n)
    g = store(mixes["g"] @ w["g"].T)
    gate = g * torch.sigmoid(g)
    dec = decay(mixes["w"], w["w1"], w["w2"], w["w0"], store).view(T, Hr, n)
    o, _ = wkv_scan(r, k, v, dec, w["u"])
    y = store(rms_unit(o, eps).reshape(T, Hr * n) * w["norm"] * gate)
    return y @ w["o"].T


# ------------------------------------------------------------------------------------------- feed-forward
def dense_ff(h, w: Dict[str, torch.Tensor], store: Callable = _keep):
    """W_down (gelu_tanh(W_gate h) * (W_up h))."""
    g, u = store(h @ w["gate"].T), store(h @ w["up"].T)
    return store(gelu_tanh(g) * u) @ w["down"].T


def expert(h, w: Dict[str, torch.Tensor], store: Callable = _keep):
    """W_down relu(W_up h)^2."""
    return store(torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


def route(h, router, r: dict):
    """Scores sigmoid(W_r h); groups of neighbours scored by the sum of their two largest; the ``top`` largest scores
    inside the best ``keep`` groups; weights = chosen scores / (their sum + 1e-20) * scale.  Returns (idx [T, top],
    weights [T, top])."""
    s = torch.sigmoid(h @ router.T)
    T, E = s.shape
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n_g, keep = groups["count"], groups["keep"]
    per = E // n_g
    allowed = torch.ones(T, E, dtype=torch.bool)
    if keep < n_g:
        gs = s.view(T, n_g, per).topk(min(2, per), -1).values.sum(-1)
        best = gs.topk(keep, -1).indices
        gm = torch.zeros(T, n_g, dtype=torch.bool)
        gm.scatter_(1, best, True)
        allowed = gm[:, :, None].expand(T, n_g, per).reshape(T, E)
    masked = s.masked_fill(~allowed, -1.0)
    idx = masked.topk(r["top"], -1).indices
    chosen = s.gather(1, idx)
    wts = chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return idx, wts


def moe_ff(h, w: Dict[str, torch.Tensor], f: dict, store: Callable = _keep):
    idx, wts = route(h, w["router"], f["router"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            e = int(idx[t, c])
            out[t] += wts[t, c] * expert(h[t:t + 1], {"up": w[f"e{e}.up"], "down": w[f"e{e}.down"]}, store)[0]
    return out


# ------------------------------------------------------------------------------------------- the model
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(tensors: Dict[str, torch.Tensor], cfg: dict, tokens, store: Callable = _keep, trace: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence.  ``trace``: gets the residual after every layer."""
    eps = cfg["norm"]["eps"]
    alpha = float(cfg["postln_alpha"])
    E = tensors["embed"].to(F64)
    x = rms_norm(E[torch.as_tensor(tokens, dtype=torch.long)], tensors["embed.norm"].to(F64), eps)
    v_first = None
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        mw = sub(tensors, p + "mix.")
        h = store(x)
        if lay["type"] == "wkv":
            y = wkv(h, mw, lay["mixer"], eps, store)
        else:
            y, v = attention(h, mw, lay["mixer"], eps, lay["type"], v_first, store)
            if lay["mixer"].get("v_mix") and v_first is None:
                v_first = v
        x = rms_norm(alpha * x + y, tensors[p + "norm1"].to(F64), eps)
        f = lay.get("mlp")
        if f is not None:
            fw = sub(tensors, p + "mlp.")
            h = store(x)
            y = dense_ff(h, fw, store) if f["kind"] == "dense" else moe_ff(h, fw, f, store)
            x = rms_norm(alpha * x + y, tensors[p + "norm2"].to(F64), eps)
        if trace is not None:
            trace.append(x.clone())
    y = rms_norm(x, tensors["final.norm"].to(F64), eps)
    return store(y) @ E.T


def greedy(tensors, cfg, prompt, n_new: int, store: Callable = _keep):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(tensors, cfg, toks, store)[-1])))
    return toks[len(prompt):]
