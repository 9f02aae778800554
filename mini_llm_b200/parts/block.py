"""Arrangements: how a layer's norms, mixer and feed-forward are wired.

"pre_norm" is the reference's block (src/model/gpt2_model.cu:271-365):
x += mixer(norm(x)); x += ff(norm(x)), with the residual stream x in 32-bit.
"parallel": x += mixer(norm_a(x)) + ff(norm_b(x)), both branches reading the same x.
"sandwich": x = join_a(x, mixer(norm_a(x))); x = join_b(x, ff(norm_b(x))): a branch's result goes through the layer's
join (a second norm and a scale per column, say) before it reaches x.
"post_norm": x = norm_a(alpha * x + mixer(x)); x = norm_b(alpha * x + ff(x)): the branches read x itself and the norm
comes after the sum (the joins are ``parts.join.PostNormJoin``); the layer has no norms in front of its branches.
"""
from __future__ import annotations

from .base import register_part


def _norm(norm, consumer, x, ctx):
    # a consumer that says so gets the norm unevaluated, to fuse it into its first product
    if getattr(consumer, "accepts_lazy_norm", False) and getattr(norm, "supports_lazy", False):
        return norm.forward(x, ctx, lazy=True)
    return norm.forward(x, ctx)


def pre_norm(layer, x, ctx, cache):
    layer.mixer.forward(_norm(layer.mixer_norm, layer.mixer, x, ctx), ctx, cache, x)
    if layer.ff is not None:
        layer.ff.forward(_norm(layer.ff_norm, layer.ff, x, ctx), ctx, x)
    return x


register_part("arrangement", "pre_norm", lambda: pre_norm)


def parallel(layer, x, ctx, cache):
    """x += mixer(norm_a(x)) + ff(norm_b(x)): both norms read the same x, so everything that reads x runs before
    anything adds to it.  With few, narrow rows (decode steps; the norms say when it pays) both norms ride in the loads of the branches' first products:
    the feed-forward's first product is issued before the mixer, whose last product changes x.  With many rows two
    RMS norms that differ only in their weights share one kernel."""
    if layer.ff is None:
        layer.mixer.forward(_norm(layer.mixer_norm, layer.mixer, x, ctx), ctx, cache, x)
        return x
    pays = getattr(layer.mixer_norm, "lazy_pays", None), getattr(layer.ff_norm, "lazy_pays", None)
    lazy = (pays[0] is not None and pays[1] is not None and pays[0](x.shape[0]) and pays[1](x.shape[0])
            and getattr(layer.mixer, "accepts_lazy_norm", False) and getattr(layer.ff, "accepts_lazy_norm", False)
            and hasattr(layer.ff, "project"))
    if lazy:
        gu = layer.ff.project(layer.ff_norm.forward(x, ctx, lazy=True, name="norm_out_b"), ctx)
        layer.mixer.forward(layer.mixer_norm.forward(x, ctx, lazy=True), ctx, cache, x)
        layer.ff.finish(gu, ctx, x)
        return x
    pair = getattr(layer.mixer_norm, "pairs_with", None)
    if pair is not None and pair(layer.ff_norm):
        h1, h2 = layer.mixer_norm.forward_pair(layer.ff_norm, x, ctx)
    else:
        h1 = layer.mixer_norm.forward(x, ctx)
        h2 = layer.ff_norm.forward(x, ctx)
        if h2.data_ptr() == h1.data_ptr():
            raise RuntimeError("parallel arrangement: the two norms wrote to the same buffer")
    layer.mixer.forward(h1, ctx, cache, x)
    layer.ff.forward(h2, ctx, x)
    return x


register_part("arrangement", "parallel", lambda: parallel)


def _branch(part, y, *args):
    """Run a mixer or feed-forward so that y holds its result (not a sum with what y held)."""
    if getattr(part, "can_overwrite", False):
        part.forward(*args, y, accumulate=False)
    else:
        y.zero_()
        part.forward(*args, y)


def sandwich(layer, x, ctx, cache):
    """x <- join(x, branch(norm(x))) for the mixer and then for the feed-forward: the branch writes a 32-bit buffer of
    its own, and the layer's join (``LayerSpec.mixer_join`` / ``ff_join``) brings it into the residual stream.  Where the
    parts allow it, the mixer's join also norms the new x for the feed-forward (one kernel), and a routed feed-forward
    leaves the weighted sum over a token's experts to its join (``forward_pairs``)."""
    import torch
    from .norm import RMSNorm
    if layer.mixer_join is None or (layer.ff is not None and layer.ff_join is None):
        raise RuntimeError("sandwich arrangement: the layer has no join for a branch")
    y = ctx.ws.buf("branch_out", x.shape[0], x.shape[1], torch.float32)
    _branch(layer.mixer, y, _norm(layer.mixer_norm, layer.mixer, x, ctx), ctx, cache)
    fuse = layer.ff is not None and isinstance(layer.ff_norm, RMSNorm) and getattr(layer.mixer_join, "norms_next", False)
    h = layer.mixer_join.forward(y, x, ctx, then_norm=layer.ff_norm) if fuse else layer.mixer_join.forward(y, x, ctx)
    if layer.ff is not None:
        if not fuse:
            h = _norm(layer.ff_norm, layer.ff, x, ctx)
        if hasattr(layer.ff, "forward_pairs") and getattr(layer.ff_join, "takes_pairs", False):
            shared, pairs = layer.ff.forward_pairs(h, ctx, y)
            layer.ff_join.forward(y if shared else None, x, ctx, pairs=pairs)
        else:
            _branch(layer.ff, y, h, ctx)
            layer.ff_join.forward(y, x, ctx)
    return x


register_part("arrangement", "sandwich", lambda: sandwich)


def post_norm(layer, x, ctx, cache):
    """x <- join_a(x, mixer(x)); x <- join_b(x, ff(x)) with joins that norm after the sum.  A branch reads x as the
    products take it (the activation dtype): the copy that the join before it made (``ctx.carry``: the embedding's norm
    or the layer before left it there), or x itself on the 32-bit path."""
    import torch
    if layer.mixer_join is None or (layer.ff is not None and layer.ff_join is None):
        raise RuntimeError("post_norm arrangement: the layer has no join for a branch")
    h = _take_act_copy(ctx, x, layer.mixer.rt.act_dtype)
    y = ctx.ws.buf("branch_out", x.shape[0], x.shape[1], torch.float32)
    _branch(layer.mixer, y, h, ctx, cache)
    h = layer.mixer_join.forward(y, x, ctx)
    if layer.ff is not None:
        if hasattr(layer.ff, "forward_pairs") and getattr(layer.ff_join, "takes_pairs", False):
            shared, pairs = layer.ff.forward_pairs(h, ctx, y)
            h = layer.ff_join.forward(y if shared else None, x, ctx, pairs=pairs)
        else:
            _branch(layer.ff, y, h, ctx)
            h = layer.ff_join.forward(y, x, ctx)
    leave_act_copy(ctx, x, h)
    return x


def leave_act_copy(ctx, x, h) -> None:
    """Whoever has just written the residual x leaves its copy in the activation dtype for the next reader."""
    if hasattr(ctx, "carry"):
        ctx.carry = ("act_copy", x, h)


def _take_act_copy(ctx, x, act_dtype):
    """The copy of x in the activation dtype that the last writer of x left, or one made now."""
    left = getattr(ctx, "carry", None)
    if isinstance(left, tuple) and len(left) == 3 and left[0] == "act_copy" and left[1].data_ptr() == x.data_ptr():
        ctx.carry = None
        return left[2]
    if x.dtype == act_dtype:
        return x
    raise RuntimeError("post_norm arrangement: nobody left a copy of the residual in the activation dtype "
                       "(the embedding of such a model norms its rows and leaves one)")


register_part("arrangement", "post_norm", lambda: post_norm)
