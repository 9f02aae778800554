"""Mumopel without a GPU: the configuration reader and its errors, the model description (schedule, cache units, cache
needs, tensor names), pages that a block mask lets go, the random-weights folder, and the plain statement against
itself."""
import copy
import json
import math

import pytest
import torch

import plain_mumopel as P
from mumopel_models import CFG_R, CFG_S, attn, config, dense, layer, make_tensors, moe


def _spec(cfg):
    import mini_llm_b200  # noqa: F401
    from mini_llm_b200.config.base import config_from_dict, get_architecture
    c = config_from_dict(cfg)
    return c, get_architecture(c.architecture).build_spec(c)


def test_every_size_is_read_per_layer():
    c, spec = _spec(CFG_R)
    assert c.architecture == "Mumopel" and (c.vocab, c.width, c.norm_eps, c.streams, c.logit_softcap) == (97, 64, 1e-5, 2, 8.0)
    a, b, d = (l.mixer for l in c.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.rot_dims, a.rot_base, a.chunk) == (6, 2, 20, 12, 0.45, 8, 100.0, 24)
    assert (b.heads, b.kv_heads, b.rot_dims, b.chunk) == (2, 2, 16, 37) and (d.rot_dims, d.chunk, d.kv_heads) == (0, None, 1)
    f0, f1, f2 = (l.mlp for l in c.layers)
    assert (f0.experts, f0.top, f0.expert_ff, f0.expert_limit, f0.shared_ff, f0.shared_limit) == (5, 2, 24, 0.7, 40, 1.5)
    assert f1.ff == 72 and f2 is None
    assert (c.loop.start, c.loop.stop, c.loop.times) == (0, 2, 2) and c.layer_order() == [0, 1, 0, 1, 2] == P.layer_order(CFG_R)
    # the second run of a looped layer has a cache of its own, beyond the layers' own units
    assert [(e.layer, e.private_cache, e.cache_unit) for e in spec.schedule] == \
        [(0, False, 0), (1, False, 1), (0, True, 3), (1, True, 4), (2, False, 2)]
    assert all(l.arrangement == "hyper" for l in spec.layers) and spec.layers[2].ff is None and spec.layers[2].ff_join is None
    assert spec.layers[0].ff.kind == "moe" and spec.layers[1].ff.kind == "gated_mlp"
    assert spec.embedding.params["copies"] == 2 and spec.final_norm.kind == "stream_sum_layernorm"
    assert spec.head.kind == "tied" and spec.head.params["softcap"] == 8.0 and spec.positions.kind == "none"
    p = spec.layers[0].ff.params
    assert (p["selection"], p["activation"], p["router_bias"], p["limit"], p["shared_limit"], p["alpha"]) == \
        ("softmax_top", "swiglu_clamp", True, 0.7, 1.5, 1.702)


def test_a_model_without_streams_loop_and_cap():
    c, spec = _spec(CFG_S)
    assert c.streams is None and c.loop is None and c.logit_softcap is None
    assert all(l.arrangement == "pre_norm" and l.mixer_join is None for l in spec.layers)
    assert spec.final_norm.kind == "layernorm" and spec.embedding.params["copies"] == 1 and spec.head.params["softcap"] is None
    assert [(e.layer, e.private_cache) for e in spec.schedule] == [(0, False), (1, False), (2, False)]
    assert spec.layers[0].ff.params["shared_size"] is None and spec.layers[2].ff.params["top"] == 3


def test_cache_needs_and_tensor_names():
    from mini_llm_b200.cache.manager import CacheManager, PagedNeed
    from mini_llm_b200.parts.model import Model
    _, spec = _spec(CFG_R)
    needs = Model(spec).layer_needs()
    # key rows padded to 16-byte pieces (20 -> 24); values of another size; the block size travels with the need
    assert needs[0] == needs[3] == PagedNeed(kv_heads=2, head_dim=24, v_head_dim=12, chunk=24)
    assert needs[1] == needs[4] == PagedNeed(kv_heads=2, head_dim=16, chunk=37)
    assert needs[2] == PagedNeed(kv_heads=1, head_dim=8, v_head_dim=24)
    cm = CacheManager(needs, page_size=8, num_pages=4, max_num_seqs=2, allocate=False)
    assert sorted(sorted(g.layers) for g in cm.groups) == [[0, 3], [1, 4], [2]]
    names = {ref.canonical for _, ps in spec.all_part_specs() for ref in ps.weights.values()}
    assert names == set(make_tensors(CFG_R, 0))
    assert {"l0.mix.q.norm", "l0.mix.sink", "l0.mlp.router.b", "l0.mlp.e4.down", "l0.mlp.shared.up", "l1.mlp.gate", "l0.hc2.mix",
            "l2.hc1.in", "l1.norm2.b", "final.norm.b"} <= names and not {"l2.norm2", "l2.hc2.in", "l2.mlp.gate"} & names
    _, spec_s = _spec(CFG_S)
    assert {ref.canonical for _, ps in spec_s.all_part_specs() for ref in ps.weights.values()} == set(make_tensors(CFG_S, 0))


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="mamba2"), "type must be one of"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "not a multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=22), "at most dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(base=1.0), "greater than 1"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size must be >= 1"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim must be an integer"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top=6 of 5"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0), "limit must be positive"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("limit"), "limit must be a number"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "kind must be one of"),
    (lambda c: c["loop"].update(stop=4), "no stretch of the 3 layers"),
    (lambda c: c["loop"].update(start=2, stop=2), "no stretch"),
    (lambda c: c["loop"].update(times=0), "times must be >= 1"),
    (lambda c: c.update(streams=0), "streams must be >= 1"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap must be positive"),
    (lambda c: c.pop("norm"), "missing required key 'norm'"),
])
def test_config_errors(change, match):
    from mini_llm_b200.config.base import ConfigError
    cfg = copy.deepcopy(CFG_R)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        _spec(cfg)


def test_more_streams_than_the_kernel_takes_are_refused_before_a_device_is_touched():
    from mini_llm_b200.parts.model import Model
    _, spec = _spec(config(32, 20, 1e-5, [layer(attn(1, 1, 8, 8, 0.3), None)], streams=9))
    assert any("9 streams" in m for m in Model(spec).kernel_limits("float32"))


def test_pages_of_finished_blocks_go_back():
    """A block mask lets go of what lies before the start of the next query's block, page by page."""
    from mini_llm_b200.cache.manager import RELEASED, CacheManager, PagedNeed
    cm = CacheManager({0: PagedNeed(1, 8, chunk=24), 1: PagedNeed(1, 8, v_head_dim=16)}, page_size=8, num_pages=12,
                      max_num_seqs=2, allocate=False)
    masked = cm.group_of_layer[0]
    cm.admit("a")
    assert cm.reserve("a", 23)
    cm.commit("a", 23)                       # the next query stands at 23, in block 0: everything stays
    assert cm.num_free_pages(masked) == 9
    assert cm.reserve("a", 1)
    cm.commit("a", 1)                        # the next query stands at 24: block 0 (three pages) is never read again
    assert cm.table("a", masked)[:3] == [RELEASED] * 3 and cm.num_free_pages(masked) == 12
    assert cm.reserve("a", 30)
    cm.commit("a", 30)                       # at 54: blocks 0 and 1 are gone; block 2 starts at 48 = page 6
    tab = cm.table("a", masked)
    assert tab[:6] == [RELEASED] * 6 and tab[6] != RELEASED and cm.num_free_pages(masked) == 11
    assert cm.num_free_pages(cm.group_of_layer[1]) == 12 - 7        # the unmasked layer keeps everything
    cm.check()
    cm.release("a")
    assert cm.num_free_pages(masked) == 12 and cm.num_free_pages(cm.group_of_layer[1]) == 12
    cm.check()
    # a block size that is no multiple of the page: the page that holds the block's start stays
    cm2 = CacheManager({0: PagedNeed(1, 8, chunk=20)}, page_size=8, num_pages=12, max_num_seqs=1, allocate=False)
    cm2.admit("b")
    cm2.reserve("b", 41)
    cm2.commit("b", 41)                      # block 2 starts at 40 = page 5
    assert cm2.table("b", 0)[:5] == [RELEASED] * 5 and cm2.table("b", 0)[5] != RELEASED


def test_random_weights_folder_loads_by_name(tmp_path):
    from mini_llm_b200 import write_random_model
    from mini_llm_b200.weights.safetensors_io import Checkpoint
    out = write_random_model(CFG_R, 5, str(tmp_path / "m"), dtype="bfloat16")
    ck = Checkpoint(out)
    assert set(ck.names()) == set(make_tensors(CFG_R, 0))
    assert tuple(ck.shape("l0.mix.q")) == (120, 64) and tuple(ck.shape("l0.mix.k.norm")) == (40,)
    assert tuple(ck.shape("l0.mix.o")) == (64, 72) and tuple(ck.shape("l0.hc1.mix")) == (2, 2) and tuple(ck.shape("l0.mix.sink")) == (6,)
    assert tuple(ck.shape("l0.mlp.router.b")) == (5,) and tuple(ck.shape("l0.mlp.shared.down")) == (64, 40)
    with open(tmp_path / "m" / "config.json") as f:
        assert json.load(f)["architecture"] == "Mumopel"


def test_plain_statement_against_itself():
    g = torch.Generator().manual_seed(0)
    F64 = torch.float64
    # a prefix's logits do not depend on what follows
    t = make_tensors(CFG_R, 1)
    ids = torch.randint(0, CFG_R["vocab"], (60,), generator=g).tolist()
    full = P.forward(t, CFG_R, ids)
    assert torch.allclose(P.forward(t, CFG_R, ids[:31]), full[:31], rtol=1e-9, atol=1e-9)
    assert full.abs().max() < 8.0            # the cap
    # when every layer has the same block size, a token's logits depend on the tokens of its block only
    cfg = config(32, 50, 1e-5, [layer(attn(2, 1, 8, 8, 0.5, rot=(4, 10.0), chunk=16), dense(16)),
                                layer(attn(1, 1, 16, 8, 0.5, rot=(16, 10.0), chunk=16), moe(3, 2, 8, 1.0))], streams=3)
    t2 = make_tensors(cfg, 2)
    ids2 = torch.randint(0, 50, (40,), generator=g).tolist()
    other = [(x + 7) % 50 for x in ids2[:16]] + ids2[16:]
    a, b = P.forward(t2, cfg, ids2), P.forward(t2, cfg, other)
    assert torch.allclose(a[16:], b[16:], rtol=1e-9, atol=1e-9) and not torch.allclose(a[:16], b[:16])
    # the block mask by hand
    m = P.visible(7, 3)
    assert m.tolist() == [[j <= i and i // 3 == j // 3 for j in range(7)] for i in range(7)]
    # the sink only takes weight away: rows sum to 1 - exp(sink) / (exp(sink) + sum exp(s))
    s = torch.randn(2, 5, 5, generator=g, dtype=F64)
    sink = torch.tensor([0.3, -40.0], dtype=F64)
    p = P.sink_softmax(s, P.visible(5, None), sink)
    z = torch.exp(s[0, 4]).sum()
    assert torch.allclose(p[0, 4].sum(), z / (z + math.exp(0.3))) and torch.allclose(p[1].sum(-1), torch.ones(5, dtype=F64))
    # a pair turned to position p and one turned to position q score by p - q alone (angles are 32-bit)
    u, v = torch.randn(1, 8, generator=g, dtype=F64), torch.randn(1, 8, generator=g, dtype=F64)
    dot = lambda i, j: float((P.rotate_pairs(u, torch.tensor([i]), 6, 50.0) * P.rotate_pairs(v, torch.tensor([j]), 6, 50.0)).sum())
    assert dot(9, 4) == pytest.approx(dot(25, 20), rel=1e-5, abs=1e-5) and abs(dot(9, 4) - dot(9, 5)) > 1e-3
    assert torch.equal(P.rotate_pairs(u, torch.tensor([3]), 6, 50.0)[:, 6:], u[:, 6:])
    # the router: the largest logits after the bias, weights that sum to one
    h = torch.randn(30, 16, generator=g, dtype=F64)
    W, bias = torch.randn(6, 16, generator=g, dtype=F64), torch.tensor([0.0, 0.0, 50.0, 0.0, 0.0, -50.0], dtype=F64)
    idx, w = P.route(h, W, bias, 2)
    assert torch.all(idx[:, 0] == 2) and not torch.any(idx == 5) and torch.allclose(w.sum(-1), torch.ones(30, dtype=F64))
    # an expert's limits: a large gate is cut off, a large up value on both sides
    big = dict(gate=torch.tensor([[100.0]], dtype=F64), up=torch.tensor([[-100.0]], dtype=F64), down=torch.ones(1, 1, dtype=F64))
    y = P.clamped_expert(torch.ones(1, 1, dtype=F64), big, 2.0)
    assert float(y) == pytest.approx(2.0 / (1.0 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0))
    # streams: with the identity as the mixing matrix and unit weights, S streams of one model are S copies of a plain residual
    x = [torch.randn(4, 8, generator=g, dtype=F64)] * 2
    hc = {"in": torch.tensor([0.5, 0.5], dtype=F64), "out": torch.ones(2, dtype=F64), "mix": torch.eye(2, dtype=F64)}
    w8, b8 = torch.ones(8, dtype=F64), torch.zeros(8, dtype=F64)
    two = P.sublayer(x, lambda z: 2.0 * z, hc, w8, b8, 1e-5, lambda z: z)
    one = P.sublayer(x[:1], lambda z: 2.0 * z, None, w8, b8, 1e-5, lambda z: z)
    assert torch.allclose(two[0], one[0]) and torch.allclose(two[1], one[0])
