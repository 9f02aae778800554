"""Kusirax without a GPU: the configuration reader and its errors, the model description (arrangement, joins, cache
needs, tensor names), a state row that is used again, the random-weights folder, and the plain statement against
itself."""
import copy
import json
import math

import pytest
import torch

import plain_kusirax as P
from kusirax_models import CFG_A, CFG_B, attn, attn2, clean, config, dense, layer, make_tensors, moe, wkv


def _spec(cfg):
    import mini_llm_b200  # noqa: F401
    from mini_llm_b200.config.base import config_from_dict, get_architecture
    c = config_from_dict(clean(cfg))
    return c, get_architecture(c.architecture).build_spec(c)


def test_every_size_is_read_per_layer():
    c, spec = _spec(CFG_A)
    assert c.architecture == "Kusirax" and (c.vocab, c.width, c.norm_eps, c.postln_alpha) == (97, 64, 1e-5, 2.0)
    a, b, d, e = (l.mixer for l in c.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.chunk, a.softcap, a.v_mix, a.rot_dims) == (6, 2, 20, 12, 0.9, 24, 5.0, True, 0)
    assert (b.heads, b.dim, b.decay_rank) == (3, 16, None) and (e.heads, e.dim) == (1, 40)
    assert (d.heads, d.kv_heads, d.rot_dims, d.rot_base, d.chunk, d.softcap) == (2, 1, 8, 100.0, None, None)
    assert d.rot_scaling == dict(factor=4.0, low=1.0, high=4.0, original=32.0)
    f0, f1, f2, f3 = (l.mlp for l in c.layers)
    assert (f0.experts, f0.top, f0.expert_ff, f0.scale, f0.groups, f0.keep) == (6, 3, 24, 1.7, 3, 2)
    assert f1.ff == 72 and f2 is None and (f3.experts, f3.top, f3.groups, f3.keep, f3.scale) == (4, 1, 1, 1, 1.0)
    assert all(l.arrangement == "post_norm" and l.mixer_norm is None and l.ff_norm is None for l in spec.layers)
    assert all(l.mixer_join.kind == "post_norm" and l.mixer_join.params["alpha"] == 2.0 for l in spec.layers)
    assert spec.layers[2].ff is None and spec.layers[2].ff_join is None and spec.layers[0].ff_join.kind == "post_norm"
    assert [l.mixer.kind for l in spec.layers] == ["rotary_attention", "wkv", "rotary_attention", "wkv"]
    m0, m2 = spec.layers[0].mixer.params, spec.layers[2].mixer.params
    # the first layer that mixes values keeps them, the later one mixes them in; only attention_2 has biases, a cap and slopes
    assert (m0["value_mix"], m0["bias"], m0["softcap"], m0["distance_slopes"], m0["rot_dims"], m0["head_norm"]) == ("first", True, 5.0, True, 0, True)
    assert (m2["value_mix"], m2["bias"], m2["softcap"], m2["distance_slopes"], m2["rot_interleaved"], m2["qk_norm"]) == ("mix", False, None, False, False, False)
    p = spec.layers[0].ff.params
    assert (p["selection"], p["activation"], p["group_sum"], p["weight_scale"], p["groups"], p["keep"]) == ("sigmoid", "relu_sq", 2, 1.7, 3, 2)
    assert spec.layers[1].ff.kind == "gated_mlp" and spec.layers[1].ff.params["activation"] == "gelu_tanh"
    assert spec.embedding.params["norm_eps"] == 1e-5 and spec.final_norm.kind == "rmsnorm" and spec.head.kind == "tied"


def test_a_layer_that_alone_mixes_values_and_one_that_does_not():
    _, spec = _spec(CFG_B)
    assert [l.mixer.params.get("value_mix") for l in spec.layers] == [None, None, "first", None, None]
    assert spec.layers[4].ff is None and spec.layers[3].ff.params["top"] == 3
    assert r"^l1\.mix\.vmix$" in spec.ignored_tensors and r"^l4\.norm2$" in spec.ignored_tensors


def test_cache_needs_and_tensor_names():
    from mini_llm_b200.cache.manager import CacheManager, PagedNeed, StateNeed
    from mini_llm_b200.parts.model import Model
    _, spec = _spec(CFG_A)
    needs = Model(spec).layer_needs()
    # key rows padded to 16-byte pieces (20 -> 24); values of another size; the block size travels with the need; a
    # recurrence keeps its heads' states and one row of the width
    assert needs[0] == PagedNeed(kv_heads=2, head_dim=24, v_head_dim=12, chunk=24)
    assert needs[2] == PagedNeed(kv_heads=1, head_dim=16, v_head_dim=24)
    assert needs[1] == StateNeed((3 * 16 * 16 + 64,), "float32") and needs[3] == StateNeed((40 * 40 + 64,), "float32")
    cm = CacheManager(needs, page_size=8, num_pages=4, max_num_seqs=2, allocate=False)
    assert sorted(sorted(g.layers) for g in cm.groups) == [[0], [2]]
    names = {ref.canonical for _, ps in spec.all_part_specs() for ref in ps.weights.values()}
    assert names == set(make_tensors(CFG_A, 0))
    assert {"embed.norm", "l0.mix.q.b", "l0.mix.vmix", "l2.mix.vmix", "l0.mlp.router", "l0.mlp.e5.down", "l1.mix.mu.w", "l1.mix.w1",
            "l1.mix.w2", "l1.mix.w0", "l1.mix.u", "l1.mix.norm", "l1.mlp.gate", "l3.mlp.e0.up", "final.norm"} <= names
    assert not {"l2.norm2", "l2.mix.q.b", "l0.mlp.e0.gate", "l1.mix.w"} & names
    _, spec_b = _spec(CFG_B)
    assert {ref.canonical for _, ps in spec_b.all_part_specs() for ref in ps.weights.values()} == set(make_tensors(CFG_B, 0))


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="mamba2"), "type must be one of"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "not a multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=22), "at most dim"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(base=1.0), "greater than 1"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].update(high=0.5), "high > low"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("original"), "original must be a number"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size must be >= 1"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=0.0), "softcap must be positive"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim must be an integer"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=20), "mixes its 20 values"),
    (lambda c: c["layers"][1]["mixer"].pop("dim"), "dim must be an integer"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top=5 of 2 groups of 2"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "6 experts in 4 groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind must be one of"),
    (lambda c: c.pop("postln_alpha"), "missing required key 'postln_alpha'"),
    (lambda c: c.pop("norm"), "missing required key 'norm'"),
])
def test_config_errors(change, match):
    from mini_llm_b200.config.base import ConfigError
    cfg = copy.deepcopy(clean(CFG_A))
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        _spec(cfg)


def test_sizes_no_kernel_takes_are_refused_before_a_device_is_touched():
    from mini_llm_b200.parts.model import Model
    _, spec = _spec(config(32, 20, 1e-5, 1.0, [layer(wkv(1, 300, 2), None)]))
    assert any("heads of 300" in m for m in Model(spec).kernel_limits("float32"))


def test_a_state_row_that_is_used_again_is_zero():
    from mini_llm_b200.cache.manager import CacheManager
    from mini_llm_b200.parts.model import Model
    _, spec = _spec(CFG_A)
    cm = CacheManager(Model(spec).layer_needs(), page_size=8, num_pages=8, max_num_seqs=1, allocate=True, device="cpu")
    cm.admit("a")
    slot = cm.slot("a")
    for st in cm.states.values():
        st[slot].fill_(5.0)
    cm.release("a")
    cm.admit("b")
    assert cm.slot("b") == slot and all(float(st[slot].abs().max()) == 0.0 for st in cm.states.values())


def test_random_weights_folder_loads_by_name(tmp_path):
    from mini_llm_b200 import write_random_model
    from mini_llm_b200.weights.safetensors_io import Checkpoint
    cfg = clean(CFG_A)
    with pytest.raises(ValueError, match="leaves a size"):         # the decay's rank is a size of the checkpoint: random weights need it
        write_random_model(cfg, 5, str(tmp_path / "no"), dtype="bfloat16")
    cfg["layers"][1]["mixer"]["decay_rank"], cfg["layers"][3]["mixer"]["decay_rank"] = 5, 3
    out = write_random_model(cfg, 5, str(tmp_path / "m"), dtype="bfloat16")
    ck = Checkpoint(out)
    assert set(ck.names()) == set(make_tensors(CFG_A, 0))
    assert tuple(ck.shape("l0.mix.q")) == (120, 64) and tuple(ck.shape("l0.mix.k.b")) == (40,) and tuple(ck.shape("l0.mix.vmix")) == ()
    assert tuple(ck.shape("l1.mix.w1")) == (5, 64) and tuple(ck.shape("l1.mix.w2")) == (48, 5) and tuple(ck.shape("l1.mix.u")) == (3, 16)
    assert tuple(ck.shape("l3.mix.w2")) == (40, 3) and tuple(ck.shape("l0.mlp.e2.up")) == (24, 64) and tuple(ck.shape("l2.mix.o")) == (64, 48)
    with open(tmp_path / "m" / "config.json") as f:
        assert json.load(f)["architecture"] == "Kusirax"


def test_plain_statement_against_itself():
    g = torch.Generator().manual_seed(0)
    F64 = torch.float64
    cfg = clean(CFG_A)
    t = make_tensors(CFG_A, 1)
    ids = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    full = P.forward(t, cfg, ids)
    # a prefix's logits do not depend on what follows
    assert torch.allclose(P.forward(t, cfg, ids[:31]), full[:31], rtol=1e-9, atol=1e-9)
    # the recurrence cut in two with the state handed on equals the recurrence in one piece; so does the shift
    r, k, v = (torch.randn(20, 2, 6, generator=g, dtype=F64) for _ in range(3))
    w = torch.rand(20, 2, 6, generator=g, dtype=F64)
    u = torch.randn(2, 6, generator=g, dtype=F64)
    o, S = P.wkv_scan(r, k, v, w, u)
    o1, S1 = P.wkv_scan(r[:7], k[:7], v[:7], w[:7], u)
    o2, S2 = P.wkv_scan(r[7:], k[7:], v[7:], w[7:], u, S1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(S2, S)
    h = torch.randn(9, 5, generator=g, dtype=F64)
    mu = torch.rand(5, generator=g, dtype=F64)
    assert torch.allclose(torch.cat([P.token_shift(h[:4], mu), P.token_shift(h[4:], mu, h[3])]), P.token_shift(h, mu))
    assert torch.allclose(P.token_shift(h, mu)[0], h[0] * (1.0 - mu))          # zeros before the first token
    # the closed form of one state row: S_T[i] = sum_t (prod_{s>t} w_s[i]) k_t[i] v_t; the bonus touches the output only
    i = 3
    closed = sum(torch.prod(w[t + 1:, 0, i]) * k[t, 0, i] * v[t, 0] for t in range(20))
    assert torch.allclose(S[0, i], closed)
    o_no_bonus, _ = P.wkv_scan(r, k, v, w, torch.zeros_like(u))
    assert torch.allclose(o[0] - o_no_bonus[0], (r[0] * u * k[0]).sum(-1, keepdim=True) * v[0])
    # the decay lies in (0, 1): a very negative w0 never forgets, a large one forgets at once
    d = P.decay(torch.zeros(1, 4, dtype=F64), torch.zeros(2, 4, dtype=F64), torch.zeros(3, 2, dtype=F64), torch.tensor([-30.0, 0.0, 3.0], dtype=F64))
    assert d[0, 0] > 1 - 1e-12 and d[0, 1] == pytest.approx(math.exp(-1.0)) and d[0, 2] < 1e-8
    # the block mask by hand
    assert P.visible(7, 3).tolist() == [[j <= i and i // 3 == j // 3 for j in range(7)] for i in range(7)]
    # slopes: powers of two when the heads divide 8; the penalty is on i - j, not on j
    assert P.slopes(4).tolist() == [0.25, 0.0625, 0.015625, 0.00390625] and P.slopes(3)[0] == pytest.approx(2.0 ** (-8.0 / 3.0))
    # frequencies: short wavelengths stay, long ones are slowed by the factor, between the two the mix
    f = P.frequencies(48, 5e5, dict(factor=6.0, low=1.0, high=4.0, original=512))
    plain = P.frequencies(48, 5e5, None)
    assert torch.equal(f[:6], plain[:6]) and torch.allclose(f[-4:], plain[-4:] / 6.0) and torch.all((f <= plain) & (f >= plain / 6.0))
    assert any(plain[n] / 6.0 * 1.0001 < f[n] < plain[n] * 0.9999 for n in range(24))
    # a pair turned to position p and one turned to position q score by p - q alone (angles are 32-bit)
    a, b = torch.randn(1, 8, generator=g, dtype=F64), torch.randn(1, 8, generator=g, dtype=F64)
    fr = P.frequencies(6, 50.0, None)
    dot = lambda i, j: float((P.rotate_half(a, torch.tensor([i]), 6, fr) * P.rotate_half(b, torch.tensor([j]), 6, fr)).sum())
    assert dot(9, 4) == pytest.approx(dot(25, 20), rel=1e-5, abs=1e-5) and abs(dot(9, 4) - dot(9, 5)) > 1e-3
    assert torch.equal(P.rotate_half(a, torch.tensor([3]), 6, fr)[:, 6:], a[:, 6:])
    # the router: only experts of the kept groups, weights that sum to the scale
    hh = torch.randn(30, 16, generator=g, dtype=F64)
    W = torch.randn(6, 16, generator=g, dtype=F64)
    idx, wt = P.route(hh, W, dict(top=2, scale=1.7, groups=dict(count=3, keep=1)))
    assert torch.all(idx[:, 0] // 2 == idx[:, 1] // 2) and torch.allclose(wt.sum(-1), torch.full((30,), 1.7, dtype=F64))
    # an expert: the square of relu, so a negative product gives nothing
    y = P.expert(torch.ones(1, 1, dtype=F64), dict(up=torch.tensor([[-3.0], [2.0]], dtype=F64), down=torch.ones(1, 2, dtype=F64)))
    assert float(y) == 4.0
    # the norm after the sum: alpha weighs the residual against the branch
    x = torch.randn(3, 8, generator=g, dtype=F64)
    assert torch.allclose(P.rms_norm(5.0 * x, torch.ones(8, dtype=F64), 0.0), P.rms_norm(x, torch.ones(8, dtype=F64), 0.0))
