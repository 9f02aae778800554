"""The kernels that came with the Mumopel design, each alone against the plain float64 statement of its mechanism
(tests/plain_mumopel.py), at sizes of their own: the norm over whole query and key projections with the rotation and
the cache write, attention under a block mask with a sink in all its kernels, the pass over a residual of several
streams, the router that weighs the chosen logits, clamped experts, capped logits, the embedding's copies."""
import math

import pytest
import torch

import plain_mumopel as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from mini_llm_b200 import ops as o
    o.library()
    return o


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.2e-2


class _Ctx:
    pass


# ------------------------------------------------------------------------------------------------ norm + rotation + cache
def _rotate_halves(x, positions, dims, base):
    """The other pairing: entry i with i + dims/2 (x [..., T, d])."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    f = (float(base) ** (-2.0 * i / dims)).to(torch.float32)
    a = (positions.to(torch.float32)[:, None] * f[None, :]).to(F64)
    cos, sin = torch.cos(a), torch.sin(a)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.clone()
    out[..., :dims // 2] = u * cos - v * sin
    out[..., dims // 2:dims] = v * cos + u * sin
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("H,G,dk,dv,rot,base,normed", [
    (6, 2, 20, 12, 8, 100.0, True), (2, 2, 16, 16, 16, 20.0, True), (4, 1, 8, 24, 0, 10.0, True), (3, 3, 32, 32, 16, 3e4, False),
    (1, 1, 64, 16, 64, 1e3, True), (8, 2, 128, 128, 64, 1e4, True), (5, 5, 6, 2, 2, 3.0, False)])
def test_norm_rotation_and_cache_write(ops, dtype, interleaved, H, G, dk, dv, rot, base, normed):
    T, page, pages, eps = 23, 4, 9, 1e-5
    nq, nk, nv = H * dk, G * dk, G * dv
    lead = 8                                                  # the projection is a column slice of a wider buffer
    wide = rnd(T, lead + nq + nk + nv + 4, seed=H + dk, scale=1.5, dtype=dtype)
    qw = (rnd(nq, seed=2) * 0.5 + 1.2) * torch.where(rnd(nq, seed=3) > 0, 1.0, -1.0)
    kw = (rnd(nk, seed=4) * 0.5 + 1.2) * torch.where(rnd(nk, seed=5) > 0, 1.0, -1.0)
    g = torch.Generator().manual_seed(7)
    positions = torch.randint(0, 9000, (T,), generator=g)
    positions[0], positions[1] = 0, 1
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    dkp = -(-dk // 8) * 8
    k_pages = torch.full((pages, G, page, dkp), 7.0, device=DEV, dtype=dtype)
    k_pages[..., dk:] = 0                                     # a pool starts as zeros and the padding is never written
    v_pages = torch.full((pages, G, page, dv), 7.0, device=DEV, dtype=dtype)
    ctx = _Ctx()
    ctx.positions = positions.to(torch.int32).to(DEV)
    freq = None
    if rot:
        i = torch.arange(rot // 2, dtype=F64)
        freq = (float(base) ** (-2.0 * i / rot)).float().to(DEV)
    q_out = torch.empty(T, nq, device=DEV, dtype=dtype)
    ops.qk_norm_rope(wide[:, lead:], 0, nq, nq + nk, ctx, q_out, k_pages, v_pages, slots.to(DEV), heads=H, kv_heads=G,
                     head_dim=dk, v_head_dim=dv, q_norm=qw if normed else None, k_norm=kw if normed else None, eps=eps,
                     freq=freq, rot_dims=rot, interleaved=interleaved)
    ops.check_device_errors()
    x = wide[:, lead:].double().cpu()
    q, k, v = x[:, :nq], x[:, nq:nq + nk], x[:, nq + nk:nq + nk + nv]
    if normed:
        q = P.rms_unit(q, eps) * qw.double().cpu()
        k = P.rms_unit(k, eps) * kw.double().cpu()
    turn = P.rotate_pairs if interleaved else _rotate_halves
    q = turn(q.view(T, H, dk).transpose(0, 1), positions, rot, base).transpose(0, 1).reshape(T, nq)
    k = turn(k.view(T, G, dk).transpose(0, 1), positions, rot, base).transpose(0, 1)
    tol = _tol(dtype) * max(1.0, q.abs().max().item())
    assert (q_out.double().cpu() - q).abs().max() < tol
    kp, vp = k_pages.double().cpu(), v_pages.double().cpu()
    for t in range(T):
        s = int(slots[t])
        assert (kp[s // page, :, s % page, :dk] - k[t]).abs().max() < tol
        assert torch.all(kp[s // page, :, s % page, dk:] == 0)          # the padding of a key row is zero
        assert torch.equal(vp[s // page, :, s % page].reshape(-1), v[t])
    used = set(int(s) for s in slots)
    for s in range(pages * page):
        if s not in used:
            assert torch.all(kp[s // page, :, s % page, :dk] == 7.0) and torch.all(vp[s // page, :, s % page] == 7.0)
    # without a slot mapping nothing is cached (a layer that reads another's rows)
    k_pages.fill_(3.0)
    ops.check_device_errors()
    ops.qk_norm_rope(wide[:, lead:], 0, nq, nq + nk, ctx, q_out, k_pages, v_pages, None, heads=H, kv_heads=G, head_dim=dk,
                     v_head_dim=dv, q_norm=qw if normed else None, k_norm=kw if normed else None, eps=eps, freq=freq,
                     rot_dims=rot, interleaved=interleaved)
    assert torch.all(k_pages == 3.0) and (q_out.double().cpu() - q).abs().max() < tol


def test_the_norm_is_over_the_whole_projection_with_eps_inside_the_root(ops):
    # two heads of which one is tiny: a norm per head would blow the tiny head up to unit size
    T, H, dk = 2, 2, 8
    x = torch.zeros(T, 3 * H * dk, device=DEV)
    x[:, :dk] = 3.0
    x[:, dk:2 * dk] = 1e-3
    x[1] *= 1e-4                                              # a row so small that eps decides
    w = torch.ones(H * dk, device=DEV)
    ctx = _Ctx()
    ctx.positions = torch.zeros(T, dtype=torch.int32, device=DEV)
    q_out = torch.empty(T, H * dk, device=DEV)
    eps = 1e-6
    ops.qk_norm_rope(x, 0, H * dk, 2 * H * dk, ctx, q_out, None, None, None, heads=H, kv_heads=H, head_dim=dk, v_head_dim=dk,
                     q_norm=w, k_norm=w, eps=eps)
    for t in range(T):
        row = x[t, :H * dk].double().cpu()
        want = row / math.sqrt(float((row * row).mean()) + eps)
        assert (q_out[t].double().cpu() - want).abs().max() < 1e-6
    assert abs(q_out[0, dk].item()) < 1e-3 and abs(q_out[1, 0].item() - 3e-4 / math.sqrt(4.5e-8 + 1e-6 + 5e-15)) < 1e-6


# ------------------------------------------------------------------------------------------------ attention
def _case(dtype, seqs, H, G, dk, dv, page, seed, sharp=None, scale=None):
    """seqs: (context length, new tokens) per request.  Pages in a shuffled order, dense copies, the tile list.
    ``sharp``: {request: [positions]}: the keys there answer a direction that all of the request's queries share with
    a score that stands out, and carry value rows of their own (2, 4, 6, ...), so that a key that is dropped or wrongly
    admitted moves the result by O(1)."""
    from mini_llm_b200.engine.context import Workspace, attention_tiles
    g = torch.Generator().manual_seed(seed)
    num_pages = sum((c + page - 1) // page for c, _ in seqs) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    k_pages = torch.zeros(num_pages, G, page, -(-dk // 8) * 8)
    v_pages = torch.zeros(num_pages, G, page, dv)
    tables, dense, token_seq, positions = [], [], [], []
    for s, (c, ql) in enumerate(seqs):
        tab = [perm.pop() for _ in range((c + page - 1) // page)]
        tables.append(tab)
        dense.append((torch.randn(c, G, dk, generator=g), torch.randn(c, G, dv, generator=g)))
        token_seq += [s] * ql
        positions += list(range(c - ql, c))
    T = len(token_seq)
    q = torch.randn(T, H * dk, generator=g)
    scale = dk ** -0.5 if scale is None else scale
    if sharp:
        for s, where in sharp.items():
            u = torch.randn(G, dk, generator=g)
            u = u / u.norm(dim=1, keepdim=True) * math.sqrt(dk)
            rows = [t for t, ts in enumerate(token_seq) if ts == s]
            q[rows] = q[rows] * 0.3 + u.repeat_interleave(H // G, dim=0).reshape(1, H * dk) * 1.5
            K, V = dense[s]
            for i, p in enumerate(where):
                K[p] = u * (30.0 / math.sqrt(dk)) / (scale * math.sqrt(dk))      # a score of about 45
                V[p] = 2.0 * (i + 1)
    for s, tab in enumerate(tables):
        K, V = dense[s]
        for p in range(K.shape[0]):
            k_pages[tab[p // page], :, p % page, :dk] = K[p]
            v_pages[tab[p // page], :, p % page] = V[p]
    mp = max(len(t) for t in tables)
    bt = torch.zeros(len(seqs), mp, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    ctx = _Ctx()
    ctx.token_seq = torch.tensor(token_seq, dtype=torch.int32, device=DEV)
    ctx.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    ctx.ws = Workspace(torch.device(DEV), 64)
    ctx.max_ctx_len = max(c for c, _ in seqs)
    ctx.decode_only = all(ql == 1 for _, ql in seqs)
    tiles = attention_tiles([ql for _, ql in seqs], [c - ql for c, ql in seqs])
    ctx.attn_tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    ctx.n_tiles = len(tiles) // 3
    return dict(q=q.to(dtype).to(DEV), k_pages=k_pages.to(dtype).to(DEV), v_pages=v_pages.to(dtype).to(DEV), bt=bt.to(DEV),
                token_seq=token_seq, positions=positions, dense=dense, ctx=ctx, scale=scale, H=H, G=G, dk=dk, dv=dv,
                dtype=dtype, tables=tables, page=page)


def _want(case, chunk=None, sink=None, out_scale=1.0):
    """Query at position p of block b = floor(p / chunk) sees keys b * chunk .. p; the sink adds exp(sink_h) to the
    denominator only."""
    H, G, dk, dv, dtype = case["H"], case["G"], case["dk"], case["dv"], case["dtype"]
    q = case["q"].cpu().double()
    out = torch.zeros(q.shape[0], H * dv, dtype=F64)
    for t, (s, p) in enumerate(zip(case["token_seq"], case["positions"])):
        K, V = (x.to(dtype).double() for x in case["dense"][s])
        lo = (p // chunk) * chunk if chunk else 0
        for h in range(H):
            g = h // (H // G)
            sc = (K[lo:p + 1, g] @ q[t, h * dk:(h + 1) * dk]) * case["scale"]
            m = sc.max() if sink is None else max(sc.max(), sink[h].double().cpu())
            e = torch.exp(sc - m)
            den = e.sum() + (torch.exp(sink[h].double().cpu() - m) if sink is not None else 0.0)
            out[t, h * dv:(h + 1) * dv] = out_scale * ((e / den) @ V[lo:p + 1, g])
    return out


def _run(ops, case, impl, chunk=None, sink=None, out_scale=1.0):
    H, dv = case["H"], case["dv"]
    wide = torch.zeros(case["q"].shape[0], H * dv + 8, device=DEV, dtype=case["dtype"])
    out = wide[:, 8:] if case["dtype"] == torch.float32 else wide[:, :H * dv]
    ops.biased_attention(case["q"], case["k_pages"], case["v_pages"], case["bt"], case["ctx"], out, num_heads=H,
                         num_kv_heads=case["G"], scale=case["scale"], out_scale=out_scale, chunk=chunk, sink=sink, impl=impl)
    ops.check_device_errors()
    return out.double().cpu()


def _sinks(H, seed):
    return rnd(H, seed=seed, scale=2.0)


SHAPES = [(4, 2, 16, 24, 8), (3, 3, 32, 32, 16), (6, 1, 96, 40, 4), (2, 2, 8, 1, 16), (8, 2, 64, 256, 32), (4, 2, 20, 12, 8),
          (4, 2, 96, 80, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
@pytest.mark.parametrize("impl", ["simt", "tiled"])
def test_block_mask_and_sink_in_a_mixed_batch(ops, dtype, impl, H, G, dk, dv, page):
    # portions that start in the middle of a page and of a block, a whole prompt, single tokens, a portion of two
    seqs = [(150, 97), (31, 31), (200, 1), (67, 2), (1, 1), (130, 65)]
    case = _case(dtype, seqs, H, G, dk, dv, page, seed=H * 100 + dk)
    sink = _sinks(H, 9)
    for kw in (dict(chunk=24, sink=sink), dict(chunk=37), dict(sink=sink, out_scale=0.7), dict(chunk=64, sink=sink),
               dict(chunk=7, sink=sink), dict(chunk=1, sink=sink), dict(chunk=1000, sink=sink)):
        got, want = _run(ops, case, impl, **kw), _want(case, **kw)
        assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item()), (impl, kw.get("chunk"))


@pytest.mark.parametrize("H,G,dk,dv,page", [(3, 3, 32, 32, 16), (4, 2, 64, 128, 16), (2, 1, 128, 16, 8), (6, 2, 96, 48, 4),
                                            (4, 2, 96, 80, 16), (2, 2, 16, 16, 32)])
def test_block_mask_and_sink_on_tensor_cores(ops, H, G, dk, dv, page):
    seqs = [(150, 97), (31, 31), (200, 1), (67, 2), (1, 1), (130, 65), (260, 129)]
    case = _case(torch.bfloat16, seqs, H, G, dk, dv, page, seed=H * 100 + dk + 1)
    sink = _sinks(H, 11)
    n0 = ops.attention_launches.get("bias_mma", 0)
    for kw in (dict(chunk=24, sink=sink), dict(chunk=37), dict(sink=sink, out_scale=0.7), dict(chunk=64, sink=sink),
               dict(chunk=128, sink=sink), dict(chunk=7, sink=sink), dict(chunk=112, sink=sink)):
        got, want = _run(ops, case, "mma", **kw), _want(case, **kw)
        assert (got - want).abs().max() < _tol(torch.bfloat16) * 2 * max(1.0, want.abs().max().item()), kw.get("chunk")
    assert ops.attention_launches.get("bias_mma", 0) == n0 + 7
    _run(ops, case, None, chunk=24, sink=sink)      # left to itself the wrapper takes this kernel for such steps
    assert ops.attention_launches["bias_mma"] == n0 + 8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
def test_block_mask_and_sink_for_single_tokens(ops, dtype, H, G, dk, dv, page):
    # contexts on both sides of a block's edge, of a split of keys and of a page; the first tokens of a sequence
    for chunk in (100, 256, 24):
        seqs = [(c, 1) for c in (1, 2, chunk - 1, chunk, chunk + 1, chunk + 2, 2 * chunk, 2 * chunk + 1, 255, 256, 257, 513, 700)]
        case = _case(dtype, seqs, H, G, dk, dv, page, seed=H * 10 + dv + chunk)
        sink = _sinks(H, 13)
        for kw in (dict(chunk=chunk, sink=sink), dict(chunk=chunk), dict(sink=sink, out_scale=1.3)):
            want = _want(case, **kw)
            for impl in ("split", "simt"):
                got = _run(ops, case, impl, **kw)
                assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item()), (impl, chunk)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
@pytest.mark.parametrize("chunk", [48, 112, 64])
def test_keys_just_inside_and_just_outside_a_block(ops, impl, dtype, chunk):
    """Sharp keys on both sides of every block's first position, at page (16), key-tile (32, 64) and split edges and at
    the first positions.  A query sees the sharp keys of its own block up to itself and nothing else: the expected
    result comes from the statement, and a key admitted from the block before would move it by O(1)."""
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    c = 5 * chunk + 9
    ql = 1 if impl == "split" else chunk + 11                # the portion covers a whole block and both its edges
    where = sorted(set([0, 1, 15, 16, 31, 32, 63, 64, 255, 256] + [b * chunk + d for b in range(1, 6) for d in (-2, -1, 0, 1)]))
    where = [p for p in where if p < c - 1]
    cases = [(c, ql), (c - 8, ql), (c - 9, ql), (c - 10, ql)] if impl != "split" else \
        [(n, 1) for n in (4 * chunk - 1, 4 * chunk, 4 * chunk + 1, 4 * chunk + 2, 5 * chunk, 5 * chunk + 1, c)]
    case = _case(dtype, cases, 2, 1, 16, 16, 16, seed=6, sharp={s: [p for p in where if p < n - 1] for s, (n, _) in enumerate(cases)})
    sink = torch.tensor([-3.0, 2.0], device=DEV)
    got, want = _run(ops, case, impl, chunk=chunk, sink=sink), _want(case, chunk=chunk, sink=sink)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())
    # the statement itself: the query at a block's first position sees no sharp key (only itself), the next one sees one
    if impl == "split":
        first = got[2]                                       # context 4 * chunk + 1: the query is position 4 * chunk
        assert first.abs().max() < 6.0 and got[3].abs().min() > 6.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
def test_one_far_key_among_hundreds_inside_a_block(ops, impl, dtype):
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    ql = 1 if impl == "split" else 40
    # blocks of 1,024: the sharp key lies 600 and more positions back, in the block's first page; its value row is 2
    case = _case(dtype, [(1024 + 640, ql), (1024 + 701, ql)], 4, 2, 32, 32 if impl == "mma" else 24, 16, seed=5,
                 sharp={0: [1024 + 3], 1: [1024 + 16]})
    sink = torch.full((4,), 1.0, device=DEV)
    got, want = _run(ops, case, impl, chunk=1024, sink=sink), _want(case, chunk=1024, sink=sink)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())
    assert (got - 2.0).abs().max() < 0.05
    # the same key one block earlier is out of sight: no trace of its value row
    case = _case(dtype, [(1024 + 640, ql), (1024 + 701, ql)], 4, 2, 32, 32 if impl == "mma" else 24, 16, seed=5,
                 sharp={0: [1023], 1: [1000]})
    got, want = _run(ops, case, impl, chunk=1024, sink=sink), _want(case, chunk=1024, sink=sink)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
def test_the_sink_counts_once_unscaled_and_has_no_value(ops, impl):
    """One visible key (blocks of one position): the output is v * e^s / (e^s + e^sink) exactly, whatever ``scale`` is; a
    sink far below the scores changes nothing; a sink far above them leaves nothing."""
    dtype = torch.bfloat16 if impl == "mma" else torch.float32
    H, G, dk, dv = 4, 2, 16, 16
    ql = 1 if impl == "split" else 20
    for scale in (0.25, 3.0):
        case = _case(dtype, [(50, ql), (33, ql)], H, G, dk, dv, 8, seed=21, scale=scale)
        sink = torch.tensor([0.5, -1.0, 2.0, 0.0], device=DEV)
        got = _run(ops, case, impl, chunk=1, sink=sink)
        for t, (s, p) in enumerate(zip(case["token_seq"], case["positions"])):
            K, V = (x.to(dtype).double() for x in case["dense"][s])
            for h in range(H):
                sc = float(K[p, h // 2] @ case["q"][t, h * dk:(h + 1) * dk].double().cpu()) * scale
                w = 1.0 / (1.0 + math.exp(float(sink[h]) - sc))
                assert (got[t, h * dv:(h + 1) * dv] - w * V[p, h // 2]).abs().max() < _tol(dtype) * 4
        low, none = _run(ops, case, impl, chunk=16, sink=torch.full((H,), -80.0, device=DEV)), _run(ops, case, impl, chunk=16)
        assert (low - none).abs().max() < 1e-6
        high = _run(ops, case, impl, chunk=16, sink=torch.full((H,), 80.0, device=DEV))
        assert high.abs().max() < 1e-12


def test_the_result_does_not_depend_on_the_batch(ops):
    """A token's sums run in an order that depends on its position only: alone or beside others, bit for bit."""
    H, G, dk, dv, page, chunk = 4, 2, 32, 48, 8, 40
    sink = _sinks(H, 3)
    for dtype, impls in ((torch.float32, ("tiled", "simt")), (torch.bfloat16, ("tiled", "mma"))):
        big = _case(dtype, [(150, 97), (90, 90), (200, 1), (67, 2)], H, G, dk, dv, page, seed=77)
        for impl in impls:
            whole = _run(ops, big, impl, chunk=chunk, sink=sink)
            # the second request alone, from the same pages, cut in two
            from mini_llm_b200.engine.context import attention_tiles
            for lo, hi in ((0, 33), (33, 90)):
                one = dict(big)
                ctx = _Ctx()
                ctx.__dict__.update(big["ctx"].__dict__)
                ctx.token_seq = torch.zeros(hi - lo, dtype=torch.int32, device=DEV)
                ctx.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
                tiles = attention_tiles([hi - lo], [lo])
                ctx.attn_tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
                ctx.n_tiles = len(tiles) // 3
                one.update(q=big["q"][97 + lo:97 + hi].contiguous(), bt=big["bt"][1:2].contiguous(), ctx=ctx)
                part = _run(ops, one, impl, chunk=chunk, sink=sink)
                assert torch.equal(part, whole[97 + lo:97 + hi]), (dtype, impl, lo)


# ------------------------------------------------------------------------------------------------ several residual streams
def _hyper_want(x, S, y, mix, out_w, in_w, gamma, beta, eps):
    """(new streams [T, S, D], read [T, D], normed read)."""
    T, D = x.shape[0], x.shape[1] // S
    xs = x.view(T, S, D)
    new = xs
    if y is not None:
        new = torch.einsum("st,bsd->btd", mix, xs) + out_w[None, :, None] * y[:, None, :]
    u = torch.einsum("s,bsd->bd", in_w if in_w is not None else torch.ones(S, dtype=F64), new)
    h = None
    if gamma is not None:
        h = P.layer_norm(u, gamma, beta, eps) if beta is not None else P.rms_unit(u, eps) * gamma
    return new, u, h


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,D,T", [(1, 64, 5), (2, 100, 37), (3, 320, 9), (4, 768, 130), (8, 24, 3), (2, 2048, 17), (5, 48, 4),
                                   (7, 33, 2)])
def test_stream_pass(ops, out_dtype, S, D, T):
    eps = 1e-5
    x0 = rnd(T, S * D, seed=S + D, scale=2.0) + 0.3
    y = rnd(T, D + 8, seed=2, scale=1.5)[:, 8:]                 # a column slice: rows are not contiguous
    mix = rnd(S, S, seed=3, scale=0.4) + 0.6 * torch.eye(S, device=DEV)
    out_w, in_w = rnd(S, seed=4) + 0.2, rnd(S, seed=5, scale=0.5) + 0.6
    gamma, beta = rnd(D, seed=6, scale=0.3) + 1.0, rnd(D, seed=7, scale=0.2)
    c = lambda t: t.double().cpu()
    tol = _tol(out_dtype)
    # the write of one sublayer and the read and norm of the next in one pass
    x, h = x0.clone(), torch.empty(T, D, device=DEV, dtype=out_dtype)
    ops.hyper_step(x, S, y=y, mix=mix, out_weights=out_w, in_weights=in_w, gamma=gamma, beta=beta, eps=eps, h=h)
    new, _, hw = _hyper_want(c(x0), S, c(y), c(mix), c(out_w), c(in_w), c(gamma), c(beta), eps)
    assert (c(x).view(T, S, D) - new).abs().max() < 2e-5 * max(1.0, new.abs().max().item())
    assert (c(h) - hw).abs().max() < tol * max(1.0, hw.abs().max().item())
    # the write alone; the read alone (of the streams as they are), with and without a bias, into a column slice
    x2 = x0.clone()
    ops.hyper_step(x2, S, y=y, mix=mix, out_weights=out_w)
    assert torch.equal(x2, x)
    for b in (beta, None):
        wide = torch.zeros(T, D + 16, device=DEV, dtype=out_dtype)
        ops.hyper_step(x, S, in_weights=in_w, gamma=gamma, beta=b, eps=eps, h=wide[:, 16:])
        _, _, hw = _hyper_want(c(x), S, None, None, None, c(in_w), c(gamma), None if b is None else c(b), eps)
        assert (c(wide[:, 16:]) - hw).abs().max() < tol * max(1.0, hw.abs().max().item())
        assert torch.all(wide[:, :16] == 0) and torch.equal(x, x2)
    # the plain sum of gathered rows, normed, and the sum itself
    rows = torch.tensor([T - 1, 0, T - 1], dtype=torch.int32, device=DEV)
    h3, s3 = torch.empty(3, D, device=DEV, dtype=out_dtype), torch.empty(3, D, device=DEV)
    ops.hyper_step(x, S, gamma=gamma, beta=beta, eps=eps, rows=rows, h=h3, sum_out=s3)
    _, u, hw = _hyper_want(c(x), S, None, None, None, None, c(gamma), c(beta), eps)
    assert (c(s3) - u[rows.long().cpu()]).abs().max() < 2e-5 * max(1.0, u.abs().max().item())
    assert (c(h3) - hw[rows.long().cpu()]).abs().max() < tol * max(1.0, hw.abs().max().item())
    # a write on the way to the read of gathered rows (one of them asked for twice): the same numbers as the write of
    # all rows followed by the read, and the streams stay as they were
    x4 = x0.clone()
    h4, s4 = torch.empty(3, D, device=DEV, dtype=out_dtype), torch.empty(3, D, device=DEV)
    ops.hyper_step(x4, S, y=y, mix=mix, out_weights=out_w, gamma=gamma, beta=beta, eps=eps, rows=rows, h=h4, sum_out=s4)
    assert torch.equal(x4, x0) and torch.equal(s4, s3) and torch.equal(h4, h3)
    ops.check_device_errors()


@pytest.mark.parametrize("with_y", [True, False])
@pytest.mark.parametrize("S,D,T,top", [(2, 96, 11, 2), (3, 40, 5, 1), (6, 64, 3, 4)])
def test_stream_pass_takes_the_experts_weighted_sum(ops, S, D, T, top, with_y):
    """The written result is y (the shared expert's, if there is one) plus the sum over the token's chosen experts of
    weight * result, for all rows and on the way to a read of gathered rows."""
    eps = 1e-6
    x0 = rnd(T, S * D, seed=S + top, scale=1.5)
    y = rnd(T, D, seed=2) if with_y else None
    pair_out, pair_w = rnd(T * top, D, seed=3, scale=2.0), torch.softmax(rnd(T, top, seed=4, scale=2.0), dim=1).contiguous()
    mix = rnd(S, S, seed=5, scale=0.4) + 0.5 * torch.eye(S, device=DEV)
    out_w, in_w = rnd(S, seed=6) + 0.3, rnd(S, seed=7, scale=0.5) + 0.5
    gamma, beta = rnd(D, seed=8, scale=0.3) + 1.0, rnd(D, seed=9, scale=0.2)
    c = lambda t: t.double().cpu()
    total = (c(pair_out).view(T, top, D) * c(pair_w)[:, :, None]).sum(1) + (c(y) if with_y else 0.0)
    new, _, hw = _hyper_want(c(x0), S, total, c(mix), c(out_w), c(in_w), c(gamma), c(beta), eps)
    x, h = x0.clone(), torch.empty(T, D, device=DEV)
    ops.hyper_step(x, S, y=y, mix=mix, out_weights=out_w, in_weights=in_w, gamma=gamma, beta=beta, eps=eps, h=h,
                   pairs=(pair_out, pair_w, top))
    assert (c(x).view(T, S, D) - new).abs().max() < 2e-5 * max(1.0, new.abs().max().item())
    assert (c(h) - hw).abs().max() < 2e-5 * max(1.0, hw.abs().max().item())
    rows = torch.tensor([T - 1, 1, 1], dtype=torch.int32, device=DEV)
    x2, h2 = x0.clone(), torch.empty(3, D, device=DEV)
    ops.hyper_step(x2, S, y=y, mix=mix, out_weights=out_w, in_weights=in_w, gamma=gamma, beta=beta, eps=eps, h=h2, rows=rows,
                   pairs=(pair_out, pair_w, top))
    assert torch.equal(x2, x0) and torch.equal(h2, h[rows.long()])
    ops.check_device_errors()


def test_streams_are_written_all_at_once_from_the_old_ones(ops):
    # a mixing matrix that swaps two streams: an update in place, stream by stream, would copy one over the other
    T, D = 3, 32
    a, b = rnd(T, D, seed=1), rnd(T, D, seed=2)
    x = torch.cat([a, b], 1).contiguous()
    mix = torch.tensor([[0.0, 1.0], [1.0, 0.0]], device=DEV)       # [from, to]: stream 0 goes to 1 and back
    y = torch.zeros(T, D, device=DEV)
    ops.hyper_step(x, 2, y=y, mix=mix, out_weights=torch.zeros(2, device=DEV))
    assert torch.equal(x[:, :D], b) and torch.equal(x[:, D:], a)
    # [from, to], not [to, from]: only stream 0 feeds stream 1
    mix = torch.tensor([[0.0, 1.0], [0.0, 0.0]], device=DEV)
    x = torch.cat([a, b], 1).contiguous()
    ops.hyper_step(x, 2, y=y, mix=mix, out_weights=torch.zeros(2, device=DEV))
    assert torch.all(x[:, :D] == 0) and torch.equal(x[:, D:], a)


def test_embedding_copies(ops):
    V, D, S = 50, 40, 3
    for dtype in (torch.float32, torch.bfloat16):
        table = rnd(V, D, seed=8, dtype=dtype)
        ids = torch.tensor([4, 49, 0, 4], dtype=torch.int32, device=DEV)
        out = torch.empty(4, S * D, device=DEV)
        ops.embed(ids, torch.zeros(4, dtype=torch.int32, device=DEV), table, None, out, copies=S)
        for s in range(S):
            assert torch.equal(out[:, s * D:(s + 1) * D], table[ids.long()].float())


# ------------------------------------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("T", [1, 7, 16, 17, 300])
@pytest.mark.parametrize("E,top,D", [(5, 2, 64), (16, 4, 192), (4, 1, 96), (3, 3, 40), (64, 8, 128), (8, 2, 768)])
def test_router_weighs_the_chosen_logits(ops, T, E, top, D):
    for dtype in (torch.float32, torch.bfloat16):
        h = rnd(T, D, seed=T + E, dtype=dtype)
        router = rnd(E, D, seed=2, scale=3.0 / math.sqrt(D), dtype=dtype)
        bias = rnd(E, seed=3, scale=1.5)
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(T, top, device=DEV)
        offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
        order = torch.empty(T * top, dtype=torch.int32, device=DEV)
        ops.moe_route(h, router, idx, wts, offsets, order, top=top, bias=bias, mode="softmax_top")
        z = h.double().cpu() @ router.double().cpu().t() + bias.double().cpu()
        wi, ww = P.route(h.double().cpu(), router.double().cpu(), bias.double().cpu(), top)
        gi, gw = idx.long().cpu(), wts.double().cpu()
        for t in range(T):
            # near-ties may fall either way in 32-bit: then the chosen logit must be within rounding of the oracle's
            if not torch.equal(gi[t], wi[t]):
                assert (z[t, gi[t]] - z[t, wi[t]]).abs().max() < 1e-4
                continue
            assert (gw[t] - ww[t]).abs().max() < 2e-5
            assert abs(float(gw[t].sum()) - 1.0) < 1e-5
        # the order: every pair once, grouped by expert, tokens ascending inside an expert
        off, od = offsets.cpu().tolist(), order.cpu().tolist()
        assert off[0] == 0 and off[-1] == T * top and sorted(od) == list(range(T * top))
        for e in range(E):
            seg = od[off[e]:off[e + 1]]
            assert all(int(gi.reshape(-1)[p]) == e for p in seg) and seg == sorted(seg)
    ops.check_device_errors()


def test_router_bias_decides_and_equal_logits_take_the_lowest_index(ops):
    T, D, E = 4, 32, 6
    h = rnd(T, D, seed=1)
    router = torch.zeros(E, D, device=DEV)                      # all logits equal the bias
    bias = torch.tensor([0.0, 1.0, 1.0, -2.0, 1.0, 0.5], device=DEV)
    idx = torch.empty(T, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, 2, device=DEV)
    ops.moe_route(h, router, idx, wts, torch.empty(E + 1, dtype=torch.int32, device=DEV),
                  torch.empty(T * 2, dtype=torch.int32, device=DEV), top=2, bias=bias, mode="softmax_top")
    assert idx.cpu().tolist() == [[1, 2]] * T and torch.allclose(wts, torch.full_like(wts, 0.5))
    # the weights are a softmax over the chosen logits alone: 3 and 1 give e^3 / (e^3 + e^1) whatever the others are
    bias = torch.tensor([3.0, 0.9, -5.0, 1.0, 0.0, 0.99], device=DEV)
    ops.moe_route(h, router, idx, wts, torch.empty(E + 1, dtype=torch.int32, device=DEV),
                  torch.empty(T * 2, dtype=torch.int32, device=DEV), top=2, bias=bias, mode="softmax_top")
    assert idx.cpu().tolist() == [[0, 3]] * T
    assert abs(wts[0, 0].item() - 1.0 / (1.0 + math.exp(-2.0))) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate(ops, dtype):
    T, F = 37, 50
    wide = rnd(T, 2 * F + 6, seed=7, scale=2.5, dtype=dtype)
    gu = wide[:, :2 * F]
    for limit, alpha in ((1.0, 1.702), (2.0, 1.702), (0.5, 1.0), (7.0, 1.702)):
        out = torch.empty(T, F, device=DEV, dtype=dtype)
        ops.gated_act(gu, out, "swiglu_clamp", limit=limit, alpha=alpha)
        g = gu[:, :F].double().clamp(max=limit)                # the gate has no lower bound
        u = gu[:, F:].double().clamp(-limit, limit)
        want = g * torch.sigmoid(alpha * g) * (u + 1.0)
        assert (out.double() - want).abs().max() < _tol(dtype) * max(1.0, want.abs().max().item())
    assert (gu[:, :F] < -2.0).any() and (gu[:, :F] > 2.0).any() and (gu[:, F:].abs() > 2.0).any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,D,F", [(1, 5, 2, 64, 24), (9, 12, 3, 192, 48), (40, 4, 1, 96, 16), (200, 3, 3, 96, 8),
                                         (70, 8, 2, 768, 512), (16, 8, 2, 128, 40)])
def test_clamped_experts(ops, dtype, T, E, top, D, F):
    """Route, the experts' two products with the clamped gate between them, the weighted sum: against the statement
    with the router's own choice (so that a near-tie upstream does not decide the comparison)."""
    limit, alpha = 0.8, 1.702
    h = rnd(T, D, seed=T + F, scale=1.2, dtype=dtype)
    router = rnd(E, D, seed=2, scale=3.0 / math.sqrt(D), dtype=dtype)
    bias = rnd(E, seed=3)
    w1 = rnd(E, 2 * F, D, seed=4, scale=1.3 / math.sqrt(D), dtype=dtype)
    w2 = rnd(E, D, F, seed=5, scale=1.0 / math.sqrt(F), dtype=dtype)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(T * top, dtype=torch.int32, device=DEV)
    ops.moe_route(h, router, idx, wts, offsets, order, top=top, bias=bias, mode="softmax_top")
    mid = torch.empty(T * top, F, device=DEV, dtype=dtype)
    ops.moe_grouped(h, w1, mid, offsets, order, top=top, first=True, act="swiglu_clamp", limit=limit, alpha=alpha)
    pair_out = torch.empty(T * top, D, device=DEV)
    ops.moe_grouped(mid, w2, pair_out, offsets, order, top=top, first=False)
    out = torch.empty(T, D, device=DEV)
    ops.moe_combine(pair_out, wts, out, top=top, accumulate=False)
    ops.check_device_errors()
    store = P.to_bf16 if dtype == torch.bfloat16 else P._keep
    hd = h.double().cpu()
    want = torch.zeros(T, D, dtype=F64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            ew = {"gate": w1[e, :F].double().cpu(), "up": w1[e, F:].double().cpu(), "down": w2[e].double().cpu()}
            want[t] += float(wts[t, k]) * P.clamped_expert(hd[t:t + 1], ew, limit, store, fused=True)[0]
    assert (out.double().cpu() - want).abs().max() < _tol(dtype) * max(1.0, want.abs().max().item())


def test_capped_logits(ops):
    x = rnd(5, 1003, seed=1, scale=40.0)
    wide = torch.zeros(5, 1010, device=DEV)
    wide[:, :1003] = x
    ops.softcap(wide[:, :1003], 11.0)
    want = 11.0 * torch.tanh(x.double() / 11.0)
    assert (wide[:, :1003].double() - want).abs().max() < 2e-5 and torch.all(wide[:, 1003:] == 0)
    assert wide.abs().max() <= 11.0 and (x.abs() > 60).any()
