"""The kernels that came with the Kusirax design, each alone against the plain float64 statement of its mechanism
(tests/plain_kusirax.py), at sizes of their own: the rotation in half-split pairs with the unit norm per head and the
value mixing, attention with capped scores and a linear distance penalty in all its kernels, the recurrence with a
token-dependent decay (shift, scan, finish), the norm after the sum, the router over sigmoid scores and group sums,
experts without gates."""
import math

import pytest
import torch

import plain_kusirax as P
from test_mumopel_kernels_gpu import _Ctx, _case

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


# ------------------------------------------------------------------------------------------------ rotation, unit norm, value mixing
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,rot,base,scaling", [
    (6, 2, 20, 12, 8, 100.0, (4.0, 1.0, 4.0, 32)), (2, 2, 16, 16, 16, 20.0, None), (4, 1, 8, 24, 0, 10.0, None),
    (3, 3, 32, 32, 16, 3e4, (8.0, 0.5, 2.0, 100)), (1, 1, 64, 16, 64, 2e5, (6.0, 1.0, 4.0, 512)), (5, 5, 6, 2, 2, 3.0, None),
    (8, 2, 128, 128, 64, 1e4, (2.0, 1.0, 8.0, 64))])
def test_rotation_unit_norm_per_head_and_value_mixing(ops, dtype, H, G, dk, dv, rot, base, scaling):
    from mini_llm_b200.parts.rotary import rotary_table
    T, page, pages, eps = 23, 4, 9, 1e-5
    nq, nk, nv = H * dk, G * dk, G * dv
    wide = rnd(T, 8 + nq + nk + nv + 4, seed=H + dk, scale=1.5, dtype=dtype)        # the projection is a column slice
    g = torch.Generator().manual_seed(7)
    positions = torch.randint(0, 9000, (T,), generator=g)
    positions[0], positions[1] = 0, 1
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    dkp = -(-dk // 8) * 8
    k_pages = torch.zeros(pages, G, page, dkp, device=DEV, dtype=dtype)
    v_pages = torch.full((pages, G, page, dv), 7.0, device=DEV, dtype=dtype)
    ctx = _Ctx()
    ctx.positions = positions.to(torch.int32).to(DEV)
    sc = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
    freq = None
    if rot:
        f, _ = rotary_table(rot, base, sc)
        freq = torch.tensor(f, dtype=F64).float().to(DEV)
        assert (torch.tensor(f, dtype=F64) - P.frequencies(rot, base, sc)).abs().max() < 1e-15
    first = rnd(T, nv, seed=5, scale=2.0, dtype=dtype)
    lam = torch.tensor([0.37], device=DEV)
    kept = torch.zeros(T, nv, device=DEV, dtype=dtype)
    q_out = torch.empty(T, nq, device=DEV, dtype=dtype)
    x = wide[:, 8:].double().cpu()
    q = P.rotate_half(x[:, :nq].view(T, H, dk).transpose(0, 1), positions, rot, P.frequencies(rot, base, sc) if rot else None)
    k = P.rotate_half(x[:, nq:nq + nk].view(T, G, dk).transpose(0, 1), positions, rot, P.frequencies(rot, base, sc) if rot else None)
    q = P.rms_unit(q, eps).transpose(0, 1).reshape(T, nq)
    k = P.rms_unit(k, eps).transpose(0, 1)
    v = x[:, nq + nk:nq + nk + nv]
    tol = _tol(dtype) * max(1.0, q.abs().max().item())
    for mix in ("first", "mix", None):
        kw = {} if mix is None else (dict(v_keep=kept) if mix == "first" else dict(v_first=first, v_lambda=lam))
        ops.qk_norm_rope(wide[:, 8:], 0, nq, nq + nk, ctx, q_out, k_pages, v_pages, slots.to(DEV), heads=H, kv_heads=G,
                         head_dim=dk, v_head_dim=dv, eps=eps, freq=freq, rot_dims=rot, interleaved=False, head_norm=True, **kw)
        ops.check_device_errors()
        assert (q_out.double().cpu() - q).abs().max() < tol
        vw = v if mix != "mix" else P.mix_values(v, first.double().cpu(), 0.37)
        kp, vp = k_pages.double().cpu(), v_pages.double().cpu()
        for t in range(T):
            s = int(slots[t])
            assert (kp[s // page, :, s % page, :dk] - k[t]).abs().max() < tol
            assert torch.all(kp[s // page, :, s % page, dk:] == 0)          # the padding of a key row is zero
            assert (vp[s // page, :, s % page].reshape(-1) - vw[t]).abs().max() < _tol(dtype) * 4
        if mix == "first":
            assert torch.equal(kept.double().cpu(), v)           # the values as they are cached, for the layers that mix them in
    # every head has a root mean square of one, whatever the others hold: not a norm over the whole projection
    for h in range(H):
        rms = q_out[:, h * dk:(h + 1) * dk].double().pow(2).mean(1).sqrt().cpu()
        assert (rms - 1.0).abs().max() < (1e-4 if dtype == torch.float32 else 1e-2)


# ------------------------------------------------------------------------------------------------ attention
def _want(case, chunk=None, cap=None, slopes=False):
    """Query at position p sees keys floor(p / chunk) * chunk .. p; score = cap * tanh(q . k * scale / cap) - slope_h (p - j)."""
    H, G, dk, dv, dtype = case["H"], case["G"], case["dk"], case["dv"], case["dtype"]
    q = case["q"].cpu().double()
    sl = P.slopes(H)
    out = torch.zeros(q.shape[0], H * dv, dtype=F64)
    for t, (s, p) in enumerate(zip(case["token_seq"], case["positions"])):
        K, V = (x.to(dtype).double() for x in case["dense"][s])
        lo = (p // chunk) * chunk if chunk else 0
        for h in range(H):
            g = h // (H // G)
            sc = (K[lo:p + 1, g] @ q[t, h * dk:(h + 1) * dk]) * case["scale"]
            if cap:
                sc = cap * torch.tanh(sc / cap)
            if slopes:
                sc = sc - sl[h] * (p - torch.arange(lo, p + 1, dtype=F64))
            out[t, h * dv:(h + 1) * dv] = torch.softmax(sc, 0) @ V[lo:p + 1, g]
    return out


def _run(ops, case, impl, chunk=None, cap=None, slopes=False):
    H, dv = case["H"], case["dv"]
    wide = torch.zeros(case["q"].shape[0], H * dv + 8, device=DEV, dtype=case["dtype"])
    out = wide[:, 8:] if case["dtype"] == torch.float32 else wide[:, :H * dv]
    sl = P.slopes(H).float().to(DEV) if slopes else None
    ops.biased_attention(case["q"], case["k_pages"], case["v_pages"], case["bt"], case["ctx"], out, num_heads=H,
                         num_kv_heads=case["G"], scale=case["scale"], chunk=chunk, softcap=cap or 0.0, slopes=sl, impl=impl)
    ops.check_device_errors()
    return out.double().cpu()


SHAPES = [(4, 2, 16, 24, 8), (3, 3, 32, 32, 16), (6, 1, 96, 40, 4), (2, 2, 8, 1, 16), (4, 2, 20, 12, 8), (8, 2, 48, 32, 16)]
VARIANTS = [dict(chunk=24, cap=3.0, slopes=True), dict(chunk=37, slopes=True), dict(cap=1.5), dict(chunk=64, cap=45.0, slopes=True),
            dict(chunk=7, cap=2.0, slopes=True), dict(slopes=True), dict(chunk=112, cap=8.0, slopes=True)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
@pytest.mark.parametrize("impl", ["simt", "tiled"])
def test_capped_scores_and_slopes_in_a_mixed_batch(ops, dtype, impl, H, G, dk, dv, page):
    # portions that start in the middle of a page and of a block, a whole prompt, single tokens, a portion of two
    seqs = [(150, 97), (31, 31), (200, 1), (67, 2), (1, 1), (130, 65)]
    case = _case(dtype, seqs, H, G, dk, dv, page, seed=H * 100 + dk, scale=1.7 / math.sqrt(dk))
    for kw in VARIANTS:
        got, want = _run(ops, case, impl, **kw), _want(case, **kw)
        assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item()), (impl, kw)


@pytest.mark.parametrize("H,G,dk,dv,page", [(3, 3, 32, 32, 16), (4, 2, 64, 128, 16), (2, 1, 128, 16, 8), (6, 2, 96, 48, 4),
                                            (8, 2, 48, 32, 16), (2, 2, 16, 16, 32)])
def test_capped_scores_and_slopes_on_tensor_cores(ops, H, G, dk, dv, page):
    seqs = [(150, 97), (31, 31), (200, 1), (67, 2), (1, 1), (130, 65), (260, 129)]
    case = _case(torch.bfloat16, seqs, H, G, dk, dv, page, seed=H * 100 + dk + 1, scale=1.7 / math.sqrt(dk))
    n0 = ops.attention_launches.get("bias_mma", 0)
    for kw in VARIANTS:
        got, want = _run(ops, case, "mma", **kw), _want(case, **kw)
        assert (got - want).abs().max() < _tol(torch.bfloat16) * 2 * max(1.0, want.abs().max().item()), kw
    assert ops.attention_launches.get("bias_mma", 0) == n0 + len(VARIANTS)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
def test_capped_scores_and_slopes_for_single_tokens(ops, dtype, H, G, dk, dv, page):
    # contexts on both sides of a block's edge, of a split of keys and of a page; the first tokens of a sequence
    for chunk in (100, 256, 24, None):
        c = chunk or 300
        seqs = [(n, 1) for n in (1, 2, c - 1, c, c + 1, c + 2, 2 * c, 2 * c + 1, 255, 256, 257, 513, 700)]
        case = _case(dtype, seqs, H, G, dk, dv, page, seed=H * 10 + dv + c, scale=1.7 / math.sqrt(dk))
        for kw in (dict(chunk=chunk, cap=4.0, slopes=True), dict(chunk=chunk, slopes=True), dict(chunk=chunk, cap=0.5)):
            want = _want(case, **kw)
            for impl in ("split", "simt"):
                got = _run(ops, case, impl, **kw)
                assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item()), (impl, chunk)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
@pytest.mark.parametrize("chunk", [48, 112, 64])
def test_keys_just_inside_and_just_outside_a_block_under_a_cap(ops, impl, dtype, chunk):
    """Sharp keys on both sides of every block's first position, at page (16), key-tile (32, 64) and split edges and at
    the first positions; the cap (40) leaves their scores standing out and the slopes pull on the far ones.  A query sees
    the sharp keys of its own block up to itself and nothing else: a key admitted from the block before, or a penalty
    taken at the wrong distance, would move the result by O(1)."""
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    c = 5 * chunk + 9
    ql = 1 if impl == "split" else chunk + 11                # the portion covers a whole block and both its edges
    where = sorted(set([0, 1, 15, 16, 31, 32, 63, 64, 255, 256] + [b * chunk + d for b in range(1, 6) for d in (-2, -1, 0, 1)]))
    where = [p for p in where if p < c - 1]
    cases = [(c, ql), (c - 8, ql), (c - 9, ql), (c - 10, ql)] if impl != "split" else \
        [(n, 1) for n in (4 * chunk - 1, 4 * chunk, 4 * chunk + 1, 4 * chunk + 2, 5 * chunk, 5 * chunk + 1, c)]
    case = _case(dtype, cases, 2, 1, 16, 16, 16, seed=6, sharp={s: [p for p in where if p < n - 1] for s, (n, _) in enumerate(cases)})
    kw = dict(chunk=chunk, cap=40.0, slopes=True)
    got, want = _run(ops, case, impl, **kw), _want(case, **kw)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())
    if impl == "split":
        assert got[2].abs().max() < 6.0 and got[3].abs().min() > 6.0      # a block's first query sees itself only, the next one a sharp key


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["simt", "tiled", "split", "mma"])
def test_the_penalty_grows_with_the_distance_and_differs_by_head(ops, impl, dtype):
    """Two equally sharp keys, one 3 and one 300 positions back, no mask: head 0 (slope 1/4 with two heads) takes 75 off the
    far one's score and sees only the near one; head 1 (slope 1/256) still sees both."""
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    n = 420
    ql = 1 if impl == "split" else 70
    case = _case(dtype, [(n, ql)], 2, 1, 16, 16, 16, seed=3, sharp={0: [n - 301, n - 4]})
    got, want = _run(ops, case, impl, slopes=True), _want(case, slopes=True)
    assert (got - want).abs().max() < _tol(dtype) * 2 * max(1.0, want.abs().max().item())
    last = got[-1]
    assert (last[:16] - 4.0).abs().max() < 0.1               # head 0: the near key's value rows (4) alone
    assert ((last[16:] - 2.0).abs().min() > 0.2) and ((last[16:] - 4.0).abs().min() > 0.2)      # head 1: a mix of both


# ------------------------------------------------------------------------------------------------ recurrence
def _wkv_case(seqs, Hr, n, R, D, dtype, seed, slots=None):
    """seqs: tokens per request of one step.  Returns the inputs and a context."""
    T = sum(seqs)
    ctx = _Ctx()
    cu = [0]
    for s in seqs:
        cu.append(cu[-1] + s)
    ctx.cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
    ctx.S = len(seqs)
    ctx.state_slots = torch.tensor(slots if slots is not None else list(range(len(seqs))), dtype=torch.int32, device=DEV)
    ctx.token_seq = torch.tensor([i for i, s in enumerate(seqs) for _ in range(s)], dtype=torch.int32, device=DEV)
    N = Hr * n
    t = dict(r=rnd(T, N, seed=seed, dtype=dtype), k=rnd(T, N, seed=seed + 1, scale=0.7, dtype=dtype),
             v=rnd(T, N, seed=seed + 2, dtype=dtype), low=rnd(T, R, seed=seed + 3, scale=1.5, dtype=dtype),
             w2=rnd(N, R, seed=seed + 4, scale=0.6, dtype=dtype), u=rnd(N, seed=seed + 6, scale=0.7), h=rnd(T, D, seed=seed + 7, dtype=dtype))
    g = torch.Generator().manual_seed(seed + 5)
    t["w0"] = (torch.rand(N, generator=g) * 6.0 - 5.0).to(DEV)
    return t, ctx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hr,n,R,D", [(3, 16, 5, 64), (2, 64, 16, 96), (1, 40, 3, 64), (5, 8, 2, 24), (1, 1, 1, 8), (2, 96, 7, 32),
                                      (1, 160, 4, 16)])
def test_recurrence_in_unequal_portions_and_batches(ops, dtype, Hr, n, R, D):
    """Three requests whose tokens come in unequal portions over four steps, with slots used out of order and one
    request sitting a step out: outputs against the statement, the state the same bits as when every request runs in
    one piece, and the kept row the last row of h."""
    lens = [45, 7, 33]
    plan = [[17, 2, 1], [1, 0, 16], [16, 1, 15], [11, 4, 1]]
    slots = [2, 0, 3]
    N = Hr * n
    full, _ = _wkv_case(lens, Hr, n, R, D, dtype, seed=Hr * 7 + n)
    # a channel that never forgets next to one that forgets at once
    full["w0"][0], full["w0"][N - 1] = -30.0, 3.0
    state = torch.zeros(4, N * n + D, device=DEV)
    state[1] = 9.0                                              # a slot nobody owns: it stays as it is
    starts = [0, lens[0], lens[0] + lens[1]]
    at = [0, 0, 0]
    got = [[] for _ in lens]
    for step in plan:
        live = [i for i, c in enumerate(step) if c]
        rows = torch.cat([torch.arange(starts[i] + at[i], starts[i] + at[i] + step[i]) for i in live]).to(DEV)
        t = {k: (v[rows] if v.shape[0] == sum(lens) and k not in ("w2",) else v) for k, v in full.items()}
        _, ctx = _wkv_case([step[i] for i in live], Hr, n, R, D, dtype, seed=0, slots=[slots[i] for i in live])
        out = torch.empty(rows.numel(), N, device=DEV)
        dec = torch.empty(rows.numel(), N, device=DEV)
        ops.wkv_decay(t["low"], full["w2"], full["w0"], dec)
        ops.wkv_scan(t["r"], t["k"], t["v"], dec, full["u"], t["h"], state, N * n, ctx, out, heads=Hr, cols=(0, 32, 16, 0)[len(live) % 4])
        ops.check_device_errors()
        o = 0
        for i in live:
            got[i].append(out[o:o + step[i]].double().cpu())
            o += step[i]
            at[i] += step[i]
    one = torch.zeros(4, N * n + D, device=DEV)
    for i, L in enumerate(lens):
        sl = slice(starts[i], starts[i] + L)
        d = {k: full[k][sl].double().cpu() for k in ("r", "k", "v", "low")}
        dec = torch.exp(-torch.exp(torch.tanh(d["low"]) @ full["w2"].double().cpu().T + full["w0"].double().cpu()))
        want, S = P.wkv_scan(d["r"].view(L, Hr, n), d["k"].view(L, Hr, n), d["v"].view(L, Hr, n), dec.view(L, Hr, n),
                             full["u"].double().cpu().view(Hr, n))
        g = torch.cat(got[i])
        assert (g - want.reshape(L, N)).abs().max() < 3e-5 * max(1.0, want.abs().max().item()), i
        assert (state[slots[i], :N * n].double().cpu() - S.reshape(-1)).abs().max() < 3e-5 * max(1.0, S.abs().max().item())
        assert torch.equal(state[slots[i], N * n:].cpu(), full["h"][starts[i] + L - 1].float().cpu())
        _, ctx = _wkv_case([L], Hr, n, R, D, dtype, seed=0, slots=[slots[i]])
        out = torch.empty(L, N, device=DEV)
        dec_all = torch.empty(L, N, device=DEV)
        ops.wkv_decay(full["low"][sl], full["w2"], full["w0"], dec_all)
        assert (dec_all.double().cpu() - dec).abs().max() < 3e-6         # the decays themselves, in (0, 1)
        ops.wkv_scan(full["r"][sl], full["k"][sl], full["v"][sl], dec_all, full["u"], full["h"][sl], one, N * n, ctx, out, heads=Hr,
                     cols=16)
        assert torch.equal(one[slots[i]], state[slots[i]])       # the same bits however the tokens were cut
        # 32 or 16 columns of a state per CTA: the same outputs and the same state, bit for bit
        other, out32 = torch.zeros(4, N * n + D, device=DEV), torch.empty(L, N, device=DEV)
        ops.wkv_scan(full["r"][sl], full["k"][sl], full["v"][sl], dec_all, full["u"], full["h"][sl], other, N * n, ctx, out32, heads=Hr,
                     cols=32)
        assert torch.equal(out32, out) and torch.equal(other[slots[i]], one[slots[i]])
    assert torch.all(state[1] == 9.0)
    # the channel that never forgets still holds the first token's k v^T; the one that forgets at once only the last token's
    if N == 1:
        return
    S0 = state[slots[0], :n].double().cpu()                      # head 0, row 0
    k0 = full["k"][:lens[0], 0].double().cpu()
    v0 = full["v"][:lens[0], :n].double().cpu()
    assert (S0 - (k0[:, None] * v0).sum(0)).abs().max() < 1e-3 * max(1.0, S0.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hr,n,R,D", [(3, 16, 5, 64), (2, 64, 16, 96), (1, 40, 3, 64), (5, 8, 2, 24), (1, 1, 1, 8), (2, 96, 70, 32),
                                      (1, 128, 64, 16)])
def test_single_tokens_in_one_launch_leave_the_same_state(ops, dtype, Hr, n, R, D):
    """Five requests, a prompt portion each through decay, scan and finish, then twelve steps of single tokens through the
    single-launch kernel: its outputs equal what the three kernels give for the same tokens (rounding: the sums over the
    state's rows meet in another grouping), and the states and kept rows are the same bits."""
    assert ops.wkv_step_ok(n, R)
    lens, steps, eps = [9, 1, 20, 3, 16], 12, 1e-5
    N, B = Hr * n, 5
    slots = [4, 0, 2, 1, 3]
    state_a = torch.zeros(5, N * n + D, device=DEV)
    full, ctx = _wkv_case(lens, Hr, n, R, D, dtype, seed=n + R, slots=slots)
    z = rnd(sum(lens), N, seed=9, dtype=dtype)
    weight = rnd(N, seed=10) * 0.3 + 1.0
    dec = torch.empty(sum(lens), N, device=DEV)
    raw = torch.empty(sum(lens), N, device=DEV)
    ops.wkv_decay(full["low"], full["w2"], full["w0"], dec)
    ops.wkv_scan(full["r"], full["k"], full["v"], dec, full["u"], full["h"], state_a, N * n, ctx, raw, heads=Hr)
    state_b = state_a.clone()
    for step in range(steps):
        t, ctx1 = _wkv_case([1] * B, Hr, n, R, D, dtype, seed=100 + step, slots=slots)
        ctx1.decode_only = True
        z1 = rnd(B, N, seed=200 + step, dtype=dtype)
        dec1, raw1 = torch.empty(B, N, device=DEV), torch.empty(B, N, device=DEV)
        want = torch.empty(B, N, device=DEV, dtype=dtype)
        ops.wkv_decay(t["low"], full["w2"], full["w0"], dec1)
        ops.wkv_scan(t["r"], t["k"], t["v"], dec1, full["u"], t["h"], state_a, N * n, ctx1, raw1, heads=Hr)
        ops.wkv_finish(raw1, z1, weight, want, heads=Hr, eps=eps)
        got = torch.empty(B, N, device=DEV, dtype=dtype)
        ops.wkv_step(t["r"], t["k"], t["v"], t["low"], full["w2"], full["w0"], full["u"], z1, weight, t["h"], state_b, N * n, ctx1,
                     got, heads=Hr, eps=eps)
        ops.check_device_errors()
        assert (got.double() - want.double()).abs().max() < _tol(dtype) * max(1.0, want.double().abs().max().item()), step
        assert torch.equal(state_a, state_b), step


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_reads_the_row_before_also_across_steps(ops, dtype):
    D, NS = 40, 5
    mu = torch.rand(NS, D, generator=torch.Generator().manual_seed(1)).to(DEV)
    seqs = [5, 1, 3, 2]
    T = sum(seqs)
    _, ctx = _wkv_case(seqs, 1, 1, 1, D, dtype, seed=0, slots=[3, 1, 0, 2])
    ctx.positions = torch.tensor([0, 1, 2, 3, 4, 17, 0, 1, 2, 9, 10], dtype=torch.int32, device=DEV)
    h = rnd(T, D, seed=4, dtype=dtype)
    state = rnd(4, 7 + D, seed=5)
    mixes = torch.empty(NS, T, D, device=DEV, dtype=dtype)
    ops.wkv_shift(h, mu, state, 7, ctx, mixes)
    ops.check_device_errors()
    hd, kept = h.double().cpu(), state[:, 7:].double().cpu()
    # request 0 and 2 start at position 0 (zeros before them, whatever their slot holds); 1 and 3 go on from their kept row
    before = [None, kept[1], None, kept[2]]
    at = 0
    for i, n in enumerate(seqs):
        for s in range(NS):
            want = P.token_shift(hd[at:at + n], mu[s].double().cpu(), before[i])
            assert (mixes[s, at:at + n].double().cpu() - want).abs().max() < _tol(dtype)
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,Hr,n", [(1, 3, 16), (37, 2, 64), (9, 1, 40), (64, 5, 8), (3, 1, 1)])
def test_unit_norm_weight_and_gate(ops, dtype, T, Hr, n):
    eps = 1e-5
    o = rnd(T, Hr * n, seed=1, scale=3.0)
    z = rnd(T, Hr * n, seed=2, scale=2.0, dtype=dtype)
    w = rnd(Hr * n, seed=3) * 0.3 + 1.0
    out = torch.empty(T, Hr * n, device=DEV, dtype=dtype)
    ops.wkv_finish(o, z, w, out, heads=Hr, eps=eps)
    zd = z.double().cpu()
    want = P.rms_unit(o.double().cpu().view(T, Hr, n), eps).reshape(T, Hr * n) * w.double().cpu() * (zd * torch.sigmoid(zd))
    assert (out.double().cpu() - want).abs().max() < _tol(dtype) * max(1.0, want.abs().max().item())


# ------------------------------------------------------------------------------------------------ the norm after the sum
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16, None])
@pytest.mark.parametrize("T,D,top,alpha", [(1, 64, 0, 1.5), (37, 352, 3, 2.0), (5, 1536, 2, 0.5), (130, 40, 1, 1.0)])
def test_norm_after_the_sum(ops, out_dtype, T, D, top, alpha):
    eps = 1e-6
    x0 = rnd(T, D, seed=1, scale=2.0)
    y = rnd(T, D, seed=2, scale=3.0)
    w = rnd(D, seed=3) * 0.3 + 1.0
    pairs = rnd(T * top, D, seed=4) if top else None
    pw = rnd(T, top, seed=5).abs() if top else None
    for with_y in (True, False):
        x = x0.clone()
        h = None if out_dtype is None else torch.empty(T, D, device=DEV, dtype=out_dtype)
        ops.post_norm(x, w, eps, alpha, y=y if with_y else None, pairs=pairs, pair_weights=pw, top=top, h=h)
        v = alpha * x0.double().cpu() + (y.double().cpu() if with_y else 0.0)
        if top:
            v = v + (pw.double().cpu()[:, :, None] * pairs.double().cpu().view(T, top, D)).sum(1)
        want = P.rms_norm(v, w.double().cpu(), eps)
        assert (x.double().cpu() - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
        if h is not None:
            assert torch.equal(h, x.to(out_dtype))


# ------------------------------------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("T", [1, 7, 16, 17, 300])
@pytest.mark.parametrize("E,top,groups,keep,D", [(6, 3, 3, 2, 64), (16, 4, 4, 2, 192), (4, 1, 1, 1, 96), (3, 3, 1, 1, 40),
                                                 (10, 3, 2, 1, 272), (64, 8, 8, 4, 128), (4, 2, 4, 2, 32), (1, 1, 1, 1, 8)])
def test_router_over_sigmoid_scores_and_group_sums(ops, T, E, top, groups, keep, D):
    for dtype in (torch.float32, torch.bfloat16):
        h = rnd(T, D, seed=T + E, dtype=dtype)
        router = rnd(E, D, seed=2, scale=3.0 / math.sqrt(D), dtype=dtype)
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(T, top, device=DEV)
        offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
        order = torch.empty(T * top, dtype=torch.int32, device=DEV)
        ops.moe_route(h, router, idx, wts, offsets, order, top=top, groups=groups, keep=keep, mode="sigmoid", group_sum=2,
                      weight_scale=1.9)
        r = dict(top=top, scale=1.9, groups=dict(count=groups, keep=keep))
        wi, ww = P.route(h.double().cpu(), router.double().cpu(), r)
        gi, gw = idx.long().cpu(), wts.double().cpu()
        flips = 0
        for t in range(T):
            if not torch.equal(gi[t], wi[t]):        # near-ties may fall either way in 32-bit
                flips += 1
                continue
            assert (gw[t] - ww[t]).abs().max() < 2e-5
            assert abs(float(gw[t].sum()) - 1.9) < 1e-5
        assert flips <= max(1, T // 50)
        off, od = offsets.cpu().tolist(), order.cpu().tolist()
        assert off[0] == 0 and off[-1] == T * top and sorted(od) == list(range(T * top))
        for e in range(E):
            seg = od[off[e]:off[e + 1]]
            assert all(int(gi.reshape(-1)[p]) == e for p in seg) and seg == sorted(seg)
    ops.check_device_errors()


def test_a_group_is_scored_by_its_two_largest_and_scores_are_not_a_softmax(ops):
    """Group 0 holds the single largest score, group 1 the two next: by largest score group 0 would win, by the sum of two
    group 1 does.  The weights are the sigmoid scores over their sum, not a softmax."""
    D, E = 8, 6
    h = torch.zeros(1, D, device=DEV)
    h[0, 0] = 1.0
    z = torch.tensor([3.0, -4.0, -5.0, 2.0, 1.5, -6.0])
    router = torch.zeros(E, D, device=DEV)
    router[:, 0] = z.to(DEV)
    idx = torch.empty(1, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(1, 2, device=DEV)
    args = (torch.empty(E + 1, dtype=torch.int32, device=DEV), torch.empty(2, dtype=torch.int32, device=DEV))
    ops.moe_route(h, router, idx, wts, *args, top=2, groups=2, keep=1, mode="sigmoid", group_sum=2, weight_scale=1.0)
    assert idx.cpu().tolist() == [[3, 4]]
    s = torch.sigmoid(z.double())
    assert abs(wts[0, 0].item() - float(s[3] / (s[3] + s[4]))) < 1e-6
    ops.moe_route(h, router, idx, wts, *args, top=2, groups=2, keep=1, mode="sigmoid", group_sum=1, weight_scale=1.0)
    assert idx.cpu().tolist() == [[0, 1]]
    pi, pw = P.route(h.double().cpu(), router.double().cpu(), dict(top=2, scale=1.0, groups=dict(count=2, keep=1)))
    assert pi.tolist() == [[3, 4]]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,D,F", [(1, 5, 2, 64, 24), (9, 12, 3, 192, 48), (40, 4, 1, 96, 16), (200, 3, 3, 96, 8),
                                         (70, 8, 2, 768, 512), (16, 8, 2, 128, 40), (33, 6, 3, 288, 80)])
def test_experts_without_gates(ops, dtype, T, E, top, D, F):
    """Route, the experts' two products with the square of relu between them, the weighted sum: against the statement
    with the router's own choice (so that a near-tie upstream does not decide the comparison)."""
    h = rnd(T, D, seed=T + F, scale=1.2, dtype=dtype)
    router = rnd(E, D, seed=2, scale=3.0 / math.sqrt(D), dtype=dtype)
    w1 = rnd(E, F, D, seed=4, scale=1.3 / math.sqrt(D), dtype=dtype)
    w2 = rnd(E, D, F, seed=5, scale=1.0 / math.sqrt(F), dtype=dtype)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(T * top, dtype=torch.int32, device=DEV)
    ops.moe_route(h, router, idx, wts, offsets, order, top=top, mode="sigmoid", weight_scale=1.3)
    mid = torch.empty(T * top, F, device=DEV, dtype=dtype)
    ops.moe_grouped(h, w1, mid, offsets, order, top=top, first=True, act="relu_sq")
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
            want[t] += float(wts[t, k]) * P.expert(hd[t:t + 1], {"up": w1[e].double().cpu(), "down": w2[e].double().cpu()}, store)[0]
    assert (out.double().cpu() - want).abs().max() < _tol(dtype) * max(1.0, want.abs().max().item())
