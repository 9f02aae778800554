"""Kusirax through the engine (ModelRunner, the cache manager, the scheduler, LLM.generate, bin/trace_run) against the
plain float64 statement in tests/plain_kusirax.py, on small models made here with weights that make faults show."""
import os

import numpy as np
import pytest
import torch

import plain_kusirax as P
from helpers import Replay, random_ids, write_model
from kusirax_models import CONFIGS, PAGE, attn, attn2, clean, config, dense, layer, make_tensors, moe, wkv

pytestmark = pytest.mark.gpu


def oracle(tensors, cfg, ids, dtype):
    return P.forward(tensors, clean(cfg), ids, store=P.to_bf16 if dtype == "bfloat16" else P._keep).numpy()


def close(got, want, dtype, what):
    """float32, row by row: relative error at most 4e-5 (a norm after every sum carries each sublayer's rounding forward,
    and the experts' outputs partly cancel in their weighted sum).  bfloat16: a router may send a token whose candidate
    experts score alike to the other one when a bfloat16 rounding upstream falls the other way; that token then differs
    by as much as two experts differ, and through the cache and the recurrent state so do some after it: the median row
    within 1e-2 and all but three in a hundred within 3e-2.  (The float32 runs hold every row; the kernels that only
    bfloat16 steps use are held row by row in tests/test_kusirax_kernels_gpu.py.)"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    err = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-12)
    if dtype == "float32":
        assert err.max() <= 4e-5, f"{what}: row {err.argmax()}: relative error {err.max():.3e}"
        return
    assert np.median(err) <= 1e-2 and (err <= 3e-2).mean() >= 0.97, \
        f"{what}: {np.sort(err)[-5:]} median {np.median(err):.3e}, {(err <= 3e-2).mean():.2f} within 3e-2"


def runner_for(folder, which, dtype, pages=160, seqs=4, graphs=False):
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=PAGE[which], num_pages=pages, max_num_seqs=seqs,
                                            use_cuda_graphs=graphs))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in CONFIGS:
        tensors = make_tensors(CONFIGS[which], seed=3)
        folder = write_model(str(tmp_path_factory.mktemp("kusirax_" + which)), clean(CONFIGS[which]), tensors, torch.bfloat16)
        out[which] = (folder, tensors)
    return out


def test_layers_one_by_one_in_float32(models):
    """The residual after every layer against the oracle's."""
    from mini_llm_b200 import ops
    from mini_llm_b200.engine.runner import StepEntry
    for which in CONFIGS:
        folder, tensors = models[which]
        cfg = CONFIGS[which]
        ids = random_ids(75, cfg["vocab"], 5)
        res = []
        P.forward(tensors, clean(cfg), ids, trace=res)
        r = runner_for(folder, which, "float32")
        r.add_request("a")
        ctx = r.prepare_step([StepEntry("a", ids, [0])])
        m = r.model
        assert len(m.spec.schedule) == len(res) == len(cfg["layers"])
        with ops.stream_scope():
            x = m.embedding.forward(ctx, m.positions)
            for i, (entry, cache) in enumerate(zip(m.spec.schedule, m._caches)):
                lay = m.layers[entry.layer]
                x = lay.arrangement(lay, x, ctx, cache)
                assert (x.double().cpu() - res[i]).abs().max() < 3e-5 * res[i].abs().max(), (which, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
def test_whole_prompts_then_token_by_token(models, which, dtype):
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    n = 330                                    # many blocks of every layer's mask, past a split of 256 keys
    ids = random_ids(n, cfg["vocab"], 7)
    want = oracle(tensors, cfg, ids, dtype)
    r = runner_for(folder, which, dtype)
    r.add_request("w")
    got = r.step([StepEntry("w", ids, list(range(n)))]).cpu().numpy()
    close(got, want, dtype, "whole")
    r.finish_request("w")
    # most of it in one step, the rest one by one: long decoding over the edges of blocks of 24, 100 and 7, with the state
    # carried from token to token, through pages and a state row that the request before has just given back
    r.add_request("d")
    head = n - 120
    rows = [r.step([StepEntry("d", ids[:head], [0, 1, 2, head - 1])]).cpu().numpy()]
    for t in range(head, n):
        rows.append(r.step([StepEntry("d", [ids[t]], [0])]).cpu().numpy())
    close(np.concatenate(rows), want[[0, 1, 2, head - 1] + list(range(head, n))], dtype, "decode")
    r.finish_request("d")
    # from the very first token on, one by one: a single key, a state that is still zero, no row before the first
    r.add_request("f")
    rows = [r.step([StepEntry("f", [ids[t]], [0])]).cpu().numpy() for t in range(40)]
    close(np.concatenate(rows), want[:40], dtype, "first tokens")
    r.finish_request("f")
    r.cache.check()
    assert r.cache.num_live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
def test_portions_of_many_sizes(models, which, dtype):
    """Cuts of one and two tokens, mid-page, mid-block, exactly at a block's edge and one token to either side, and at
    the edges of the recurrence's chunks of 16 tokens."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    n = 290
    ids = random_ids(n, cfg["vocab"], 11)
    want = oracle(tensors, cfg, ids, dtype)
    r = runner_for(folder, which, dtype)
    for cuts in ([2, 2, 3, 64, 1, 31, 2, 17, 33, 2, 1, 1, 2, 129], [24, 13, 27, 36, 99, 1, 90], [7] * 41 + [3],
                 [23, 2, 12, 26, 37, 28, 100, 62], [16, 16, 15, 17, 32, 1, 193]):
        assert sum(cuts) == n
        r.add_request("p")
        rows, at = [], 0
        for c in cuts:
            rows.append(r.step([StepEntry("p", ids[at:at + c], list(range(c)))]).cpu().numpy())
            at += c
        close(np.concatenate(rows), want, dtype, f"portions {cuts[:4]}")
        r.finish_request("p")
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
@pytest.mark.parametrize("graphs", [False, True])
def test_unequal_requests_batched_with_pages_used_again(models, which, dtype, graphs):
    """Five requests through three places and a pool that cannot hold them all at once: portions beside single tokens,
    requests that sit a step out, pages given back (also by the mask, while a request runs) and state rows taken by the
    next request.  Every row equals the request run alone (the oracle)."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    lens = {"a": 90, "b": 13, "c": 121, "d": 2, "e": 64}
    ids = {k: random_ids(n, cfg["vocab"], 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: oracle(tensors, cfg, v, dtype) for k, v in ids.items()}
    plan = {"a": [30, 2, 1, 1, 40, 1, 1, 14], "b": [2, 1, 1, 9], "c": [64, 1, 0, 50, 2, 1, 1, 1, 1], "d": [2],
            "e": [1, 1, 1, 1, 1, 59]}
    ps = PAGE[which]
    r = runner_for(folder, which, dtype, pages=(90 + 16 + 121 + 64) // ps + 6, seqs=3, graphs=graphs)
    waiting, live, at, got = ["a", "b", "c", "d", "e"], [], {k: 0 for k in lens}, {k: [] for k in lens}
    while waiting or live:
        while waiting and len(live) < 3:
            k = waiting.pop(0)
            r.add_request(k)
            live.append(k)
        entries = []
        for k in live:
            c = plan[k].pop(0)
            if c:
                entries.append(StepEntry(k, ids[k][at[k]:at[k] + c], list(range(c))))
        out = r.step(entries).cpu().numpy()
        o = 0
        for e in entries:
            c = len(e.tokens)
            got[e.req].append(out[o:o + c])
            o += c
            at[e.req] += c
        for k in list(live):
            if not plan[k]:
                r.finish_request(k)
                live.remove(k)
        r.cache.check()
    for k in lens:
        close(np.concatenate(got[k]), want[k], dtype, f"request {k}")
    assert r.cache.num_live == 0
    assert all(g.allocator.num_in_use == 0 for g in r.cache.groups)


def test_a_request_alone_and_in_a_batch(models):
    """What else is in the step changes nothing beyond rounding (a product of more rows may take another kernel)."""
    from mini_llm_b200.engine.runner import StepEntry
    for which in CONFIGS:
        folder, _ = models[which]
        cfg = CONFIGS[which]
        a, b, c = (random_ids(n, cfg["vocab"], 70 + n) for n in (37, 9, 64))
        r = runner_for(folder, which, "float32")
        r.add_request("a")
        alone = [r.step([StepEntry("a", a[:30], [29])]).clone()]
        alone += [r.step([StepEntry("a", [t], [0])]).clone() for t in a[30:]]
        r.finish_request("a")
        for k in "abc":
            r.add_request(k)
        r.step([StepEntry("c", c[:5], []), StepEntry("b", b[:3], [])])
        both = [r.step([StepEntry("b", b[3:], []), StepEntry("a", a[:30], [29]), StepEntry("c", c[5:40], [0])])[:1].clone()]
        for i, t in enumerate(a[30:]):
            both.append(r.step([StepEntry("c", [c[40 + i]], [0]), StepEntry("a", [t], [0])])[1:2].clone())
        a1, a2 = torch.cat(alone).double(), torch.cat(both).double()
        assert ((a1 - a2).norm(dim=1) / a1.norm(dim=1)).max() < 2e-5, which


def test_a_state_row_that_is_used_again_starts_from_zero(models):
    """One place, three requests one after the other: the second and third find the state and the kept row of the one
    before in their slot and must not see them."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models["B"]
    cfg = CONFIGS["B"]
    r = runner_for(folder, "B", "float32", seqs=1)
    for i, n in enumerate((50, 21, 34)):
        ids = random_ids(n, cfg["vocab"], 90 + i)
        r.add_request(i)
        got = [r.step([StepEntry(i, ids[:n - 5], list(range(n - 5)))]).cpu().numpy()]
        got += [r.step([StepEntry(i, [t], [0])]).cpu().numpy() for t in ids[n - 5:]]
        close(np.concatenate(got), oracle(tensors, cfg, ids, "float32"), "float32", f"request {i} in the only slot")
        r.finish_request(i)


def test_pages_of_finished_blocks_go_back_while_a_request_runs():
    """Blocks of 64 positions over pages of 8: once a request has passed a block's edge the pages of the block before
    return to the pool, so a pool far smaller than the sequence carries it, and the rows stay right."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    cfg = config(48, 61, 1e-5, 1.5, [layer(attn2(2, 1, 16, 16, 0.8, 64, 6.0, v_mix=True), dense(32)),
                                     layer(wkv(2, 8, 4), None),
                                     layer(attn2(4, 2, 8, 8, 0.9, 64, 3.0, v_mix=True), None)])
    tensors = make_tensors(cfg, 8)
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        folder = write_model(d, clean(cfg), tensors, torch.bfloat16)
        n = 400
        ids = random_ids(n, cfg["vocab"], 2)
        want = oracle(tensors, cfg, ids, "float32")
        r = ModelRunner(folder, EngineConfig(dtype="float32", page_size=8, num_pages=22, max_num_seqs=1, use_cuda_graphs=False))
        r.add_request("a")
        rows, at = [], 0
        for c in [50, 30, 47, 1, 1, 1, 70] + [1] * 200:
            rows.append(r.step([StepEntry("a", ids[at:at + c], list(range(c)))]).cpu().numpy())
            at += c
            assert all(g.allocator.num_in_use <= 18 for g in r.cache.groups)
        assert at == n
        close(np.concatenate(rows), want, "float32", "a pool smaller than the sequence")
        r.finish_request("a")
        r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    """LLM.generate (scheduler, prompt portions under a small token budget, several requests decoding together, places
    used again) gives the oracle's greedy tokens; where the oracle's two best logits are closer than the comparison
    rule allows, either token is taken and the oracle follows the engine."""
    from mini_llm_b200 import LLM, SamplingParams
    folder, tensors = models["A"]
    cfg = CONFIGS["A"]
    prompts = [random_ids(n, cfg["vocab"], 40 + n) for n in (33, 5, 70, 1, 18)]
    new = 12
    llm = LLM(folder, dtype=dtype, page_size=8, num_pages=60, max_num_seqs=3, max_num_batched_tokens=48, prefill_chunk=32)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    margin = 1e-3 if dtype == "float32" else 0.25
    for p, out in zip(prompts, outs):
        assert len(out) == new
        seq = list(p)
        for tok in out:
            logits = oracle(tensors, cfg, seq, dtype)[-1]
            best = int(np.argmax(logits))
            assert tok == best or logits[best] - logits[tok] < margin, (len(p), len(seq))
            seq.append(tok)
    assert llm.runner.cache.num_live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_with_graphs(models, dtype, tmp_path):
    """bin/trace_run on a Kusirax folder: config.json picks the model class; steps that come back are replayed as CUDA
    graphs."""
    folder, tensors = models["B"]
    cfg = CONFIGS["B"]
    ids = {k: random_ids(n, cfg["vocab"], 60 + i) for i, (k, n) in enumerate({"p": 70, "q": 45}.items())}
    want = {k: oracle(tensors, cfg, v, dtype) for k, v in ids.items()}
    os.makedirs(tmp_path / "out")
    rp = Replay(folder, dtype, str(tmp_path / "out"), 192, page_size=PAGE["B"])
    got = {k: [] for k in ids}
    at = {k: 0 for k in ids}
    plan = [[("p", 40), ("q", 30)]] + [[("p", 1), ("q", 1)]] * 15 + [[("p", 15)]]
    for step in plan:
        entries = [(k, ids[k][at[k]:at[k] + c], list(range(c))) for k, c in step]
        end = [k for k, c in step if at[k] + c == len(ids[k])]
        out = rp.step(entries, end)
        o = 0
        for k, c in step:
            got[k].append(out[o:o + c])
            o += c
            at[k] += c
    assert rp.close() == 0
    assert rp.stats["graph_replays"] >= 13
    for k in ids:
        close(np.concatenate(got[k]), want[k], dtype, f"replayed request {k}")


def test_long_contexts_with_a_key_far_back(tmp_path):
    """1,500 tokens: a rotary layer that sees everything (keys a thousand positions back, several splits of keys, the
    scaled frequencies far into their slow range), blocks of 1,024 and 700 positions, a recurrence whose slowest channels
    still carry the first tokens; whole, then in portions and single tokens, at rows on both sides of every block's edge."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    cfg = config(72, 131, 1e-5, 2.0, [
        layer(attn(4, 2, 16, 16, 0.8, (8, 10000.0), scaling=(6.0, 1.0, 4.0, 256), v_mix=True), dense(48)),
        layer(attn2(3, 1, 24, 32, 0.7, 700, 10.0, v_mix=True), moe(4, 2, 16, 1.5, groups=(2, 2))),
        layer(wkv(2, 32, 6), None),
        layer(attn2(2, 2, 32, 16, 0.6, 1024, None, v_mix=True), None)])
    tensors = make_tensors(cfg, 11)
    folder = write_model(str(tmp_path / "long"), clean(cfg), tensors, torch.bfloat16)
    n = 1500
    ids = random_ids(n, cfg["vocab"], 1)
    rows = [0, 1, 255, 256, 257, 511, 512, 699, 700, 701, 1023, 1024, 1025, 1279, 1280, 1399, 1400, 1401, 1499]
    for dtype in ("float32", "bfloat16"):
        want = oracle(tensors, cfg, ids, dtype)
        r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, num_pages=200, max_num_seqs=2))
        r.add_request("w")
        close(r.step([StepEntry("w", ids, rows)]).cpu().numpy(), want[rows], dtype, "whole")
        r.finish_request("w")
        r.add_request("p")
        got, at = [], 0
        cuts = [690, 9, 2, 322, 2, 255, 200] + [1] * 20
        for c in cuts:
            got.append(r.step([StepEntry("p", ids[at:at + c], [c - 1])]).cpu().numpy()[0])
            at += c
        close(np.stack(got), want[np.cumsum(cuts) - 1], dtype, "portions and single tokens")
        assert r.graph_replays >= 15


def test_sizes_that_happen_to_be_one_or_equal(tmp_path):
    """One head, one expert chosen out of one, one group, blocks of one position, every entry of a head turning, values
    as wide as keys, a decay of rank one, a factor of one (and below one) on the residual, a model of recurrences only and
    one of attention only: nothing rests on two sizes being different or larger than 1."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    a = config(40, 53, 1e-5, 1.0, [layer(attn2(1, 1, 8, 8, 1.0, 1, 1.0, v_mix=True), moe(1, 1, 8, 1.0, groups=(1, 1))),
                                   layer(attn(2, 2, 8, 4, 0.9, (8, 10.0), v_mix=True), moe(2, 2, 16, 3.0, groups=(2, 2))),
                                   layer(attn2(2, 1, 8, 8, 0.5, 2, None), None)])
    b = config(32, 40, 1e-6, 0.75, [layer(wkv(1, 1, 1), dense(32)), layer(wkv(4, 8, 8), None), layer(wkv(1, 32, 1), moe(4, 2, 8, 0.5, groups=(4, 2)))])
    for name, cfg in (("a", a), ("b", b)):
        tensors = make_tensors(cfg, 4)
        folder = write_model(str(tmp_path / name), clean(cfg), tensors, torch.bfloat16)
        ids = random_ids(80, cfg["vocab"], 9)
        want = oracle(tensors, cfg, ids, "float32")
        r = ModelRunner(folder, EngineConfig(dtype="float32", page_size=8, num_pages=40, max_num_seqs=2, use_cuda_graphs=False))
        r.add_request("a")
        rows = [r.step([StepEntry("a", ids[:33], list(range(33)))]).cpu().numpy()]
        for t in range(33, 80):
            rows.append(r.step([StepEntry("a", [ids[t]], [0])]).cpu().numpy())
        close(np.concatenate(rows), want, "float32", name)
        r2 = ModelRunner(folder, EngineConfig(dtype="bfloat16", page_size=8, num_pages=40, max_num_seqs=2, use_cuda_graphs=False))
        r2.add_request("a")
        out = r2.step([StepEntry("a", ids, list(range(80)))]).cpu().numpy()
        assert np.isfinite(out).all()


def test_odd_sizes(tmp_path):
    """A width, head sizes, value sizes, inner sizes and a vocabulary that are no multiples of 8 (rows that start on no
    16-byte boundary), a recurrence of 33 entries per head with a decay of rank 70 (two tiles of its weights), three query
    heads per key/value head: every product and kernel takes them, in both dtypes."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    cfg = config(50, 77, 1e-5, 1.5, [layer(wkv(2, 33, 70), moe(5, 2, 10, 1.2)),
                                     layer(attn(3, 1, 6, 5, 0.9, (4, 50.0), v_mix=True), dense(30)),
                                     layer(attn2(3, 1, 10, 5, 0.8, 9, 4.0, v_mix=True), moe(6, 2, 7, 0.9, groups=(3, 1))),
                                     layer(wkv(3, 5, 1), dense(13))])
    tensors = make_tensors(cfg, 6)
    folder = write_model(str(tmp_path / "odd"), clean(cfg), tensors, torch.bfloat16)
    ids = random_ids(150, cfg["vocab"], 3)
    for dtype in ("float32", "bfloat16"):
        want = oracle(tensors, cfg, ids, dtype)
        r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=2, use_cuda_graphs=False))
        r.add_request("a")
        rows = [r.step([StepEntry("a", ids[:97], list(range(97)))]).cpu().numpy()]
        rows.append(r.step([StepEntry("a", ids[97:120], list(range(23)))]).cpu().numpy())
        for t in range(120, 150):
            rows.append(r.step([StepEntry("a", [ids[t]], [0])]).cpu().numpy())
        close(np.concatenate(rows), want, dtype, "odd sizes")


def test_command_line_with_random_weights(tmp_path):
    """bin/mini_llm: the random-weights mode writes a Kusirax folder from a config.json (the decay's rank given there);
    greedy tokens from the command line equal LLM.generate's."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    from mini_llm_b200 import LLM, SamplingParams
    cfg = clean(CONFIGS["A"])
    for l, src in zip(cfg["layers"], CONFIGS["A"]["layers"]):
        if "_rank" in src:
            l["mixer"]["decay_rank"] = src["_rank"]
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(cfg))
    out_dir = tmp_path / "written"
    cli = [sys.executable, os.path.join(ROOT, "bin", "mini_llm")]
    prompts = ["5 17 3 90 9 60 4", "40 2 2 31"]
    tail = ["--dtype", "float32", "--max-new-tokens", "6", "--ignore-eos", "--max-batch-num", "2"]
    for p in prompts:
        tail += ["--prompt-ids", p]
    r = subprocess.run(cli + ["--random-config", str(cfg_path), "--seed", "7", "--write-model", str(out_dir)] + tail,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and os.path.isfile(out_dir / "model.safetensors"), r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.endswith("[DONE]")]
    got = [[int(t) for t in l.replace("[DONE]", "").split()] for l in lines]
    llm = LLM(str(out_dir), dtype="float32", max_num_seqs=2)
    want = llm.generate([[int(t) for t in p.split()] for p in prompts], SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert got == want


def test_sizes_no_kernel_takes_are_refused_at_construction(tmp_path):
    from mini_llm_b200.config.base import ConfigError, EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner
    cfg = config(32, 50, 1e-5, 1.0, [layer(wkv(1, 264, 2), None)])
    folder = write_model(str(tmp_path / "bad"), clean(cfg), make_tensors(cfg, 0))
    with pytest.raises(ConfigError, match="wkv"):
        ModelRunner(folder, EngineConfig(dtype="float32", num_pages=4))
