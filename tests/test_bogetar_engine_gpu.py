"""Bogetar through the engine's own step function, cache and state manager, scheduler and entry points, against
the plain model: whole prompts, decoding token by token, portions down to two tokens, unequal requests in one
batch, pages and slots used again, long decoding past every window, greedy generation.

A routed layer's choice is discontinuous: where two group scores or the last chosen and the first left-out
expert score of a token lie closer than the engine's rounding, either choice is right.  The engine's choices are
recorded, checked to be legitimate against the plain model's scores, and the plain model is run with the same
choices."""

import json
import os
import subprocess
import sys

import pytest
import torch

import bogetar_tiny as bt
import plain_bogetar as pb
import traces
from engine_harness import run_trace

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: 4e-5 of the largest logit, plus eight times what rounding alone does to the plain model at that position
# (a head of a few numbers whose output nearly cancels before its norm is ill-conditioned whoever computes it)
TOL = {"float32": 4e-5, "bfloat16": 3e-2}
SLACK = 8.0
GAP = {"float32": 2e-5, "bfloat16": 0.03}         # how far below the last chosen score a chosen one may lie
ROUNDING = {"float32": pb.same, "bfloat16": pb.as_bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in bt.CONFIGS.items():
        w = bt.make_weights(cfg, seed=23 + ord(name))
        folder = bt.write_folder(str(tmp_path_factory.mktemp("bg_" + name)), cfg, w)
        out[name] = (folder, cfg, w)
    return out


def runner_for(folder, dtype, **kw):
    from mini_infer_b200.engine.loading import load_model
    from mini_infer_b200.engine.step import ModelRunner
    model, rt, _ = load_model(folder, dtype, "cuda:0")
    args = dict(page_size=8, num_pages=40, max_requests=4, max_tokens_per_step=256, max_context=352)
    args.update(kw)
    return ModelRunner(model, rt, **args)


def legitimate(idx, s, router, gap, what):
    """Every chosen expert lies in a group that is (within ``gap``) among the kept ones, and is (within ``gap``)
    among the best of the experts of the groups that were used."""
    E, top = router["experts"], router["top"]
    g = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = g["count"], g["keep"]
    size = E // count
    best = s.reshape(-1, count, size).max(dim=-1).values
    last_kept = torch.sort(best, dim=1, descending=True).values[:, keep - 1]
    for t, row in enumerate(idx.tolist()):
        assert len(set(row)) == top, f"{what}: an expert chosen twice"
        used = sorted({e // size for e in row})
        assert len(used) <= keep, f"{what}: experts of {len(used)} groups where {keep} are kept"
        for gi in used:
            assert float(last_kept[t] - best[t, gi]) <= gap, f"{what}: a group that should not be kept"
        # the groups that the engine kept: those it used, filled up with the best of the others
        order = [int(x) for x in torch.argsort(best[t], descending=True)]
        kept = used + [x for x in order if x not in used][:keep - len(used)]
        pool = torch.cat([s[t, x * size:(x + 1) * size] for x in kept])
        kth = torch.sort(pool, descending=True).values[top - 1]
        assert float(kth - s[t, row].min()) <= gap, f"{what}: an expert below the last one it should choose"


def reference(cfg, w, toks, routing, dtype, what="", strict=True):
    """Plain logits under the engine's routing, after checking that every choice is a legitimate one.  Without
    ``strict`` (models of random shape in bfloat16, where a tiny router may sit on a knife's edge for many tokens)
    the choices are taken as they are, and a position is allowed what 16-bit rounding alone does to the plain model
    there."""
    forced = None
    if routing:
        forced = {li: torch.tensor([per[p] for p in range(len(toks))], dtype=torch.long) for li, per in routing.items()}
    rec = {}
    out = pb.forward(cfg, w, toks, rnd=ROUNDING[dtype], chosen=rec, forced=forced)
    if strict:
        for li, (idx, s) in rec.items():
            legitimate(idx, s, cfg["layers"][li]["mlp"]["router"], GAP[dtype], f"{what} layer {li}")
    moved = None
    chosen = {li: idx for li, (idx, _) in rec.items()}
    if dtype == "float32":
        low = pb.forward(cfg, w, toks, forced=chosen, dtype=torch.float32).double()
        moved = (low - out).abs().max(dim=1).values
    elif not strict:
        exact = pb.forward(cfg, w, toks, forced=chosen)
        moved = (exact - out).abs().max(dim=1).values * 0.5
    return out, moved


def check(got, ref, tol):
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        want, moved = ref[rid]
        scale = float(want.abs().max())
        err = float((row.double() - want[pos]).abs().max()) / scale
        worst = max(worst, err)
        allowed = tol + (SLACK * float(moved[pos]) / scale if moved is not None else 0.0)
        assert err <= allowed, f"request {rid} position {pos}: {err:.2e} of the largest logit (first failing place)"
    return worst


_references = {}


def run_and_check(runner, steps, cfg, w, reqs, dtype, strict=True):
    routing = {}
    got = run_trace(runner, steps, routing)
    ref = {}
    for rid in reqs:
        if any(k[0] == rid for k in got):
            # the plain model is slow: one run per (model, request, routing)
            key = (id(w), dtype, strict, tuple(reqs[rid]), json.dumps(routing.get(rid), sort_keys=True))
            if key not in _references:
                _references[key] = reference(cfg, w, reqs[rid], routing.get(rid), dtype, rid, strict)
            ref[rid] = _references[key]
    check(got, ref, TOL[dtype])
    return got, routing


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_against_the_plain_model(models, name, dtype):
    folder, cfg, w = models[name]
    runner = runner_for(folder, dtype, max_requests=6, num_pages=60)
    reqs = bt.random_requests(cfg, [70, 1, 23, 2, 41, 9], seed=ord(name))
    results, routings = [], []
    for steps in (traces.whole(reqs), traces.tail_decoded(reqs, tail=36), traces.portions(reqs),
                  traces.portions(reqs, (2,)), traces.mixed(reqs, max_live=3, seed=2, decode_tail=14),
                  traces.decoded_together({r: t for r, t in reqs.items() if len(t) > 1},
                                          {"r0": 30, "r2": 12, "r3": 1, "r4": 40, "r5": 3})):
        got, routing = run_and_check(runner, steps, cfg, w, reqs, dtype)
        results.append(got)
        routings.append(routing)
        assert runner.cache.used_pages() == [0] * len(runner.cache.pools)
    if name in "CE" and dtype == "bfloat16":
        assert all(l.parts["mixer"]._tensor_cores for l in runner.model.layers if "mixer_b" in l.parts)
    if name == "E" and dtype == "bfloat16":
        # prompt portions took the tensor-memory attention
        assert all(l.parts["mixer"]._logistic_tc for l in runner.model.layers if "mixer_b" in l.parts)
    if dtype == "float32":
        # the 32-bit path gives the same bits however the work was cut and batched
        for other, routing in zip(results[1:5], routings[1:5]):
            assert routing == routings[0]
            for key, row in other.items():
                assert torch.equal(row, results[0][key]), key


def test_layer_by_layer(models):
    """The residual stream after every layer."""
    from mini_infer_b200.engine.step import StepEntry
    for name in ("A", "B", "D"):
        folder, cfg, w = models[name]
        runner = runner_for(folder, "float32")
        toks = bt.random_requests(cfg, [29], 3)["r0"]
        want, low = [], []
        pb.forward(cfg, w, toks, layers_out=want)
        pb.forward(cfg, w, toks, layers_out=low, dtype=torch.float32)
        seen = {}
        runner.model.layer_observer = lambda pos, hidden: seen.__setitem__(pos, hidden.cpu().double())
        runner.add_request("a")
        runner.step([StepEntry("a", toks, [])])
        runner.release("a")
        runner.model.layer_observer = None
        assert len(seen) == len(want)
        for n in range(len(want)):
            moved = float((low[n].double() - want[n]).abs().max())
            assert float((seen[n] - want[n]).abs().max()) <= 3e-5 * float(want[n].abs().max()) + SLACK * moved, (name, n)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_slots_and_pages_used_again(models, dtype):
    """Four requests decode 150 tokens each through replayed decode passes, past every window, while a fifth and
    sixth wait for a slot; the pool holds fewer pages than all six requests together would need, so the pages and
    state slots of the first four serve the last two (whose states must start from zero)."""
    folder, cfg, w = models["A" if dtype == "float32" else "C"]
    runner = runner_for(folder, dtype, num_pages=100, max_requests=4, max_context=200)
    reqs = bt.random_requests(cfg, [160, 170, 158, 165, 175, 181], seed=9)
    first, second = dict(list(reqs.items())[:4]), dict(list(reqs.items())[4:])
    for part in (first, second):
        run_and_check(runner, traces.decoded_together(part, 150), cfg, w, part, dtype)
    assert runner.graph_replays > 100
    assert runner.cache.used_pages() == [0] * len(runner.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_longer_prompts_after_a_captured_decode_pass(models, dtype):
    """A request of one token captures the decode pass; then prompts arrive that are each longer than any step
    before, and every one's last tokens replay that pass: what a part keeps from step to step (the two mixers'
    weights as vectors, say) must not move under a captured pass when a longer step makes it grow."""
    folder, cfg, w = models["B" if dtype == "float32" else "C"]
    runner = runner_for(folder, dtype, page_size=16, num_pages=90, max_requests=4, max_tokens_per_step=1300,
                        max_context=1300)
    reqs = bt.random_requests(cfg, [1, 40, 300, 38, 1200, 36], seed=12)
    for rid, toks in reqs.items():
        steps = traces.tail_decoded({rid: toks}, tail=6) if len(toks) > 6 else traces.whole({rid: toks})
        run_and_check(runner, steps, cfg, w, {rid: toks}, dtype)
    assert runner.graph_replays >= 30


def test_a_slot_and_its_pages_serve_one_request_after_another(models):
    folder, cfg, w = models["B"]
    runner = runner_for(folder, "float32", max_requests=1, num_pages=12)
    reqs = bt.random_requests(cfg, [33, 20, 27], seed=1)
    for rid, toks in reqs.items():
        run_and_check(runner, traces.portions({rid: toks}, (5, 2, 11)), cfg, w, {rid: toks}, "float32")


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(models, name):
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = models[name]
    prompts, wants = [], []
    seed = 0
    while len(prompts) < 4:
        seed += 1
        p = bt.random_requests(cfg, [3 + 7 * len(prompts)], seed)["r0"]
        gen = pb.greedy(cfg, w, p, 10)
        rec = {}
        logits = pb.forward(cfg, w, p + gen, chosen=rec)[len(p) - 1:-1]
        top2 = torch.topk(logits, 2, dim=-1).values
        gaps = []
        for li, (idx, s) in rec.items():
            r = cfg["layers"][li]["mlp"]["router"]
            g = r.get("groups") or {"count": 1, "keep": 1}
            srt = torch.sort(s, dim=1, descending=True).values
            gaps.append(float(srt.diff(dim=1).abs().min()))        # no two scores of a token close to each other
            best = torch.sort(s.reshape(s.shape[0], g["count"], -1).max(dim=-1).values, dim=1).values
            if g["count"] > 1:
                gaps.append(float(best.diff(dim=1).abs().min()))
        # no near-tie that rounding could turn, among the tokens, the experts or the groups
        if float((top2[:, 0] - top2[:, 1]).min()) > 1e-3 and min(gaps, default=1.0) > 1e-5:
            prompts.append(p)
            wants.append(gen)
    llm = LLM(folder, dtype="float32", max_seq_len=96, max_running=3, max_tokens_per_step=16, prefill_chunk=8,
              page_size=8)
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=10))
    assert [o.token_ids for o in outs] == wants
    assert any(s.prefill_tokens and s.decode_tokens for s in llm.last_history)      # portions beside decodes
    assert llm.runner.cache.used_pages() == [0] * len(llm.runner.cache.pools)
    llm16 = LLM(folder, dtype="bfloat16", max_seq_len=96, max_running=3, max_tokens_per_step=16, page_size=8)
    outs16 = llm16.generate(prompts[:2], SamplingParams(greedy=True, max_new_tokens=4))
    assert all(len(o.token_ids) == 4 for o in outs16)


def test_trace_runner_and_command_line(models, tmp_path):
    folder, cfg, w = models["D"]
    toks = bt.random_requests(cfg, [19], 2)["r0"]
    ref = pb.forward(cfg, w, toks)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": toks[:12], "want": [0, 11]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": toks[12:], "want": [6]}], "end": ["a"]})]
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out, "--max-tokens", "64"], input="\n".join(lines) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    import numpy as np
    a = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, -1).copy())
    b = torch.from_numpy(np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(1, -1).copy())
    scale = float(ref.abs().max())
    assert float((a.double() - ref[[0, 11]]).abs().max()) <= 4e-5 * scale
    assert float((b.double() - ref[[18]]).abs().max()) <= 4e-5 * scale
    # greedy generation on the command line
    seed = 0
    while True:
        seed += 1
        p = bt.random_requests(cfg, [6], seed)["r0"]
        gen = pb.greedy(cfg, w, p, 6)
        top2 = torch.topk(pb.forward(cfg, w, p + gen)[len(p) - 1:-1], 2, dim=-1).values
        if float((top2[:, 0] - top2[:, 1]).min()) > 1e-3:
            break
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "generate", "--model", folder, "--prompt-ids",
           ",".join(map(str, p)), "--max-new-tokens", "6", "--greedy", "--dtype", "float32", "--max-seq-len", "64", "--json"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.splitlines()
    assert json.loads(lines[lines.index("--- end ---") + 2])["token_ids"] == gen


def test_random_weights_of_a_configuration_are_served(tmp_path):
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(bt.CONFIG_A, f)
    out = str(tmp_path / "made")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "random-weights", "--config", cfg_path,
                        "--seed", "5", "--out", out], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    runner = runner_for(out, "bfloat16")
    from mini_infer_b200.engine.step import StepEntry
    runner.add_request("a")
    res = runner.step([StepEntry("a", [1, 2, 3], [2])])
    assert res.logits.shape == (1, bt.CONFIG_A["vocab"]) and bool(torch.isfinite(res.logits).all())
