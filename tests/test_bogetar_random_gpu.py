"""Bogetar models of random shape: layer order, sizes, head counts, windows, taps, groups and constants drawn from
a seed, served in several cuttings and compared with the plain model in both precisions.  Nothing in the engine may
rest on the sizes of one model."""

import random

import pytest
import torch

import bogetar_tiny as bt
import traces
from engine_harness import run_trace
from test_bogetar_engine_gpu import TOL, reference, run_and_check, runner_for

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    r = random.Random(seed)
    groups = r.choice([1, 1, 2, 3, 4])
    width = groups * r.choice([8, 12, 16, 20, 24, 32]) if r.random() < 0.8 else groups * r.choice([7, 9, 15])
    tensor_core_sizes = r.random() < 0.3
    if tensor_core_sizes:
        width = r.choice([64, 128])
        groups = r.choice([1, 2, 4])

    def moe():
        if r.random() < 0.2:
            return None
        count = r.choice([1, 1, 2, 3, 4])
        size = r.choice([1, 2, 3, 4])
        keep = r.randint(1, count)
        top = r.randint(1, min(keep * size, 6))
        ff = r.choice([64, 128]) if tensor_core_sizes else r.choice([8, 12, 20, 33, 48])
        named = count > 1 or r.random() < 0.5
        return bt._moe(ff, count * size, top, r.choice([1.0, 2.0, 3.5, 7.0]), (count, keep) if named else None)

    def heads():
        kv = r.choice([1, 1, 2, 3])
        return kv * r.choice([1, 1, 2, 3]), kv

    layers = []
    for _ in range(r.randint(1, 4)):
        if r.random() < 0.4:
            h, kv = heads()
            layers.append(bt._delta(h, kv, r.choice([4, 8, 12, 20, 32, 70]), r.choice([4, 6, 16, 17, 40]), r.randint(1, 5), moe()))
        else:
            h, kv = heads()
            if tensor_core_sizes:
                dim, vdim = r.choice([16, 32, 64, 128]), r.choice([64, 128])
            else:
                dim, vdim = r.choice([4, 8, 12, 20, 34]), r.choice([4, 6, 16, 18, 40])
            rot = None
            if r.random() < 0.8:
                rot = {"base": r.choice([10.0, 1000.0, 20000.0, 1e6]), "dims": r.choice([d for d in range(2, dim + 1, 2)])}
            left = bt._left(h, kv, dim, vdim, r.choice([1, 2, 5, 16, 17, 31, 64, 100]), r.choice([0.1, 0.2, 0.4]) * (16 / dim) ** 0.5, rot)
            right = bt._right(r.randint(1, 4), r.choice([4, 8, 16, 24]), r.choice([4, 8, 16, 20]), r.choice([1.0, 2.0, 8.0, 16.0, 40.0]),
                              r.randint(1, 6))
            layers.append(bt._parallel(left, right, r.choice([0.3, 0.6, 1.0, 1.4]), r.choice([0.2, 0.9, 1.0]), moe()))
    return {"architecture": "Bogetar", "vocab": r.randint(40, 300), "width": width,
            "norm": {"eps": r.choice([1e-6, 1e-5]), "groups": groups}, "canon": {"taps": r.randint(1, 5)}, "layers": layers}


@pytest.mark.parametrize("seed", list(range(8)))
def test_models_of_random_shape_in_several_cuttings(seed, tmp_path):
    cfg = random_config(seed)
    w = bt.make_weights(cfg, seed=100 + seed)
    folder = bt.write_folder(str(tmp_path / "m"), cfg, w)
    reqs = bt.random_requests(cfg, [83, 2, 37], seed=seed)
    for dtype in ("float32", "bfloat16"):
        runner = runner_for(folder, dtype, max_requests=3, num_pages=60)
        for steps in (traces.whole(reqs), traces.tail_decoded(reqs, tail=20), traces.portions(reqs),
                      traces.mixed(reqs, max_live=3, seed=seed, decode_tail=9)):
            run_and_check(runner, steps, cfg, w, reqs, dtype, strict=dtype == "float32")
            assert runner.cache.used_pages() == [0] * len(runner.cache.pools)


MEDIUM = {
    "architecture": "Bogetar", "vocab": 512, "width": 256, "norm": {"eps": 1e-6, "groups": 2}, "canon": {"taps": 4},
    "layers": [
        bt._parallel(bt._left(8, 2, 64, 128, 200, 0.11, {"base": 20000.0, "dims": 32}), bt._right(4, 32, 64, 16.0, 16), 0.6, 0.9,
                     bt._moe(128, 16, 4, 2.0, (4, 3))),
        bt._delta(4, 2, 64, 64, 4, bt._moe(128, 16, 4, 2.0, (4, 3))),
        bt._parallel(bt._left(4, 4, 128, 128, 300, 0.08, {"base": 20000.0, "dims": 128}), bt._right(8, 16, 32, 8.0, 8), 0.7, 0.8,
                     bt._moe(64, 8, 2, 3.0, (2, 1))),
        bt._delta(8, 8, 32, 128, 3, None),
        bt._parallel(bt._left(6, 3, 128, 64, 64, 0.08, None), bt._right(2, 64, 64, 4.0, 4), 1.0, 1.0, bt._moe(128, 4, 1, 2.0)),
    ],
}


def test_a_model_of_middling_size_with_long_prompts(tmp_path):
    """Sizes that every tensor-core kernel of the bfloat16 path takes (the tensor-memory attention with key and value
    heads alike and not, the tensor-core expert products), prompts long enough for windows to pass, for pages to be
    given back and for linear attention to be walked in segments.  float32: every position strictly.  bfloat16: a
    head's very first read-out is a multiple of ONE vector that is then normalised, so its sign hangs on the sign of
    one dot product, and where that lies near zero 16-bit rounding may turn it: nearly all positions must agree,
    not all."""
    cfg = MEDIUM
    w = bt.make_weights(cfg, seed=5)
    folder = bt.write_folder(str(tmp_path / "m"), cfg, w)
    reqs = bt.random_requests(cfg, [700, 3, 290, 41], seed=3)
    args = dict(page_size=16, max_requests=4, num_pages=160, max_tokens_per_step=1200, max_context=1200)
    cuttings = (traces.whole(reqs), traces.tail_decoded(reqs, tail=40), traces.portions(reqs, (257, 2, 300, 7, 64, 31)),
                traces.mixed(reqs, max_live=4, seed=1, decode_tail=12))
    runner = runner_for(folder, "float32", **args)
    for steps in cuttings:
        run_and_check(runner, steps, cfg, w, reqs, "float32")
    runner = runner_for(folder, "bfloat16", **args)
    assert all(l.parts["mixer"]._logistic_tc for l in runner.model.layers if "mixer_b" in l.parts)
    assert all(l.parts["feed_forward"]._tc for l in runner.model.layers if "feed_forward" in l.parts)
    for steps in cuttings:
        routing = {}
        got = run_trace(runner, steps, routing)
        ref = {rid: reference(cfg, w, reqs[rid], routing.get(rid), "bfloat16", rid, strict=False)[0] for rid in reqs}
        bad = 0
        for (rid, pos), row in got.items():
            assert bool(torch.isfinite(row).all())
            scale = float(ref[rid].abs().max())
            bad += float((row.double() - ref[rid][pos]).abs().max()) / scale > TOL["bfloat16"]
        assert bad <= 0.03 * len(got), f"{bad} of {len(got)} positions apart"
