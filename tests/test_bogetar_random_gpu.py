"""Bogetar models of random shape: layer order, sizes, head counts, windows, taps, groups and constants drawn from
a seed, served in several cuttings and compared with the plain model in both precisions.  Nothing in the engine may
rest on the sizes of one model."""

import random

import pytest
import torch

import bogetar_tiny as bt
import traces
from test_bogetar_engine_gpu import run_and_check, runner_for

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
