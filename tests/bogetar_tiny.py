"""Tiny Bogetar configurations and weights for the tests.

The configurations differ from one another in every size and option: number and order of layers (delta first or
last, two delta layers in a row, parallel alone), layers without a feed-forward, one, two and three norm groups,
input convolutions of one to four taps, delta convolutions of other lengths than those, heads that share a
query/key head or do not, attention with one key/value head, as many as heads or fewer, other head counts and
sizes left and right, rotation of a whole head, of part of it and of none, windows of 1, 3, 9 and more, one
expert group (or none named), all groups kept, fewer kept, one expert per token and several.  Weights are drawn
so that scores, gates and decays stay away from their saturated ends (a mixer that puts out almost nothing
hides its faults) and are rounded to bfloat16, so that both precision paths and the plain model read the same
numbers.
"""

from __future__ import annotations

import math
from typing import Dict

import torch

from nipapel_tiny import random_requests, write_folder  # noqa: F401  (container writer and request maker)


def _left(heads, kv, dim, vdim, window, scale, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    return m


def _right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def _parallel(left, right, ls, rs, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def _delta(heads, kv, dim, vdim, conv, mlp):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def _moe(ff, experts, top, limit, groups=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


CONFIG_A = {
    "architecture": "Bogetar", "vocab": 101, "width": 48, "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 3},
    "layers": [
        _delta(4, 2, 12, 10, 2, _moe(24, 6, 2, 1.5, (3, 2))),
        _parallel(_left(4, 2, 16, 10, 9, 0.3, {"base": 10000.0, "dims": 8}), _right(2, 12, 20, 8.0, 5), 0.7, 1.2,
                  _moe(40, 8, 3, 3.0, (4, 2))),
        _parallel(_left(5, 1, 12, 20, 3, 0.35, {"base": 100.0, "dims": 12}), _right(3, 8, 6, 2.0, 3), 1.1, 0.4, None),
        _delta(2, 2, 8, 16, 4, None),
        _parallel(_left(2, 2, 8, 12, 40, 0.5), _right(1, 16, 16, 30.0, 7), 0.5, 0.5, _moe(16, 5, 1, 2.5)),
    ],
}

CONFIG_B = {
    "architecture": "Bogetar", "vocab": 131, "width": 72, "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 2},
    "layers": [
        _parallel(_left(6, 3, 10, 6, 17, 0.4, {"base": 50.0, "dims": 6}), _right(4, 6, 10, 4.0, 4), 1.0, 1.0,
                  _moe(56, 4, 4, 2.0, (2, 2))),
        _parallel(_left(1, 1, 18, 30, 1, 0.3, {"base": 30.0, "dims": 18}), _right(6, 4, 4, 16.0, 2), 0.9, 0.3,
                  _moe(32, 9, 2, 1.0, (3, 1))),
        _delta(6, 1, 10, 6, 3, _moe(20, 12, 5, 4.0, (6, 3))),
        _delta(3, 3, 20, 7, 1, _moe(8, 2, 1, 2.0, (2, 1))),
    ],
}

# shapes that the bfloat16 path takes to the tensor cores (value size 64 or 128 with a key size that is a multiple
# of 16 in the attention; expert and model widths that the tensor-core grouped product takes)
CONFIG_C = {
    "architecture": "Bogetar", "vocab": 160, "width": 64, "norm": {"eps": 1e-6, "groups": 2}, "canon": {"taps": 4},
    "layers": [
        _parallel(_left(4, 2, 32, 64, 21, 0.2, {"base": 10000.0, "dims": 16}), _right(2, 16, 32, 16.0, 8), 0.6, 0.9,
                  _moe(64, 8, 2, 2.0, (4, 3))),
        _delta(2, 1, 32, 32, 4, _moe(128, 4, 1, 2.0, (2, 1))),
        _parallel(_left(2, 1, 48, 128, 70, 0.15, {"base": 10000.0, "dims": 48}), _right(4, 8, 16, 4.0, 16), 0.8, 0.8,
                  _moe(64, 4, 2, 3.0)),
        _parallel(_left(10, 2, 16, 64, 5, 0.3, {"base": 1000.0, "dims": 8}), _right(1, 64, 64, 8.0, 4), 1.3, 0.2, None),
    ],
}

# one of everything that a model may happen to make equal or one
CONFIG_D = {
    "architecture": "Bogetar", "vocab": 64, "width": 40, "norm": {"eps": 3e-6}, "canon": {"taps": 1},
    "layers": [
        _parallel(_left(1, 1, 8, 8, 2, 0.4, {"base": 10.0, "dims": 8}), _right(1, 8, 8, 1.0, 1), 1.0, 1.0,
                  _moe(16, 1, 1, 2.0, (1, 1))),
        _delta(1, 1, 8, 8, 1, _moe(8, 3, 3, 1.5)),
    ],
}

# key and value heads of 64 and 128 numbers, alike and not: prompt portions in bfloat16 take the tensor-memory
# attention, single tokens the split kernel
CONFIG_E = {
    "architecture": "Bogetar", "vocab": 192, "width": 128, "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 2},
    "layers": [
        _parallel(_left(6, 3, 64, 128, 50, 0.11, {"base": 10000.0, "dims": 32}), _right(2, 16, 16, 4.0, 8), 0.9, 0.6,
                  _moe(64, 6, 2, 2.0, (3, 2))),
        _delta(4, 2, 16, 32, 3, _moe(64, 4, 1, 1.5)),
        _parallel(_left(2, 1, 128, 64, 200, 0.08, {"base": 5000.0, "dims": 128}), _right(4, 8, 8, 2.0, 4), 0.7, 1.1,
                  _moe(128, 4, 2, 3.0, (2, 1))),
        _parallel(_left(3, 3, 128, 128, 17, 0.08), _right(1, 32, 32, 32.0, 2), 1.0, 0.5, None),
    ],
}

# delta layers only: a model that keeps no paged cache at all, only states
CONFIG_F = {
    "architecture": "Bogetar", "vocab": 77, "width": 36, "norm": {"eps": 1e-6, "groups": 2}, "canon": {"taps": 4},
    "layers": [
        _delta(3, 1, 12, 8, 2, _moe(20, 4, 2, 2.0, (2, 1))),
        _delta(2, 2, 10, 14, 3, None),
    ],
}

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E, "F": CONFIG_F}


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """``name -> bfloat16 tensor`` for every tensor the configuration implies (names built here from the
    configuration alone, so the engine's own manifest is checked against an independent one)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    taps = cfg["canon"]["taps"]

    def rnd(*shape, std=1.0):
        return torch.randn(*shape, generator=g) * std

    def lin(out, inn, gain=1.0):
        return rnd(out, inn, std=gain / math.sqrt(inn))

    def norm(n):
        return 1.0 + rnd(n, std=0.2)

    w: Dict[str, torch.Tensor] = {"embed": rnd(cfg["vocab"], W, std=0.6), "final.norm": norm(W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = norm(W), norm(W)
        w[p + "ls1"] = 0.8 + rnd(W, std=0.2)
        w[p + "canon1"] = rnd(W, taps, std=0.4)
        if L["type"] == "delta":
            q = p + "mix."
            H, G, d, e, c = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(G * d, W, 2.0), lin(G * d, W, 2.0), lin(H * e, W, 2.0)
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * e)):
                w[q + n + ".conv"] = rnd(rows, c, std=0.6)
            w[q + "b"], w[q + "a"] = lin(H, W, 2.0), lin(H, W, 2.0)
            w[q + "A_log"], w[q + "dt_bias"] = rnd(H, std=0.5) - 1.0, rnd(H, std=1.0)
            w[q + "norm"] = norm(e)
            w[q + "g"], w[q + "o"] = lin(H * e, W, 2.0), lin(W, H * e, 1.5)
        else:
            q, a = p + "mix.left.", m["left"]
            H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * d, W), lin(G * d, W), lin(G * e, W, 1.5)
            w[q + "q.norm"], w[q + "k.norm"] = 1.5 + rnd(d, std=0.3), 1.5 + rnd(d, std=0.3)
            w[q + "pb"] = rnd(H, std=1.0) - 1.0
            w[q + "g"], w[q + "o"] = lin(H * e, W, 2.0), lin(W, H * e, 1.0)
            q, r = p + "mix.right.", m["right"]
            H, d, e, rank = r["heads"], r["dim"], r["vdim"], r["decay_rank"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * d, W, 2.0), lin(H * d, W), lin(H * e, W, 1.5)
            w[q + "g"], w[q + "o"] = lin(H * e, W, 2.0), lin(W, H * e, 1.5)
            w[q + "norm"] = norm(e)
            w[q + "a1"], w[q + "a2"] = lin(rank, W), lin(H * d, rank, 2.0)
            w[q + "a2.b"] = rnd(H * d, std=1.0) + 1.0
        mlp = L.get("mlp")
        if mlp is None:
            continue
        w[p + "norm2"], w[p + "norm2b"] = norm(W), norm(W)
        w[p + "ls2"] = 0.8 + rnd(W, std=0.2)
        w[p + "canon2"] = rnd(W, taps, std=0.4)
        q = p + "mlp."
        ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
        w[q + "router"] = lin(E, W, 2.0)
        for x in range(E):
            w[f"{q}e{x}.gate"], w[f"{q}e{x}.up"], w[f"{q}e{x}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff, 1.5)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}
