"""Tiny Tofinex configurations and weights for the tests.

The configurations differ from one another in every size and option: number and order of layers, layers without
a feed-forward, dense and routed feed-forwards, one expert per token, several and all of them, with and without
a shared expert, key and value sizes that differ, one head, as many key heads as heads or fewer, rotation of all
of a head, of part of it or of none, capped and uncapped scores and logits, a residual multiplier of one and
others, value blending in all layers, in some (the first blending layer not being the first layer) and in none.
Weights are drawn so that scores and activations stay of order one (a model whose mixers put out almost nothing
hides their faults) and are rounded to bfloat16, so that both precision paths and the plain model read the same
numbers.
"""

from __future__ import annotations

import math
from typing import Dict

import torch

from nipapel_tiny import random_requests, write_folder  # noqa: F401  (container writer and request maker)


def _attn(heads, kv, dim, vdim, scale=None, cap=None, rot=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if cap is not None:
        m["softcap"] = cap
    if rot is not None:
        m["rot"] = rot
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


CONFIG_A = {
    "architecture": "Tofinex", "vocab": 101, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "logit_softcap": 12.0,
    "layers": [
        _layer(_attn(4, 2, 16, 10, 0.3, 6.0, {"base": 10000.0, "dims": 8}, v_mix=False), _dense(80)),
        _layer(_attn(5, 1, 12, 20, 0.35, 4.0, {"base": 100.0, "dims": 12}, v_mix=True), _moe(40, 5, 2, shared=24)),
        _layer(_attn(2, 2, 8, 10, 0.5, 9.0, {"base": 500.0, "dims": 2}, v_mix=True), None),
        _layer(_attn(2, 1, 20, 20, 0.2, 5.0, {"base": 77.0, "dims": 20}, v_mix=True), _moe(24, 3, 1)),
    ],
}

CONFIG_B = {
    "architecture": "Tofinex", "vocab": 131, "width": 72, "norm": {"eps": 1e-6}, "residual_mult": 1.5,
    "layers": [
        _layer(_attn(6, 1, 24, 40, 0.25, None, {"base": 50.0, "dims": 6}), _moe(56, 4, 4, shared=32)),
        _layer(_attn(3, 3, 10, 6, 0.4, 3.0), _dense(96)),
        _layer(_attn(1, 1, 18, 30, 0.3, 20.0, {"base": 30.0, "dims": 18}), _moe(32, 6, 3, shared=8)),
        _layer(_attn(8, 4, 6, 4, 0.6, 2.0, {"base": 1e6, "dims": 4}), None),
        _layer(_attn(4, 2, 14, 14, 0.3, 8.0, {"base": 200.0, "dims": 14}), _moe(16, 9, 2)),
    ],
}

# shapes that the bfloat16 path takes to the tensor cores (value size 64 or 128, key size a multiple of 16, once
# with more heads than one block finishes; expert and model widths that the tensor-core grouped product takes)
CONFIG_C = {
    "architecture": "Tofinex", "vocab": 160, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
    "logit_softcap": 25.0,
    "layers": [
        _layer(_attn(4, 2, 32, 64, 0.2, 10.0, {"base": 10000.0, "dims": 16}, v_mix=True), _moe(64, 4, 2, shared=64)),
        _layer(_attn(2, 2, 16, 64, 0.3, 7.0, {"base": 10000.0, "dims": 16}, v_mix=True), _dense(128)),
        _layer(_attn(36, 2, 16, 64, 0.3, 5.0, {"base": 1000.0, "dims": 8}, v_mix=True), _moe(64, 8, 3)),
        _layer(_attn(2, 1, 48, 128, 0.15, 30.0, {"base": 10000.0, "dims": 48}, v_mix=True), _moe(128, 2, 1, shared=64)),
    ],
}

# one of everything that a model may happen to make equal or one
CONFIG_D = {
    "architecture": "Tofinex", "vocab": 64, "width": 40, "norm": {"eps": 3e-6}, "residual_mult": 1.0,
    "logit_softcap": 3.0,
    "layers": [
        _layer(_attn(1, 1, 8, 8, 0.4, 1.0, {"base": 10.0, "dims": 8}, v_mix=True), _moe(16, 1, 1, shared=16)),
        _layer(_attn(4, 4, 6, 2, 0.3, 2.5, {"base": 1000.0, "dims": 4}, v_mix=True), _dense(48)),
    ],
}

# key and value heads of one size that the tensor-memory attention takes for prompt portions in bfloat16 (64 and
# 128), beside single tokens on the split kernel
CONFIG_E = {
    "architecture": "Tofinex", "vocab": 192, "width": 128, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
    "logit_softcap": 30.0,
    "layers": [
        _layer(_attn(4, 2, 64, 64, 0.125, 30.0, {"base": 10000.0, "dims": 64}, v_mix=True), _dense(256)),
        _layer(_attn(2, 1, 128, 128, 0.09, 4.0, {"base": 5000.0, "dims": 64}, v_mix=False), _moe(64, 8, 2, shared=128)),
        _layer(_attn(8, 2, 64, 64, 0.2, None, {"base": 300.0, "dims": 32}, v_mix=True), _moe(128, 4, 1, shared=64)),
    ],
}

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E}


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """``name -> bfloat16 tensor`` for every tensor the configuration implies (names built here from the
    configuration alone, so the engine's own manifest is checked against an independent one)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def rnd(*shape, std=1.0):
        return torch.randn(*shape, generator=g) * std

    def lin(out, inn, gain=1.0):
        return rnd(out, inn, std=gain / math.sqrt(inn))

    w: Dict[str, torch.Tensor] = {"embed": rnd(cfg["vocab"], W, std=0.35), "embed.norm": 1.0 + rnd(W, std=0.2),
                                  "final.norm": 1.0 + rnd(W, std=0.2)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = 1.0 + rnd(W, std=0.2)
        q = p + "mix."
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * d, W), lin(G * d, W), lin(G * e, W, 1.5)
        w[q + "q.norm"], w[q + "k.norm"] = 1.5 + rnd(d, std=0.3), 1.5 + rnd(d, std=0.3)
        w[q + "o"] = lin(W, H * e, 1.5)
        if m.get("v_mix"):
            w[q + "vmix"] = 0.2 + 0.6 * torch.rand((), generator=g)
        mlp = L.get("mlp")
        q = p + "mlp."
        if mlp is None:
            continue
        w[p + "norm2"] = 1.0 + rnd(W, std=0.2)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            w[q + "gate"], w[q + "up"], w[q + "down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
        else:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            w[q + "router"] = lin(E, W, 2.0)
            for x in range(E):
                w[f"{q}e{x}.gate"], w[f"{q}e{x}.up"], w[f"{q}e{x}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff, 1.5)
            if mlp.get("shared") is not None:
                sf = mlp["shared"]["ff"]
                w[q + "shared.gate"], w[q + "shared.up"] = lin(sf, W, 2.0), lin(sf, W, 2.0)
                w[q + "shared.down"], w[q + "shared.sg"] = lin(W, sf, 1.5), lin(1, W, 2.0)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}
