"""A plain, slow Tofinex in PyTorch on the CPU: one function per mechanism, whole sequences at once, no
cache carried between calls.  It shares no code with the engine and is what the engine's kernels, parts and
step function are compared with.  ``dtype`` float64 gives an oracle whose own rounding is far below the
float32 engine's.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``d`` key size, ``e`` value
size.  Weights are a dict ``name -> tensor`` with the checkpoint's names; a configuration is the dictionary
of ``config.json``.

The design: the sublayers of a layer read the residual itself and only their OUTPUT is normalised,
``x <- x + m n1(mixer(x))``, ``x <- x + m n2(ff(x))``; attention with normalised, neighbour-rotated query and
key heads, capped scores, a softmax whose denominator counts one key more (score 0, no value), and values that
every layer but the first blends with the first layer's values of the same token; a dense gated feed-forward or
a mixture of experts whose sigmoid scores weigh the experts' INPUTS, beside a gated shared expert; the output
head is the embedding table, its logits capped.
"""

from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch


def same(t):
    return t


def as_bfloat16(t):
    """Round to bfloat16 and back: handed to ``forward`` as ``rnd`` it rounds where the engine's bfloat16
    path stores 16 bits (the inputs of its matrix products and the cache)."""
    return t.to(torch.bfloat16).to(t.dtype)


# --------------------------------------------------------------------------- #
# norms, activations, caps
# --------------------------------------------------------------------------- #

def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def cap(z, limit: float):
    """``limit * tanh(z / limit)``."""
    return limit * torch.tanh(z / limit)


# --------------------------------------------------------------------------- #
# rotation
# --------------------------------------------------------------------------- #

def rotate_neighbours(x, dims: int, base: float, first_position: int = 0):
    """``x [T, heads, d]``: coordinate ``2i`` of the first ``dims`` is paired with ``2i + 1`` and the pair is
    turned by ``p * base^(-2i/dims)`` at position ``p``; the other coordinates pass."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    p = torch.arange(first_position, first_position + T, dtype=torch.float64)
    a = p[:, None] * f[None, :]
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #

def sink_softmax(s: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """``p_j = exp(s_j) / (1 + sum_visible exp(s_j))`` over the last dimension."""
    s = s.masked_fill(~visible, float("-inf"))
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))


def blend_values(v: torch.Tensor, v_first: Optional[torch.Tensor], lam) -> torch.Tensor:
    """``(1 - lam) v + lam v_first`` over a token's values as one row (heads side by side); the first
    blending layer keeps its own values."""
    if v_first is None:
        return v
    return (1.0 - lam) * v + lam * v_first.reshape(v.shape)


def attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, v_first, rnd: Callable = same):
    """``h [T, W]`` -> ``(output [T, W], the values this layer attends over [T, G, e])``."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, e)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = norm_plain(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_neighbours(q, rot["dims"], rot["base"])
        k = rotate_neighbours(k, rot["dims"], rot["base"])
    if m.get("v_mix"):
        v = blend_values(v, v_first, w[p + "vmix"])
    q, k, v = rnd(q), rnd(k), rnd(v)
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    if m.get("softcap"):
        s = cap(s, m["softcap"])
    pos = torch.arange(T)
    visible = (pos[None, :] <= pos[:, None])[None]
    pr = sink_softmax(s, visible.expand(H, T, T))
    a = torch.einsum("hij,jhe->ihe", pr, vv).reshape(T, H * e)
    return rnd(a) @ w[p + "o"].T, v


# --------------------------------------------------------------------------- #
# feed-forward
# --------------------------------------------------------------------------- #

def gated_unit(h, gate, up, down, rnd: Callable = same):
    return rnd(silu(h @ gate.T) * (h @ up.T)) @ down.T


def router_choice(h, w_router, top: int):
    """Sigmoid scores, the ``top`` largest per token (lowest index on ties); the weights are the scores."""
    s = torch.sigmoid(h @ w_router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order), s


def moe(h, w: Dict[str, torch.Tensor], p: str, mlp: dict, rnd: Callable = same, forced=None):
    """The sum of ``expert(weight * h)`` over the chosen experts plus the gated shared expert.  ``forced``
    ``[T, top]`` replaces the choice (to follow another implementation's proven near-ties)."""
    top = mlp["router"]["top"]
    idx, wt, scores = router_choice(h, w[p + "router"], top)
    if forced is not None:
        idx = forced.to(torch.long)
        wt = torch.gather(scores, 1, idx)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            q = f"{p}e{e}."
            out[t] += gated_unit(rnd(wt[t, j] * h[t:t + 1]), w[q + "gate"], w[q + "up"], w[q + "down"], rnd)[0]
    if mlp.get("shared") is not None:
        q = p + "shared."
        g = torch.sigmoid(h @ w[q + "sg"].T)
        out = out + g * gated_unit(h, w[q + "gate"], w[q + "up"], w[q + "down"], rnd)
    return out, (idx, scores)


def feed_forward(h, w, p: str, mlp: dict, rnd: Callable = same, forced=None):
    if mlp["kind"] == "dense":
        return gated_unit(h, w[p + "gate"], w[p + "up"], w[p + "down"], rnd), None
    return moe(h, w, p, mlp, rnd, forced)


# --------------------------------------------------------------------------- #
# the model
# --------------------------------------------------------------------------- #

def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            rnd: Callable = same, forced: Optional[Dict[int, torch.Tensor]] = None, layers_out: Optional[list] = None,
            chosen: Optional[dict] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence.  ``layers_out`` collects the residual after every layer;
    ``chosen[layer] = (experts [T, top], scores [T, experts])`` what every routed layer chose."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = norm_plain(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y, v = attention_mixer(rnd(x), w, p + "mix.", L["mixer"], eps, v_first, rnd)
        if L["mixer"].get("v_mix") and v_first is None:
            v_first = v
        x = x + mult * norm_plain(y, w[p + "norm1"], eps)
        if L.get("mlp") is not None:
            y, rec = feed_forward(rnd(x), w, p + "mlp.", L["mlp"], rnd, None if forced is None else forced.get(i))
            if chosen is not None and rec is not None:
                chosen[i] = rec
            x = x + mult * norm_plain(y, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    z = rnd(norm_plain(x, w["final.norm"], eps)) @ w["embed"].T
    return cap(z, cfg["logit_softcap"]) if cfg.get("logit_softcap") else z


def greedy(cfg: dict, weights, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    """``n`` tokens, each the arg-max of the logits at the last position of all tokens so far."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, weights, toks, dtype)[-1])))
    return toks[len(prompt):]
