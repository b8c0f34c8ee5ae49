"""A plain, slow Bogetar: one function per mechanism, float64 on the CPU, written from the design's
equations and sharing no code with the engine.

``forward(config, weights, tokens)`` runs one whole sequence and returns the logits ``[T, V]`` (with
``layers_out``, a list, the residual stream after every layer is appended to it).  ``weights`` maps checkpoint names to tensors.  With ``rnd`` (a function that
rounds a tensor, ``as_bfloat16``) the places where the engine's bfloat16 path stores 16 bits are rounded too,
so that a tiny model's own sensitivity to rounding does not drown a comparison.  ``forced`` replays expert
choices (``{layer: [T, top] indices}``) after a test has checked that they are legitimate.
"""

from __future__ import annotations

import math
from typing import Callable, Dict, Optional

import torch

F64 = torch.float64


def as_bfloat16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def same(x: torch.Tensor) -> torch.Tensor:
    return x


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def group_rms_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Every row in ``groups`` equal consecutive parts, each divided by its own root mean square; then ``w``."""
    T, n = x.shape
    parts = x.reshape(T, groups, n // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(T, n) * w


def causal_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y_t = sum_j w[:, j] x_(t - taps + 1 + j)`` per channel, zeros before the sequence."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """``x [T, heads, d]``: dimension ``i < dims/2`` turns with ``i + dims/2`` by ``p * base^(-2i/dims)``."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def windowed_sigmoid_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                               rnd: Callable) -> torch.Tensor:
    """The left half of the parallel mixer: every visible key weighs in with ``sigmoid(score + pb[head])``,
    and the weights of a query are not normalised."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, G, d)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * W[p + "q.norm"]
    k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * W[p + "k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rnd(rotate_halves(q, pos, rot["dims"], rot["base"]))
    k = rnd(rotate_halves(k, pos, rot["dims"], rot["base"]))
    v = rnd(v)
    i, j = pos[:, None], pos[None, :]
    visible = (j <= i) & (i - j < m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        score = (q[:, hd] @ k[:, g].T) * m["scale"] + W[p + "pb"][hd]
        weight = torch.where(visible, sigmoid(score), torch.zeros((), dtype=h.dtype))
        out[:, hd] = weight @ v[:, g]
    gate = sigmoid(h @ W[p + "g"].T)
    return rnd(rnd(out.reshape(T, H * dv)) * gate) @ W[p + "o"].T


def gated_linear_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                           rnd: Callable) -> torch.Tensor:
    """The right half: ``S <- diag(alpha_t) S + k_t v_t^T``, ``o_t = S^T q_t`` per head."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    z = rnd(h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[p + "norm"]
    y = o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return rnd(y) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps, rnd):
    left = windowed_sigmoid_attention(h, W, p + "left.", m["left"], eps, rnd)
    right = gated_linear_attention(h, W, p + "right.", m["right"], eps, rnd)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_delta_rule(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                     rnd: Callable) -> torch.Tensor:
    """``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` per head, one decay per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].T)
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    rep = H // G
    for t in range(T):
        kt = k[t].repeat_interleave(rep, dim=0)
        qt = q[t].repeat_interleave(rep, dim=0)
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, qt)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[p + "norm"]
    y = o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return rnd(y) @ W[p + "o"].T


def route(h: torch.Tensor, w_router: torch.Tensor, r: dict):
    """Softmax over all experts; only experts of the ``keep`` groups with the largest best score can be chosen;
    the ``top`` largest scores among them, used as they are.  Returns ``(indices [T, top], scores [T, E])``."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ w_router.T, dim=-1)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    allowed = torch.ones_like(s, dtype=torch.bool)
    if keep < count:
        best = s.reshape(-1, count, E // count).max(dim=-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        mask = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        allowed = mask.repeat_interleave(E // count, dim=1)
    idx = torch.topk(torch.where(allowed, s, torch.full_like(s, -1.0)), top, dim=-1).indices
    return idx, s


def expert(h, W, p, limit, rnd):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return rnd(g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def mixture_of_experts(h, W, p, mlp, rnd, forced=None):
    r = mlp["router"]
    idx, s = route(h, W[p + "router"], r)
    if forced is not None:
        idx = forced
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(r["experts"]):
        rows = (idx == e).any(dim=-1).nonzero().flatten()
        if rows.numel():
            out[rows] += s[rows, e][:, None] * expert(h[rows], W, f"{p}e{e}.", mlp["expert"]["limit"], rnd)
    return out, idx, s


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, rnd: Optional[Callable] = None,
            forced: Optional[Dict[int, torch.Tensor]] = None, chosen: Optional[dict] = None,
            layers_out: Optional[list] = None, dtype: torch.dtype = F64) -> torch.Tensor:
    """``dtype`` float32 runs the same plain arithmetic in 32 bits: how far it lies from the float64 run says how
    much rounding alone moves a position of THIS model (tiny heads make some positions ill-conditioned)."""
    rnd = rnd or same
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = config["norm"]["eps"], config["norm"].get("groups", 1)
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = group_rms_norm(x, W[p + "norm1"], groups, eps)
        h = rnd(h + causal_conv(h, W[p + "canon1"]))
        if layer["type"] == "delta":
            y = gated_delta_rule(h, W, p + "mix.", layer["mixer"], eps, rnd)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, W, p + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + group_rms_norm(y, W[p + "norm1b"], groups, eps) * W[p + "ls1"]
        if layer.get("mlp") is not None:
            h = group_rms_norm(x, W[p + "norm2"], groups, eps)
            h = rnd(h + causal_conv(h, W[p + "canon2"]))
            y, idx, s = mixture_of_experts(h, W, p + "mlp.", layer["mlp"], rnd,
                                           None if forced is None else forced.get(i))
            if chosen is not None:
                chosen[i] = (idx, s)
            x = x + group_rms_norm(y, W[p + "norm2b"], groups, eps) * W[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    h = rnd(group_rms_norm(x, W["final.norm"], groups, eps))
    return h @ W["embed"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt, n: int):
    ids, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(config, weights, ids)[-1]))
        ids.append(tok)
        out.append(tok)
    return out
