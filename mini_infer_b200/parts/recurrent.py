"""Mixers that keep a fixed-size state per request instead of a cache that grows with the context.

``channel_gated_delta``: the delta rule with a write strength per head and a decay per head and key channel.
With ``q``, ``k`` unit vectors per head (``q`` also times ``dim^-1/2``), ``beta = sigmoid(W_b h)`` and
``g = exp(-exp(A_log) * softplus(W_a2 W_a1 h + dt_bias))`` laid out heads x dim::

    S <- diag(g) S ;   u = beta (v - S^T k) ;   S <- S + k u^T ;   o = S^T q

and the output is ``rmsnorm_per_head(o) * norm * sigmoid(W_g2 W_g1 h)`` through ``W_o``.  ``q``, ``k`` and ``v``
pass a short causal convolution and silu first.

``gated_delta``: the same rule with ONE decay per head, ``g = exp(-exp(A_log) * softplus(W_a h + dt_bias))``, full
projections for the decay and the gate, and the gate after the norm as ``silu(W_g h)``.

``gated_linear_attention``: ``S <- diag(alpha) S + k v^T``, ``o = S^T q`` per head with ``q = W_q h * dim^-1/2``,
``k`` and ``v`` as projected and a decay per key channel ``alpha = sigmoid(W_a2 W_a1 h + b)^(1 / tau)``; the
output is ``rmsnorm_per_head(o) * norm * silu(W_g h)`` through ``W_o``.

``residual_short_conv``: ``x + conv(x)`` with a causal convolution over time per channel and no activation; its
state is the last ``taps - 1`` rows it read.

``mamba2``: the state-space recurrence ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x`` with
``dt = softplus(dt + dt_bias)``, ``x``, ``B``, ``C`` behind one causal convolution with bias and silu,
``y * silu(z)`` normalised in groups, through ``W_o``.

Both keep ``S`` and the last ``taps - 1`` inputs of their convolutions in one float32 row per request
(:class:`StateNeed`), are computed in float32 beyond the projections, and walk a request's tokens in order
whatever the cut of the step.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..ops import functional as F
from .base import CacheBinding, Mixer, Runtime, StateNeed, StepContext, TensorDecl, linear
from .tuning import TUNING


def _f32(t: torch.Tensor, dev) -> torch.Tensor:
    return t.to(device=dev, dtype=torch.float32).contiguous()


class ChannelGatedDelta(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads`` (heads of q and k), ``head_dim`` (q, k),
    ``value_dim``, ``conv`` (taps), ``decay_rank``, ``gate_rank``, ``eps`` (of the output norm).

    Tensors below the prefix: ``q``, ``k`` ``[kv_heads*head_dim, hidden]``, ``v [heads*value_dim, hidden]``,
    each with ``.conv [channels, taps]``; ``b [heads, hidden]``; ``a1 [decay_rank, hidden]``,
    ``a2 [heads*head_dim, decay_rank]``, ``dt_bias [heads*head_dim]``, ``A_log [heads]``;
    ``g1 [gate_rank, hidden]``, ``g2 [heads*value_dim, gate_rank]``; ``norm [value_dim]``;
    ``o [hidden, heads*value_dim]``."""

    graph_safe = True
    kernel_files = ("recurrent.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.dv = int(p["value_dim"])
        self.taps = int(p["conv"])
        self.ra = int(p["decay_rank"])
        self.rg = int(p["gate_rank"])
        self.eps = float(p["eps"])
        if self.nkv < 1 or self.nh % self.nkv:
            raise ValueError(f"delta rule: {self.nh} heads are not a multiple of {self.nkv} key heads")
        if not 1 <= self.taps <= F.CONV_MAX_TAPS:
            raise ValueError(f"delta rule: a convolution of {self.taps} taps (at most {F.CONV_MAX_TAPS})")
        self.n_qk = self.nkv * self.d
        self.n_v = self.nh * self.dv
        self.channels = 2 * self.n_qk + self.n_v
        self.state_floats = self.nh * self.d * self.dv
        self.conv_floats = (self.taps - 1) * self.channels

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        return [TensorDecl(p + "q", (self.n_qk, self.H)), TensorDecl(p + "q.conv", (self.n_qk, self.taps), "conv"),
                TensorDecl(p + "k", (self.n_qk, self.H)), TensorDecl(p + "k.conv", (self.n_qk, self.taps), "conv"),
                TensorDecl(p + "v", (self.n_v, self.H)), TensorDecl(p + "v.conv", (self.n_v, self.taps), "conv"),
                TensorDecl(p + "b", (self.nh, self.H)), TensorDecl(p + "A_log", (self.nh,), "bias"),
                TensorDecl(p + "norm", (self.dv,), "norm"),
                TensorDecl(p + "a1", (self.ra, self.H)), TensorDecl(p + "a2", (self.nh * self.d, self.ra), "low_rank"),
                TensorDecl(p + "dt_bias", (self.nh * self.d,), "bias"),
                TensorDecl(p + "g1", (self.rg, self.H)), TensorDecl(p + "g2", (self.n_v, self.rg), "low_rank"),
                TensorDecl(p + "o", (self.H, self.n_v))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        self.w_in = torch.cat([m(tensors[p + n], dev) for n in ("q", "k", "v", "b")], dim=0)
        self.w_low = torch.cat([m(tensors[p + "a1"], dev), m(tensors[p + "g1"], dev)], dim=0)
        # both second projections as one product: [a2 0; 0 g2] on [a1 h ; g1 h]
        w_up = torch.zeros(self.nh * self.d + self.n_v, self.ra + self.rg, dtype=rt.act, device=dev)
        w_up[:self.nh * self.d, :self.ra] = m(tensors[p + "a2"], dev)
        w_up[self.nh * self.d:, self.ra:] = m(tensors[p + "g2"], dev)
        self.w_up = w_up
        self.w_conv = torch.cat([_f32(tensors[p + n + ".conv"], dev) for n in ("q", "k", "v")], dim=0)
        self.a_log = _f32(tensors[p + "A_log"], dev)
        self.dt_bias = _f32(tensors[p + "dt_bias"], dev)
        self.norm_w = _f32(tensors[p + "norm"], dev)
        self.w_o = m(tensors[p + "o"], dev)

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        F.l2_prefetch(self.w_in)

    def cache_need(self):
        return StateNeed((self.state_floats + self.conv_floats,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        state = ctx.states[cache.group]
        proj = linear(x, self.w_in, torch.float32)                       # q | k | v | beta
        low = linear(x, self.w_low, self.rt.act)
        up = linear(low, self.w_up, torch.float32)                       # decay input | gate input
        qkv = F.causal_conv_silu(proj, 0, self.channels, self.w_conv, None, state, self.state_floats,
                                 ctx.q_start, ctx.req_of_token, ctx.state_slot)
        o = F.delta_scan(qkv, proj, self.channels, up, 0, self.a_log, self.dt_bias, state, 0, ctx.q_start,
                         ctx.state_slot, self.nh, self.nkv, self.d, self.dv, self.d ** -0.5)
        y = F.gated_group_rmsnorm(o, up, self.nh * self.d, self.norm_w, self.nh, False, self.eps, self.rt.act)
        return linear(y, self.w_o, torch.float32)


class Mamba2(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim``, ``state_size``, ``groups`` (of B and C),
    ``norm_groups``, ``conv`` (taps), ``eps``.

    Tensors below the prefix: ``in [2*inner + 2*groups*state + heads, hidden]`` (rows z | x | B | C | dt),
    ``conv [inner + 2*groups*state, taps]``, ``conv.b``, ``dt_bias``, ``A_log``, ``D`` ``[heads]``,
    ``norm [inner]``, ``o [hidden, inner]``; ``inner = heads * head_dim``."""

    graph_safe = True
    kernel_files = ("recurrent.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.P = int(p["head_dim"])
        self.N = int(p["state_size"])
        self.G = int(p.get("groups", 1))
        self.norm_groups = int(p.get("norm_groups", 1))
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        self.inner = self.nh * self.P
        if self.G < 1 or self.nh % self.G:
            raise ValueError(f"mamba2: {self.nh} heads are not a multiple of {self.G} groups")
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} channels do not split into {self.norm_groups} norm groups")
        if not 1 <= self.taps <= F.CONV_MAX_TAPS:
            raise ValueError(f"mamba2: a convolution of {self.taps} taps (at most {F.CONV_MAX_TAPS})")
        self.channels = self.inner + 2 * self.G * self.N
        self.state_floats = self.nh * self.N * self.P
        self.conv_floats = (self.taps - 1) * self.channels

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        return [TensorDecl(p + "in", (2 * self.inner + 2 * self.G * self.N + self.nh, self.H)),
                TensorDecl(p + "conv", (self.channels, self.taps), "conv"),
                TensorDecl(p + "conv.b", (self.channels,), "bias"),
                TensorDecl(p + "dt_bias", (self.nh,), "bias"), TensorDecl(p + "A_log", (self.nh,), "bias"),
                TensorDecl(p + "D", (self.nh,), "norm"), TensorDecl(p + "norm", (self.inner,), "norm"),
                TensorDecl(p + "o", (self.H, self.inner))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        self.w_in = m(tensors[p + "in"], dev)
        self.w_conv = _f32(tensors[p + "conv"], dev)
        self.b_conv = _f32(tensors[p + "conv.b"], dev)
        self.dt_bias = _f32(tensors[p + "dt_bias"], dev)
        self.a_log = _f32(tensors[p + "A_log"], dev)
        self.d_skip = _f32(tensors[p + "D"], dev)
        self.norm_w = _f32(tensors[p + "norm"], dev)
        self.w_o = m(tensors[p + "o"], dev)

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        F.l2_prefetch(self.w_in)

    def cache_need(self):
        return StateNeed((self.state_floats + self.conv_floats,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        state = ctx.states[cache.group]
        proj = linear(x, self.w_in, torch.float32)                       # z | x | B | C | dt
        xbc = F.causal_conv_silu(proj, self.inner, self.channels, self.w_conv, self.b_conv, state,
                                 self.state_floats, ctx.q_start, ctx.req_of_token, ctx.state_slot)
        y = F.ssd_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d_skip, state, 0,
                       ctx.q_start, ctx.state_slot, self.nh, self.G, self.N, self.P)
        y = F.gated_group_rmsnorm(y, proj, 0, self.norm_w, self.norm_groups, True, self.eps, self.rt.act)
        return linear(y, self.w_o, torch.float32)


class GatedDelta(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads`` (heads of q and k; head ``h`` uses q/k head
    ``h // (heads / kv_heads)``), ``head_dim`` (q, k), ``value_dim``, ``conv`` (taps), ``eps`` (of the output
    norm).

    Tensors below the prefix: ``q``, ``k`` ``[kv_heads*head_dim, hidden]``, ``v [heads*value_dim, hidden]``,
    each with ``.conv [channels, taps]``; ``b``, ``a`` ``[heads, hidden]``; ``dt_bias``, ``A_log`` ``[heads]``;
    ``g [heads*value_dim, hidden]``; ``norm [value_dim]``; ``o [hidden, heads*value_dim]``."""

    graph_safe = True
    kernel_files = ("recurrent.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.dv = int(p["value_dim"])
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        if self.nkv < 1 or self.nh % self.nkv:
            raise ValueError(f"delta rule: {self.nh} heads are not a multiple of {self.nkv} key heads")
        if not 1 <= self.taps <= F.CONV_MAX_TAPS:
            raise ValueError(f"delta rule: a convolution of {self.taps} taps (at most {F.CONV_MAX_TAPS})")
        self.n_qk = self.nkv * self.d
        self.n_v = self.nh * self.dv
        self.channels = 2 * self.n_qk + self.n_v
        self.state_floats = self.nh * self.d * self.dv
        self.conv_floats = (self.taps - 1) * self.channels

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        return [TensorDecl(p + "q", (self.n_qk, self.H)), TensorDecl(p + "q.conv", (self.n_qk, self.taps), "conv"),
                TensorDecl(p + "k", (self.n_qk, self.H)), TensorDecl(p + "k.conv", (self.n_qk, self.taps), "conv"),
                TensorDecl(p + "v", (self.n_v, self.H)), TensorDecl(p + "v.conv", (self.n_v, self.taps), "conv"),
                TensorDecl(p + "b", (self.nh, self.H)), TensorDecl(p + "A_log", (self.nh,), "bias"),
                TensorDecl(p + "norm", (self.dv,), "norm"),
                TensorDecl(p + "a", (self.nh, self.H)), TensorDecl(p + "dt_bias", (self.nh,), "bias"),
                TensorDecl(p + "g", (self.n_v, self.H)), TensorDecl(p + "o", (self.H, self.n_v))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        # one product for everything that reads the layer's input: q | k | v | gate | beta | decay
        self.w_in = torch.cat([m(tensors[p + n], dev) for n in ("q", "k", "v", "g", "b", "a")], dim=0)
        self.col_gate = self.channels
        self.col_beta = self.channels + self.n_v
        self.col_decay = self.col_beta + self.nh
        self.w_conv = torch.cat([_f32(tensors[p + n + ".conv"], dev) for n in ("q", "k", "v")], dim=0)
        self.a_log = _f32(tensors[p + "A_log"], dev)
        self.dt_bias = _f32(tensors[p + "dt_bias"], dev)
        self.norm_w = _f32(tensors[p + "norm"], dev)
        self.w_o = m(tensors[p + "o"], dev)

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        F.l2_prefetch(self.w_in)

    def cache_need(self):
        return StateNeed((self.state_floats + max(self.conv_floats, 1),), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        state = ctx.states[cache.group]
        proj = linear(x, self.w_in, torch.float32)
        qkv = F.causal_conv_silu(proj, 0, self.channels, self.w_conv, None, state, self.state_floats,
                                 ctx.q_start, ctx.req_of_token, ctx.state_slot)
        o = F.delta_scan(qkv, proj, self.col_beta, proj, self.col_decay, self.a_log, self.dt_bias, state, 0,
                         ctx.q_start, ctx.state_slot, self.nh, self.nkv, self.d, self.dv, self.d ** -0.5,
                         form="head_decay")
        y = F.gated_group_rmsnorm(o, proj, self.col_gate, self.norm_w, self.nh, False, self.eps, self.rt.act,
                                  silu_after=True)
        return linear(y, self.w_o, torch.float32)


class GatedLinearAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (q, k), ``value_dim``, ``tau`` (the decay is
    ``sigmoid(.)^(1 / tau)``), ``decay_rank`` (rows of ``a1``), ``eps`` (of the output norm).

    Tensors below the prefix: ``q``, ``k`` ``[heads*head_dim, hidden]``, ``v``, ``g`` ``[heads*value_dim,
    hidden]``, ``a1 [decay_rank, hidden]``, ``a2 [heads*head_dim, decay_rank]``, ``a2.b [heads*head_dim]``,
    ``norm [value_dim]``, ``o [hidden, heads*value_dim]``."""

    graph_safe = True
    kernel_files = ("recurrent.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.d = int(p["head_dim"])
        self.dv = int(p["value_dim"])
        self.tau = float(p["tau"])
        self.ra = int(p["decay_rank"])
        self.eps = float(p["eps"])
        if not self.tau > 0:
            raise ValueError(f"gated linear attention: tau = {self.tau} must be positive")
        self.n_qk = self.nh * self.d
        self.n_v = self.nh * self.dv

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        return [TensorDecl(p + "q", (self.n_qk, self.H)), TensorDecl(p + "k", (self.n_qk, self.H)),
                TensorDecl(p + "v", (self.n_v, self.H)), TensorDecl(p + "g", (self.n_v, self.H)),
                TensorDecl(p + "o", (self.H, self.n_v)), TensorDecl(p + "norm", (self.dv,), "norm"),
                TensorDecl(p + "a1", (self.ra, self.H)), TensorDecl(p + "a2", (self.n_qk, self.ra), "low_rank"),
                TensorDecl(p + "a2.b", (self.n_qk,), "bias")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        self.w_in = torch.cat([m(tensors[p + n], dev) for n in ("q", "k", "v", "g")], dim=0)
        self.w_a1 = m(tensors[p + "a1"], dev)
        self.w_a2 = m(tensors[p + "a2"], dev)
        self.b_a2 = _f32(tensors[p + "a2.b"], dev)
        self.norm_w = _f32(tensors[p + "norm"], dev)
        self.w_o = m(tensors[p + "o"], dev)

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        F.l2_prefetch(self.w_in)

    def cache_need(self):
        return StateNeed((self.nh * self.d * self.dv,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        state = ctx.states[cache.group]
        proj = linear(x, self.w_in, torch.float32)                       # q | k | v | gate
        z = linear(linear(x, self.w_a1, self.rt.act), self.w_a2, torch.float32)
        # long portions of the bfloat16 path are walked in segments side by side; the float32 path keeps one walk for
        # every step, so that its sums run in one order however a prompt was cut
        segs, per = (1, 0) if self.rt.act != torch.bfloat16 else F.scan_segments(
            ctx.max_q_len, TUNING.scan_segments_min_tokens, TUNING.scan_segment_tokens, TUNING.scan_max_segments)
        o = F.delta_scan(proj, None, 0, z, 0, None, self.b_a2, state, 0, ctx.q_start, ctx.state_slot, self.nh,
                         self.nh, self.d, self.dv, self.d ** -0.5, form="sigmoid_decay", tau=self.tau,
                         segments=segs, segment_tokens=per)
        y = F.gated_group_rmsnorm(o, proj, 2 * self.n_qk + self.n_v, self.norm_w, self.nh, False, self.eps,
                                  self.rt.act, silu_after=True)
        return linear(y, self.w_o, torch.float32)


class ResidualShortConv(Mixer):
    """``x + conv(x)``: a causal convolution over time on each channel, ``conv(x)_t = sum_j w[:, j] x_(t - taps +
    1 + j)``, zeros before a request's start, no bias and no activation.  It reads float32 rows and writes the
    activation type; the last ``taps - 1`` rows it read are the request's state.
    params: ``channels``, ``taps``, optional ``tensor`` (default ``weight``).  Tensor: ``<prefix><tensor>
    [channels, taps]``."""

    graph_safe = True
    kernel_files = ("recurrent.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.C = int(self.params["channels"])
        self.taps = int(self.params["taps"])
        if not 1 <= self.taps <= F.CONV_MAX_TAPS:
            raise ValueError(f"short convolution: {self.taps} taps (at most {F.CONV_MAX_TAPS})")

    def _name(self) -> str:
        return self.prefix + self.params.get("tensor", "weight")

    def tensor_decls(self) -> List[TensorDecl]:
        return [TensorDecl(self._name(), (self.C, self.taps), "conv")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.w = _f32(tensors[self._name()], rt.device)

    def cache_need(self):
        return StateNeed((max((self.taps - 1) * self.C, 1),), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        return F.causal_conv_residual(x, self.w, ctx.states[cache.group], 0, ctx.q_start, ctx.req_of_token,
                                      ctx.state_slot, self.rt.act)

    def forward_from_residual(self, hidden: torch.Tensor, norm, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        """``forward(norm(hidden))``.  A decode step of the bfloat16 path (one token per request) runs the norm in
        groups, the convolution and the state's update in one launch; the float32 path keeps one kernel per
        mechanism for every step, so that its sums run in one order however a prompt was cut."""
        groups = getattr(norm, "group_parameters", None)
        if groups is not None and ctx.all_decode and self.rt.act == torch.bfloat16:
            weight, eps, n = groups()
            return F.norm_conv_decode(hidden, weight, n, eps, self.w, ctx.states[cache.group], 0, ctx.q_start,
                                      ctx.state_slot, self.rt.act)
        return self.forward(norm.apply_float(hidden), ctx, cache)


register_part("mixer", "channel_gated_delta", ChannelGatedDelta)
register_part("mixer", "gated_delta", GatedDelta)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "residual_short_conv", ResidualShortConv)
register_part("mixer", "mamba2", Mamba2)
