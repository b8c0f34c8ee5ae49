"""Block arrangement, embedding and output head.

``prenorm_residual``: ``a = x + Mixer(Norm1(x))``; ``y = a + FFN(Norm2(a))``
(src/model/transformer_model.h:25-28, src/model/transformer_model.cpp:578-641).
The residual stream ``hidden`` is float32 in both precision paths.  A part's
output is not added at once: it travels as ``pending`` to the next norm, whose
kernel adds it while it reads the row anyway.  A feed-forward may even leave its last
step (the weighted sum of its experts' rows) to that kernel: ``pending`` is then a
``Deferred``.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import part_class, register_part
from ..ops import functional as F
from .tuning import TUNING
from .base import (Block, BuiltLayer, CacheBinding, Embedding, LMHead, RoundedResidual, Runtime, StepContext,
                   TensorDecl, TensorSum, WeightedRowSum, apply_norm, linear, resolve, split_sum)


class PreNormResidual(Block):
    graph_safe = True
    accepts_deferred = True
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, layer: BuiltLayer, hidden: torch.Tensor, pending, ctx: StepContext, caches):
        x = apply_norm(layer.mixer_norm, hidden, pending)
        y = layer.mixer.forward(x, ctx, caches.get("mixer"))
        return layer.feed_forward.forward_from_residual(hidden, y, layer.feed_forward_norm, ctx)

    def prefetch_layer(self, layer: BuiltLayer, ctx: StepContext, caches) -> None:
        layer.mixer.prefetch_first(ctx, caches.get("mixer"))


class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``hidden_size``, optional ``tensor`` (the tensor's name below the prefix,
    default ``weight``) and ``norm`` (a ``PartSpec`` of category ``norm`` whose ``rms_parameters()`` are
    applied to every gathered row before it becomes the residual stream, which stays float32).
    Tensor: ``<prefix>weight [V, H]``; no scaling (src/model/transformer_model.cpp:561-565)."""

    graph_safe = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.norm = None
        spec = self.params.get("norm")
        if spec is not None:
            self.norm = part_class("norm", spec.kind)(spec.params, prefix)

    def _name(self) -> str:
        return self.prefix + self.params.get("tensor", "weight")

    def tensor_decls(self) -> List[TensorDecl]:
        out = [TensorDecl(self._name(), (self.params["vocab_size"], self.params["hidden_size"]))]
        if self.norm is not None:
            out += self.norm.tensor_decls()
        return out

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = rt.precision.matrix(tensors[self._name()], rt.device)
        if self.norm is not None:
            self.norm.load(tensors, rt)
            if self.norm.rms_parameters() is None:
                raise ValueError("token_embedding: the norm of the embedding must be a plain RMS norm")

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        hidden = F.embed_gather(token_ids, self.weight)
        if self.norm is None:
            return hidden
        weight, eps = self.norm.rms_parameters()
        return F.add_rmsnorm(hidden, None, weight, eps, torch.float32)


class LinearHead(LMHead):
    """params: ``vocab_size``, ``hidden_size``, ``tied_to`` (name of the embedding tensor, or
    None), optional ``tensor`` (the tensor's name below the prefix, default ``weight``) and ``softcap``
    (the logits become ``softcap * tanh(logits / softcap)``; 0 or absent: as they are).  Tensor:
    ``<prefix>weight [V, H]`` unless tied (src/model/transformer_model.cpp:355-361;
    the reference deep-copies the tied matrix, here it is the same storage)."""

    graph_safe = True

    def _name(self) -> str:
        return self.prefix + self.params.get("tensor", "weight")

    def tensor_decls(self) -> List[TensorDecl]:
        if self.params.get("tied_to"):
            return []
        return [TensorDecl(self._name(), (self.params["vocab_size"], self.params["hidden_size"]))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = None
        if not self.params.get("tied_to"):
            self.weight = rt.precision.matrix(tensors[self._name()], rt.device)

    def tie(self, embedding_weight: torch.Tensor) -> None:
        self.weight = embedding_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = linear(x, self.weight, torch.float32)
        cap = float(self.params.get("softcap", 0.0) or 0.0)
        return F.softcap_rows(logits, cap) if cap > 0.0 else logits


class OutputNormResidual(Block):
    """``x <- x + m Norm1(Mixer(x))``, then ``x <- x + m Norm2(FFN(x))``: the parts read the residual stream
    itself, and what is normalised is their OUTPUT, scaled by one number ``m`` before it is added.
    params: ``residual_mult`` (``m``, default 1), ``feed_forward`` (default True; False: a layer of a mixer
    alone, with the roles ``mixer`` and ``mixer_norm`` only).  Both norms must be plain RMS norms
    (``rms_parameters()``).

    One kernel per part takes the root mean square of the part's output, adds the scaled, normalised row to
    the float32 residual and writes the new row once more in the activation type, which is what the next part
    reads (in the float32 path the parts read the residual's own rows).  A feed-forward that leaves the sum of
    its experts' rows to its consumer has it formed inside that kernel.  The residual is up to date when the
    block returns; the rounded rows travel on as a :class:`RoundedResidual`, so that a next block of this kind
    does not round them again."""

    graph_safe = True
    accepts_deferred = True
    kernel_files = ("residual_forms.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.mult = float(self.params.get("residual_mult", 1.0))
        self.has_ff = bool(self.params.get("feed_forward", True))
        self.roles = {"mixer": "mixer", "mixer_norm": "norm"}
        if self.has_ff:
            self.roles.update({"feed_forward": "feed_forward", "feed_forward_norm": "norm"})

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt

    def _input(self, hidden: torch.Tensor, pending) -> torch.Tensor:
        if isinstance(pending, RoundedResidual):
            return pending.x
        left = resolve(pending)
        if left is not None:
            hidden.add_(left)
        return hidden if self.rt.act == torch.float32 else F.cast_rows(hidden, self.rt.act)

    def _add(self, hidden: torch.Tensor, y, norm) -> torch.Tensor:
        rms = norm.rms_parameters()
        if rms is None:
            raise ValueError("output_norm_residual: the norm of a part's output must be a plain RMS norm")
        if isinstance(y, WeightedRowSum):
            y = (y.rows, y.index, y.weights, y.extra, y.scale)
        else:
            y = resolve(y)
        x = F.out_norm_add(hidden, y, rms[0], rms[1], self.mult, None if self.rt.act == torch.float32 else self.rt.act)
        return hidden if x is None else x

    def forward(self, layer: BuiltLayer, hidden: torch.Tensor, pending, ctx: StepContext, caches):
        x = self._input(hidden, pending)
        x = self._add(hidden, layer.mixer.forward(x, ctx, caches.get("mixer")), layer.mixer_norm)
        if self.has_ff:
            x = self._add(hidden, layer.feed_forward.forward_deferred(x, ctx), layer.feed_forward_norm)
        return None if x is hidden else RoundedResidual(x)

    def prefetch_layer(self, layer: BuiltLayer, ctx: StepContext, caches) -> None:
        layer.mixer.prefetch_first(ctx, caches.get("mixer"))


class ParallelResidual(Block):
    """``x <- x + Mixer(Norm1(x)) + FFN(Norm2(x))``: both parts read the same residual and their outputs
    are added together.  params: ``feed_forward`` (default True; False: a layer of a mixer alone, with the
    roles ``mixer_norm`` and ``mixer`` only); ``shared_norm`` (default False; True: the layer has ONE norm,
    ``mixer_norm``, and the feed-forward reads its output too: ``x <- x + Mixer(h) + FFN(h)``, ``h = Norm(x)``).

    The two outputs travel on as one pending sum (:class:`TensorSum`) and are added by whatever reads the
    residual next.  When both norms are :class:`~mini_infer_b200.parts.norm.ScalarRMSNorm` with the same
    epsilon they differ by a factor only, and one kernel adds what is pending, takes the root mean square
    once and writes both inputs."""

    graph_safe = True
    accepts_deferred = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.has_ff = bool(self.params.get("feed_forward", True))
        self.shared_norm = bool(self.params.get("shared_norm", False))
        self._side_stream = None
        self._ones = None
        self._ones_before = []
        self.roles = {"mixer_norm": "norm", "mixer": "mixer"}
        if self.has_ff:
            self.roles.update({"feed_forward": "feed_forward"} if self.shared_norm else
                              {"feed_forward_norm": "norm", "feed_forward": "feed_forward"})

    def forward(self, layer: BuiltLayer, hidden: torch.Tensor, pending, ctx: StepContext, caches):
        n1 = layer.mixer_norm
        if not self.has_ff:
            x1 = apply_norm(n1, hidden, pending)
            return layer.mixer.forward(x1, ctx, caches.get("mixer"))
        n2 = None if self.shared_norm else layer.feed_forward_norm
        pair = getattr(n1, "apply_pair", None)
        if n2 is None:
            x1 = x2 = apply_norm(n1, hidden, pending)       # one norm: both parts read its output
        elif pair is not None and getattr(n2, "scalar_gain", None) is not None and n2.eps == n1.eps:
            x1, x2 = pair(hidden, pending, n2)
        else:
            x1 = apply_norm(n1, hidden, pending)
            x2 = apply_norm(n2, hidden, None)
        two_streams = TUNING.parallel_residual_two_streams and x1.is_cuda
        if two_streams and getattr(layer.mixer, "large_steps_fill_the_device", False):
            two_streams = ctx.num_tokens <= TUNING.parallel_residual_two_streams_max_tokens_full_sm_mixer
        if not two_streams:
            y = layer.mixer.forward(x1, ctx, caches.get("mixer"))
            return self._sum(y, layer.feed_forward.forward_deferred(x2, ctx))
        # the two branches share nothing but the residual they read: the feed-forward goes to a second stream
        main = torch.cuda.current_stream()
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=x1.device)
        side = self._side_stream
        side.wait_stream(main)
        x2.record_stream(side)
        with torch.cuda.stream(side):
            f = layer.feed_forward.forward_deferred(x2, ctx)
        for t in (f.rows, f.index, f.weights, f.extra, f.scale) if isinstance(f, WeightedRowSum) else (f,):
            if t is not None:
                t.record_stream(main)
        y = layer.mixer.forward(x1, ctx, caches.get("mixer"))
        main.wait_stream(side)
        return self._sum(y, f)

    def _sum(self, y: torch.Tensor, f):
        """The two parts' outputs as one pending sum.  A feed-forward that leaves the weighted sum of its
        experts' rows to the next norm's kernel (and has no shared expert in the place of the sum's extra
        term) takes the mixer's output along as that term, with a weight of one: the norm's kernel then adds
        both while it reads the row anyway."""
        if isinstance(f, WeightedRowSum) and f.extra is None:
            T = y.shape[0]
            if self._ones is None or self._ones.numel() < T or self._ones.device != y.device:
                # a captured pass keeps reading the tensor it was captured with: a smaller one stays alive
                self._ones_before.append(self._ones)
                self._ones = torch.ones(max(T, 1024), dtype=torch.float32, device=y.device)
            return WeightedRowSum(f.rows, f.index, f.weights, y, self._ones[:T])
        return TensorSum(y, resolve(f))

    def prefetch_layer(self, layer: BuiltLayer, ctx: StepContext, caches) -> None:
        layer.mixer.prefetch_first(ctx, caches.get("mixer"))


class StreamMerge(Block):
    """A run of no parts that re-enters the embedding into the residual stream:
    ``x <- W [x ; x0] + step[pass]`` with ``x0`` the embedding's output, ``W [H, 2H]`` (the columns of ``x``
    first) and one row of ``step [passes, H]`` chosen by the schedule entry's ``pass`` argument.  It stands
    before the first layer of every pass of a stretch of layers that runs several times.

    params: ``hidden_size``, ``passes``, ``weight`` and ``step`` (tensor names below the prefix)."""

    graph_safe = True
    accepts_deferred = True
    needs_embedding_output = True
    kernel_files = ("residual_forms.cu",)
    roles: dict = {}

    def tensor_decls(self) -> List[TensorDecl]:
        H, n = int(self.params["hidden_size"]), int(self.params["passes"])
        return [TensorDecl(self.prefix + self.params.get("weight", "in"), (H, 2 * H)),
                TensorDecl(self.prefix + self.params.get("step", "step"), (n, H), "bias")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.w = rt.precision.matrix(tensors[self.prefix + self.params.get("weight", "in")], rt.device)
        self.step = rt.precision.small(tensors[self.prefix + self.params.get("step", "step")], rt.device)

    def forward(self, layer: BuiltLayer, hidden: torch.Tensor, pending, ctx: StepContext, caches):
        a, b = split_sum(pending)
        t = int(ctx.entry_args.get("pass", 0))
        both = F.concat_cast(hidden, a, b, ctx.embedding_output, self.rt.act)
        F.rows_plus_vec(hidden, linear(both, self.w, torch.float32), self.step[t])
        return None


register_part("block", "prenorm_residual", PreNormResidual)
register_part("block", "parallel_residual", ParallelResidual)
register_part("block", "output_norm_residual", OutputNormResidual)
register_part("block", "stream_merge", StreamMerge)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear", LinearHead)
