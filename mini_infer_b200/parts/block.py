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


class SandwichResidual(Block):
    """A norm before and after each part: ``x <- x + s1 * NormB(mix(Conv(Norm(x))))``, then the same around the
    feed-forward with norms, scale and convolution of its own.  ``mix`` is one mixer or two that read the same
    input, ``a * Mixer(h) + b * MixerB(h)``; ``s`` is a vector of the width (layer scale); ``Conv`` an input part
    of its own (``h + conv(h)``, with the state that a short convolution over time needs).

    params: ``feed_forward`` (default True; False: a layer of a mixer alone), ``second_mixer`` (default False),
    ``mixer_scale`` and ``second_mixer_scale`` (``a`` and ``b``, default 1), ``input_conv`` (default False: the
    parts read the norms' outputs as they are), ``hidden_size`` and ``layer_scale`` (``{"mixer": name,
    "feed_forward": name}`` of the tensors ``s1`` and ``s2`` below the prefix; absent: no scale).

    Roles: ``mixer_norm``, ``mixer``, ``mixer_out_norm``; ``mixer_b`` with ``second_mixer``; ``mixer_conv`` with
    ``input_conv``; ``feed_forward_norm``, ``feed_forward``, ``feed_forward_out_norm`` (and
    ``feed_forward_conv``) with a feed-forward.  The norms give ``group_parameters()`` (weight, eps, groups).

    The input norm writes float32 for the convolution, which rounds to the activation type; one kernel takes
    the root mean squares of a part's output, multiplies by norm weight and layer scale (folded into one vector
    when the weights are loaded) and adds to the float32 residual.  A feed-forward that leaves the sum of its
    experts' rows to its consumer has it formed inside that kernel."""

    graph_safe = True
    accepts_deferred = True
    kernel_files = ("residual_forms.cu",)

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.has_ff = bool(p.get("feed_forward", True))
        self.second = bool(p.get("second_mixer", False))
        self.conv = bool(p.get("input_conv", False))
        self.a = float(p.get("mixer_scale", 1.0))
        self.b = float(p.get("second_mixer_scale", 1.0))
        self.scale_names = dict(p.get("layer_scale") or {})
        self.roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_out_norm": "norm"}
        if self.second:
            self.roles["mixer_b"] = "mixer"
        if self.conv:
            self.roles["mixer_conv"] = "mixer"
        if self.has_ff:
            self.roles.update({"feed_forward_norm": "norm", "feed_forward": "feed_forward",
                               "feed_forward_out_norm": "norm"})
            if self.conv:
                self.roles["feed_forward_conv"] = "mixer"
        self._folded = {}
        self._ab = None
        self._ab_before = []
        self._side_stream = None

    def tensor_decls(self) -> List[TensorDecl]:
        H = int(self.params["hidden_size"]) if self.scale_names else 0
        return [TensorDecl(self.prefix + name, (H,), "norm") for part, name in sorted(self.scale_names.items())
                if part == "mixer" or self.has_ff]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.scales = {part: tensors[self.prefix + name].to(device=rt.device, dtype=torch.float32).contiguous()
                       for part, name in self.scale_names.items() if part == "mixer" or self.has_ff}
        self._folded = {}

    def _out_weight(self, part: str, norm):
        """Weight of the output norm times the layer scale, eps, groups."""
        got = self._folded.get(part)
        if got is None:
            fn = getattr(norm, "group_parameters", None)
            if fn is not None:
                w, eps, groups = fn()
            else:
                rms = norm.rms_parameters()
                if rms is None:
                    raise ValueError("sandwich_residual: the norm of a part's output must be an RMS norm")
                w, eps, groups = rms[0], rms[1], 1
            w = w.to(torch.float32)
            if part in self.scales:
                w = (w * self.scales[part]).contiguous()
            got = self._folded[part] = (w, eps, groups)
        return got

    def _weights(self, T: int, device):
        """``[T, 1]`` times ``a`` and ``[T]`` times ``b``: the two mixers' weights as the weights of a sum of rows."""
        if self._ab is None or self._ab[0].shape[0] < T or self._ab[0].device != device:
            # a captured pass keeps reading the tensors it was captured with: smaller ones stay alive
            self._ab_before.append(self._ab)
            n = max(T, 1024)
            self._ab = (torch.full((n, 1), self.a, dtype=torch.float32, device=device),
                        torch.full((n,), self.b, dtype=torch.float32, device=device))
        return self._ab[0][:T], self._ab[1][:T]

    def _read(self, hidden: torch.Tensor, norm, conv, ctx: StepContext, cache) -> torch.Tensor:
        if conv is None:
            return apply_norm(norm, hidden, None)
        fused = getattr(conv, "forward_from_residual", None)
        if fused is not None:
            return fused(hidden, norm, ctx, cache)          # the part may run the norm inside a kernel of its own
        return conv.forward(norm.apply_float(hidden), ctx, cache)

    def _add(self, hidden: torch.Tensor, y, part: str, norm) -> None:
        w, eps, groups = self._out_weight(part, norm)
        if isinstance(y, WeightedRowSum):
            y = (y.rows, y.index, y.weights, y.extra, y.scale)
        else:
            y = resolve(y)
        F.out_norm_add(hidden, y, w, eps, 1.0, None, groups=groups)

    def forward(self, layer: BuiltLayer, hidden: torch.Tensor, pending, ctx: StepContext, caches):
        left = resolve(pending)
        if left is not None:
            hidden.add_(left)
        h = self._read(hidden, layer.mixer_norm, layer.mixer_conv if self.conv else None, ctx, caches.get("mixer_conv"))
        y2 = None
        if (self.second and TUNING.parallel_residual_two_streams and h.is_cuda
                and ctx.num_tokens <= TUNING.parallel_residual_two_streams_max_tokens_full_sm_mixer):
            # The two mixers share nothing but the input they read: in steps of few tokens, whose kernels are short
            # chains that leave the device idle, the second one goes to a second stream (decode at batch 8: 0.538 ->
            # 0.456 ms and 1.117 -> 1.005 ms at the two bench sizes).  In a prompt step the walk of the recurrence
            # beside the tensor-memory attention and the library's products, whose blocks want whole SMs, lost 7 to
            # 19 %, so large steps stay on one stream.
            main = torch.cuda.current_stream()
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=h.device)
            side = self._side_stream
            side.wait_stream(main)
            h.record_stream(side)
            with torch.cuda.stream(side):
                y2 = layer.mixer_b.forward(h, ctx, caches.get("mixer_b"))
            y2.record_stream(main)
            y = layer.mixer.forward(h, ctx, caches.get("mixer"))
            main.wait_stream(side)
        else:
            y = layer.mixer.forward(h, ctx, caches.get("mixer"))
            if self.second:
                y2 = layer.mixer_b.forward(h, ctx, caches.get("mixer_b"))
        if self.second:
            # a * y + b * y2 is formed inside the output norm's kernel, as a sum of rows with weights
            wa, wb = self._weights(y.shape[0], y.device)
            y = WeightedRowSum(y, None, wa, y2, wb)
        elif self.a != 1.0:
            y = WeightedRowSum(y, None, self._weights(y.shape[0], y.device)[0], None, None)
        self._add(hidden, y, "mixer", layer.mixer_out_norm)
        if self.has_ff:
            h = self._read(hidden, layer.feed_forward_norm, layer.feed_forward_conv if self.conv else None, ctx,
                           caches.get("feed_forward_conv"))
            self._add(hidden, layer.feed_forward.forward_deferred(h, ctx), "feed_forward", layer.feed_forward_out_norm)
        return None

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
register_part("block", "sandwich_residual", SandwichResidual)
register_part("block", "stream_merge", StreamMerge)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear", LinearHead)
