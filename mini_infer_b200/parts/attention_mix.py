"""Attention over the paged cache whose heads exchange their scores before the softmax.

Optionally every query and key head is first brought to unit root mean square and given a gain per
dimension.  ``score = (q . k) * scale``; ``score <- softcap * tanh(score / softcap)`` (if a cap is set); then every
head's score of a (query, key) pair becomes a mix of all heads' scores of that pair,
``score_h <- sum_g talk[h, g] * score_g`` (if the layer has such a matrix); then the softmax over the keys a
window lets through (behind a window the first keys of a request may stay visible).  Query/key heads and value
heads may differ in size.  One library product for q, k and v together, one kernel for head norms, rotation and
cache write, one attention kernel that owns all heads of its queries (the mix couples them), one library product
for the output.  Without a mix the heads are independent: in bfloat16, where keys and values have one size that
those kernels are built for, prompt portions then take the engine's tcgen05 attention and steps of single tokens
its split-KV kernel (both know the cap and the added key).

``key_weights`` ``logistic``: no softmax.  Every visible key weighs in with ``logistic(score + pb[h])`` (``pb``: a
number per head from the checkpoint) and a query's weights are not normalised over its keys.  ``output_gate``:
the heads' outputs are multiplied element by element with ``logistic(W_g h)`` before the output projection
(``h`` is the part's own input).

Two further options.  ``sink``: the softmax counts one key more, whose score is 0 and which has no value,
``p_j = exp(s_j) / (1 + sum exp(s_j))``, so a query may give its weight to nothing.  ``value_blend``: the layers
that name the same blend share the FIRST such layer's values of a token: every later one caches and attends over
``(1 - lam) v + lam v_first`` with its own ``lam`` (one number in the checkpoint); the first one's values travel
through the step (``StepContext.carried``), since all layers of a step see the same tokens.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..ops import functional as F
from .base import CacheBinding, KVNeed, Mixer, Runtime, StepContext, TensorDecl, linear
from .tuning import TUNING


class HeadMixAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim`` (queries and keys),
    ``value_dim``, ``window`` (0 = all keys), ``keep_first`` (behind a window the first so many keys of a
    request stay visible, at their true positions; 0 = none), ``scale``, ``softcap`` (0 = none), ``head_mix``
    (the layer has a ``[heads, heads]`` matrix that mixes the heads' scores), ``qk_norm`` (``{"eps": ...}``:
    every query and key head is divided by its root mean square and multiplied by a gain per dimension that
    the heads share, before the rotation), ``position`` (a ``PartSpec`` of category ``position``; its
    ``pairing`` says which dimensions turn together), ``sink`` (the softmax's denominator counts one more key of
    score 0), ``value_blend`` (``{"name": ..., "first": bool, "tensor": "vmix", "declared": bool}``: the
    layers of one ``name`` blend their values with those of the layer marked ``first``; ``declared`` says
    whether the checkpoint holds this layer's weight, which the first layer never reads), ``key_weights``
    (``softmax``, default, or ``logistic``: a key's weight is ``logistic(score + head_bias[h])``, not normalised;
    without head mix, cap and ``sink``), ``output_gate`` (the layer has a ``[heads*value_dim, hidden]`` matrix
    whose product with the part's input, through the logistic function, multiplies the heads' outputs), optional
    tensor names ``q``, ``k``, ``v``, ``o``, ``mix``, ``q_norm``, ``k_norm``, ``head_bias`` (default ``pb``),
    ``gate`` (default ``g``) below the prefix.

    Tensors: ``<prefix>q [heads*head_dim, hidden]``, ``<prefix>k [kv_heads*head_dim, hidden]``,
    ``<prefix>v [kv_heads*value_dim, hidden]``, ``<prefix>o [hidden, heads*value_dim]``,
    ``<prefix>talk [heads, heads]`` if ``head_mix``, ``<prefix>q.norm``, ``<prefix>k.norm [head_dim]`` if
    ``qk_norm``, ``<prefix>vmix []`` if ``value_blend``, ``<prefix>pb [heads]`` with logistic key weights,
    ``<prefix>g [heads*value_dim, hidden]`` if ``output_gate``."""

    graph_safe = True
    kernel_files = ("attention_mix.cu", "attention_mix_tc.cu", "attention_prefill_tc.cu", "attention_latent.cu")

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.dk = int(p["head_dim"])
        self.dv = int(p.get("value_dim", self.dk))
        self.window = int(p.get("window", 0))
        self.keep_first = int(p.get("keep_first", 0) or 0) if self.window > 0 else 0
        self.qk_norm = p.get("qk_norm")
        self.scale = float(p.get("scale", self.dk ** -0.5))
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.head_mix = bool(p.get("head_mix", False))
        self.sink = bool(p.get("sink", False))
        self.key_weights = p.get("key_weights", "softmax")
        if self.key_weights not in ("softmax", "logistic"):
            raise ValueError(f"attention: key weights '{self.key_weights}' are not 'softmax' or 'logistic'")
        self.logistic = self.key_weights == "logistic"
        if self.logistic and (self.head_mix or self.sink or self.softcap > 0.0):
            raise ValueError("attention: logistic key weights go without head mix, cap and added key")
        self.output_gate = bool(p.get("output_gate", False))
        if not self.head_mix and self.dk == self.dv and not self.logistic:
            # independent heads of one size may decode on the engine's split-KV kernel
            self.kernel_files = type(self).kernel_files + ("attention.cu",)
        self.blend = dict(p["value_blend"]) if p.get("value_blend") else None
        if self.blend is not None:
            self.blend_key = "value_blend:" + str(self.blend["name"])
            self.blend_first = bool(self.blend.get("first", False))
            self.blend_tensor = prefix + self.blend.get("tensor", "vmix")
            self.blend_declared = bool(self.blend.get("declared", True))
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = part_class("position", pos.kind)(pos.params, prefix)
        if self.nkv < 1 or self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} key/value heads")
        self.names = {k: prefix + p.get(k, d) for k, d in (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("mix", "talk"),
                                                            ("q_norm", "q.norm"), ("k_norm", "k.norm"),
                                                            ("head_bias", "pb"), ("gate", "g"))}

    def tensor_decls(self) -> List[TensorDecl]:
        n = self.names
        out = [TensorDecl(n["q"], (self.nh * self.dk, self.H)), TensorDecl(n["k"], (self.nkv * self.dk, self.H)),
               TensorDecl(n["v"], (self.nkv * self.dv, self.H))]
        if self.head_mix:
            out.append(TensorDecl(n["mix"], (self.nh, self.nh), "head_mix"))
        if self.qk_norm is not None:
            out += [TensorDecl(n["q_norm"], (self.dk,), "norm"), TensorDecl(n["k_norm"], (self.dk,), "norm")]
        if self.blend is not None and self.blend_declared:
            out.append(TensorDecl(self.blend_tensor, (), "blend"))
        if self.logistic:
            out.append(TensorDecl(n["head_bias"], (self.nh,), "bias"))
        if self.output_gate:
            out.append(TensorDecl(n["gate"], (self.nh * self.dv, self.H)))
        out.append(TensorDecl(n["o"], (self.H, self.nh * self.dv)))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, n = rt.precision.matrix, rt.device, self.names
        self.w_qkv = torch.cat([m(tensors[n[k]], dev) for k in ("q", "k", "v")], dim=0)
        self.w_o = m(tensors[n["o"]], dev)
        # the mix acts on float scores
        self.mix = tensors[n["mix"]].to(device=dev, dtype=torch.float32).contiguous() if self.head_mix else None
        # the head norms are float arithmetic
        self.q_gain = self.k_gain = None
        self.qk_eps = 0.0
        if self.qk_norm is not None:
            self.q_gain = tensors[n["q_norm"]].to(device=dev, dtype=torch.float32).contiguous()
            self.k_gain = tensors[n["k_norm"]].to(device=dev, dtype=torch.float32).contiguous()
            self.qk_eps = float(self.qk_norm["eps"])
        # the bias joins float scores
        self.head_bias = tensors[n["head_bias"]].to(device=dev, dtype=torch.float32).contiguous() if self.logistic else None
        self.w_gate = m(tensors[n["gate"]], dev) if self.output_gate else None
        self.inv_freq = self.position.table(dev)
        self.rot_dim = self.position.rot_dim if self.inv_freq is not None else 0
        self.neighbours = getattr(self.position, "pairing", "halves") == "neighbours"
        # the blending weight joins float arithmetic (the first layer of a blend has none to apply)
        self.blend_weight = None
        if self.blend is not None and not self.blend_first:
            if not self.blend_declared:
                raise ValueError(f"attention: '{self.blend_tensor}' is missing, and only the first layer of a "
                                 f"value blend does without its weight")
            self.blend_weight = tensors[self.blend_tensor].to(device=dev, dtype=torch.float32).reshape(1).contiguous()
        if not F.attention_mix_supported(self.nh, self.nkv, self.dk, self.dv, rt.act):
            raise ValueError(f"attention: {self.nh} heads of key size {self.dk} and value size {self.dv} "
                             f"are more than one block of the kernel holds")

        # bfloat16: scores and P.V on the tensor cores where the kernel is built for the sizes
        self._tensor_cores = rt.act == torch.bfloat16 and F.attention_mix_tc_supported(self.nh, self.nkv, self.dk, self.dv)
        # heads that exchange nothing (a cap and one key more act on a head's own scores)
        self._independent_heads = self.mix is None and self.dk == self.dv and not self.logistic
        # prompt portions on the tensor-memory attention: its blocks want whole SMs (a block arrangement that
        # runs another part beside this one asks)
        self.large_steps_fill_the_device = self._tensor_cores and self._independent_heads
        # logistic key weights on the tensor-memory attention: key and value heads of 64 or 128 numbers
        self._logistic_tc = (self.logistic and rt.act == torch.bfloat16 and self.keep_first == 0
                             and self.dk in (64, 128) and self.dv in (64, 128))
        self.large_steps_fill_the_device = self.large_steps_fill_the_device or self._logistic_tc
        # single tokens of independent heads in bfloat16: the engine's split-KV kernel where it is built for
        # the head size (it reads keys and values once per head at the memory's speed and keeps no first keys)
        self._split_decode = (rt.act == torch.bfloat16 and self._independent_heads and self.keep_first == 0
                              and F.decode_attention_supported(self.dk))

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        F.l2_prefetch(self.w_qkv)

    def cache_need(self):
        return KVNeed(self.nkv, self.dk, self.window, value_dim=self.dv, keep_first=self.keep_first)

    def _span(self, max_kv_len: int) -> int:
        """Most keys a query can see."""
        return min(self.window, max_kv_len) if self.window > 0 else max_kv_len

    def scratch_need(self, max_requests: int, max_context: int) -> Dict[str, int]:
        splits = F.attention_mix_tc_splits(self._span(max_context), self.keep_first)
        need = {"attn_mix_part_o": max_requests * splits * self.nh * self.dv,
                "attn_mix_part_ml": max_requests * splits * self.nh * 2}
        if self.dk == self.dv and F.decode_attention_supported(self.dk):
            splits = -(-max_context // min(F.DECODE_SPLIT_SIZES))
            need.update({"attn_part_o": max_requests * self.nh * splits * self.dk,
                         "attn_part_ml": max_requests * self.nh * splits * 2})
        return need

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        view = ctx.kv_groups[cache.group]
        kc, vc = view.k[cache.layer_slot], view.v[cache.layer_slot]
        qkv = linear(x, self.w_qkv, torch.float32)
        v_first = None
        if self.blend is not None:
            if self.blend_first:
                # this layer's values, as projected, for the later layers of the blend (a view: the rows stay
                # alive with the step)
                ctx.carried[self.blend_key] = qkv[:, (self.nh + self.nkv) * self.dk:]
            else:
                v_first = ctx.carried.get(self.blend_key)
                if v_first is None or v_first.shape[1] != self.nkv * self.dv:
                    raise ValueError(f"attention: the first layer of the value blend '{self.blend['name']}' has "
                                     f"not run in this step, or its values have another size")
        q = F.rope_store(qkv, ctx.positions, self.inv_freq, self.rot_dim, view.slot_mapping, kc, vc, self.nh,
                         self.nkv, self.dk, self.dv, view.page_size, self.rt.act, self.q_gain, self.k_gain,
                         self.qk_eps, neighbours=self.neighbours, v_first=v_first, blend=self.blend_weight)
        if ctx.prefetch is not None:
            ctx.prefetch((self.w_o,))       # arrives while the attention over the cache runs
        if not self._tensor_cores:
            # float32: one kernel for every step, sums in an order that the cut of the step cannot change
            a = F.attention_mix(q, kc, vc, self.mix, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                self.window, self.scale, self.softcap, self.keep_first, sink=self.sink,
                                head_bias=self.head_bias)
        elif ctx.all_decode and self._split_decode and "attn_part_o" in ctx.scratch:
            # one or two requests alone cannot fill the device with splits of 512 keys
            split = TUNING.decode_split(ctx.num_requests, F.decode_split_size())
            a = F.decode_attention(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len, ctx.scratch["attn_part_o"],
                                   ctx.scratch["attn_part_ml"], -(-ctx.max_kv_len // split), self.window,
                                   scale=self.scale, split=split, softcap=self.softcap, sink=self.sink)
        elif ctx.all_decode and "attn_mix_part_o" in ctx.scratch:
            # one token per request: a block per request could not pull a window of keys fast enough
            splits = F.attention_mix_tc_splits(self._span(ctx.max_kv_len), self.keep_first)
            a = F.attention_mix_tc(q, kc, vc, self.mix, view.block_table, ctx.q_start, ctx.kv_len, 1, self.window,
                                   self.scale, self.softcap, splits, ctx.scratch["attn_mix_part_o"],
                                   ctx.scratch["attn_mix_part_ml"], keep_first=self.keep_first, sink=self.sink,
                                   head_bias=self.head_bias)
        elif self._logistic_tc and F.prefill_attention_tc_logistic_supported(self.dk, self.dv, view.page_size):
            # prompt portions (and what decodes beside them) with logistic weights on the tensor-memory attention
            a = F.prefill_attention_tc_logistic(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                                self.window, self.scale, self.head_bias)
        elif self._independent_heads and F.prefill_attention_tc_supported(self.dk, view.page_size):
            # heads that exchange nothing, keys and values of one size the tcgen05 kernel is built for: prompt
            # portions (and what decodes beside them) take the engine's tensor-memory attention
            a = F.prefill_attention_tc(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                       self.window, self.scale, keep_first=self.keep_first, softcap=self.softcap,
                                       sink=self.sink)
        else:
            a = F.attention_mix_tc(q, kc, vc, self.mix, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len,
                                   self.window, self.scale, self.softcap, keep_first=self.keep_first,
                                   sink=self.sink, head_bias=self.head_bias)
        if self.output_gate:
            a = F.sigmoid_gate(a, False, linear(x, self.w_gate, torch.float32), 0, self.nh, self.dv)
        return linear(a.view(ctx.num_tokens, self.nh * self.dv), self.w_o, torch.float32)


register_part("mixer", "head_mix_attention", HeadMixAttention)
