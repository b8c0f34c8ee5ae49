"""``Bogetar`` described as an arrangement of parts.

A decoder whose layers put a norm in groups before AND after each part, a short convolution over time before
each part's input and a layer scale behind each output norm (``sandwich_residual``):

* ``delta``     gated delta rule with one decay per head (``gated_delta``)
* ``parallel``  two mixers that read the same input and whose outputs are added with two weights: windowed
                attention with head norms, rotation by halves, logistic key weights that are not normalised and
                a logistic output gate (``head_mix_attention``), and gated linear attention with a decay per key
                channel (``gated_linear_attention``)

The feed-forward is a mixture of bounded gated experts whose router keeps only the best groups of experts
eligible (``sparse_moe``), or none.  The output head is the embedding table.

Nothing here computes: the function turns ``config.json`` into a :class:`ModelSpec`.  The rank of the linear
attention's decay projection is given by the shape of ``a1`` alone: a folder's checkpoint header is read for it
(``tensor_shapes``), else ``decay_rank`` of the mixer's sizes, else a default.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.bogetar_config import BogetarConfig, expert_groups
from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DEFAULT_DECAY_RANK = 16
SWISH_SLOPE = 1.702         # of the experts' gated unit: g * logistic(1.702 g) * (u + 1)


def _norm(c: BogetarConfig, tensor: str) -> PartSpec:
    return PartSpec("rmsnorm_grouped", {"size": c.width, "eps": c.eps, "groups": c.norm_groups, "tensor": tensor})


def _conv(c: BogetarConfig, tensor: str) -> PartSpec:
    return PartSpec("residual_short_conv", {"channels": c.width, "taps": c.taps, "tensor": tensor})


def _attention(c: BogetarConfig, m: Mapping[str, Any]) -> PartSpec:
    position = PartSpec("none")
    rot = m.get("rot")
    if rot:
        position = PartSpec("rope", {"head_dim": m["dim"], "rot_dim": rot["dims"], "theta": rot["base"]})
    return PartSpec("head_mix_attention", {
        "hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "window": m["mask"]["size"], "scale": m["scale"], "position": position,
        "qk_norm": {"eps": c.eps}, "head_mix": False, "key_weights": "logistic", "output_gate": True})


def _linear_attention(c: BogetarConfig, m: Mapping[str, Any], i: int, shapes) -> PartSpec:
    name = f"l{i}.mix.right.a1"
    rank = int(shapes[name][0]) if shapes is not None and name in shapes else int(m.get("decay_rank", DEFAULT_DECAY_RANK))
    return PartSpec("gated_linear_attention", {
        "hidden_size": c.width, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "tau": m["tau"], "decay_rank": rank, "eps": c.eps})


def _delta(c: BogetarConfig, m: Mapping[str, Any]) -> PartSpec:
    return PartSpec("gated_delta", {
        "hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "conv": m["conv"], "eps": c.eps})


def _experts(c: BogetarConfig, mlp: Mapping[str, Any]) -> PartSpec:
    r, e = mlp["router"], mlp["expert"]
    return PartSpec("sparse_moe", {
        "hidden_size": c.width, "num_experts": r["experts"], "top_k": r["top"], "expert_intermediate_size": e["ff"],
        "shared_intermediate_size": 0, "norm_topk_prob": False, "activation": "clamped_swish", "limit": e["limit"],
        "slope": SWISH_SLOPE, "expert_groups": expert_groups(r), "router": "router", "expert": "e{e}.",
        "gate": "gate", "up": "up", "down": "down"})


def build_bogetar(config_json: Dict[str, Any]) -> ModelSpec:
    c = BogetarConfig.from_json_dict(config_json)
    shapes: Optional[Mapping[str, Tuple[int, ...]]] = config_json.get("tensor_shapes")
    layers = []
    for i, l in enumerate(c.layers):
        parts = {
            "mixer_norm": LayerPart("norm", _norm(c, "norm1"), ""),
            "mixer_conv": LayerPart("mixer", _conv(c, "canon1"), ""),
            "mixer_out_norm": LayerPart("norm", _norm(c, "norm1b"), ""),
        }
        block = {"hidden_size": c.width, "input_conv": True, "feed_forward": l.mlp is not None,
                 "layer_scale": {"mixer": "ls1", "feed_forward": "ls2"}}
        if l.type == "delta":
            parts["mixer"] = LayerPart("mixer", _delta(c, l.mixer), "mix.")
        else:
            parts["mixer"] = LayerPart("mixer", _attention(c, l.mixer["left"]), "mix.left.")
            parts["mixer_b"] = LayerPart("mixer", _linear_attention(c, l.mixer["right"], i, shapes), "mix.right.")
            block.update({"second_mixer": True, "mixer_scale": float(l.mixer["left_scale"]),
                          "second_mixer_scale": float(l.mixer["right_scale"])})
        if l.mlp is not None:
            parts["feed_forward_norm"] = LayerPart("norm", _norm(c, "norm2"), "")
            parts["feed_forward_conv"] = LayerPart("mixer", _conv(c, "canon2"), "")
            parts["feed_forward"] = LayerPart("feed_forward", _experts(c, l.mlp), "mlp.")
            parts["feed_forward_out_norm"] = LayerPart("norm", _norm(c, "norm2b"), "")
        layers.append(LayerSpec(f"l{i}", PartSpec("sandwich_residual", block), parts))
    # a layer without a feed-forward may still carry the tensors of the second half's norms, scale and filter
    unused = tuple(f"l{i}.{n}" for i, l in enumerate(c.layers) if l.mlp is None
                   for n in ("norm2", "norm2b", "ls2", "canon2"))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab, max_context=1 << 30,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=_norm(c, "final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": c.vocab, "hidden_size": c.width, "tied_to": "embed"}),
        embedding_prefix="", final_norm_prefix="", lm_head_prefix="", unused_tensors=unused)


register_architecture("Bogetar", build_bogetar,
                      "Bogetar decoder (norms in groups before and after each part, input convolutions and layer "
                      "scale; gated delta rule, or windowed attention with logistic key weights beside gated linear "
                      "attention; mixture of bounded gated experts chosen within the best expert groups)")
