"""``Tofinex`` described as an arrangement of parts.

A decoder whose parts read the residual stream itself; what is normalised is each part's OUTPUT, which joins the
residual times one number (``x <- x + m norm1(mixer(x))``, ``x <- x + m norm2(ff(x))``, block
``output_norm_residual``).  The embedding's rows pass a norm before they become the residual, and the output head
is the embedding table, its logits capped.

* mixer          grouped-query attention over all earlier tokens whose query and key heads are brought to unit
                 root mean square (a gain per dimension), rotated with neighbouring dimensions paired, scores
                 capped, a softmax that counts one key more (score 0, no value), and, where the layer says so,
                 values blended with the first such layer's values of the same token
                 (``head_mix_attention`` with ``sink``, ``value_blend`` and no head mix)
* feed-forward   dense ``silu`` gated unit (``gated_mlp``), or a mixture of experts whose router scores every
                 expert with the logistic function and whose weights scale the experts' inputs, beside a gated
                 shared expert (``sparse_moe`` with ``scoring`` and ``weight_input``), or none

Nothing here computes: the function turns ``config.json`` into a :class:`ModelSpec`.
"""

from __future__ import annotations

from typing import Any, Dict

from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.tofinex_config import TofinexConfig


def _norm(c: TofinexConfig, tensor: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": c.width, "eps": c.eps, "tensor": tensor})


def _mixer_spec(c: TofinexConfig, i: int, shapes) -> PartSpec:
    m = c.layers[i].mixer
    rot = m.get("rot")
    position = PartSpec("none")
    if rot and rot["dims"]:
        position = PartSpec("rope", {"head_dim": m["dim"], "rot_dim": rot["dims"], "theta": rot["base"],
                                     "pairing": "neighbours"})
    params = {"hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "value_dim": m["vdim"], "window": 0, "scale": m["scale"], "softcap": float(m.get("softcap") or 0.0),
              "head_mix": False, "qk_norm": {"eps": c.eps}, "sink": True, "position": position}
    if c.layers[i].blends_values:
        # a checkpoint's header says whether the layer's blending weight is stored (the first blending layer
        # never reads its own); without a header (random weights) every blending layer has one
        name = f"l{i}.mix.vmix"
        params["value_blend"] = {"name": "first", "first": i == c.first_blending_layer, "tensor": "vmix",
                                 "declared": True if shapes is None else name in shapes}
    return PartSpec("head_mix_attention", params)


def _ff_spec(c: TofinexConfig, i: int) -> PartSpec:
    mlp = c.layers[i].mlp
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": mlp["ff"], "activation": "silu",
                                      "gate": "gate", "up": "up", "down": "down"})
    shared = mlp.get("shared")
    return PartSpec("sparse_moe", {
        "hidden_size": c.width, "num_experts": mlp["router"]["experts"], "top_k": mlp["router"]["top"],
        "expert_intermediate_size": mlp["expert"]["ff"], "shared_intermediate_size": shared["ff"] if shared else 0,
        "norm_topk_prob": False, "scoring": "sigmoid", "weight_input": True, "activation": "silu",
        "router": "router", "expert": "e{e}.", "gate": "gate", "up": "up", "down": "down",
        "shared": "shared.", "shared_gate": "shared.sg"})


def build_tofinex(config_json: Dict[str, Any]) -> ModelSpec:
    c = TofinexConfig.from_json_dict(config_json)
    shapes = config_json.get("tensor_shapes")
    W = c.width
    layers, unused = [], []
    for i, l in enumerate(c.layers):
        # a writer that stores every layer alike leaves a blending weight in layers that blend nothing and a
        # second norm in layers without a feed-forward
        if not l.blends_values:
            unused.append(f"l{i}.mix.vmix")
        if l.mlp is None:
            unused.append(f"l{i}.norm2")
        parts = {"mixer": LayerPart("mixer", _mixer_spec(c, i, shapes), "mix."),
                 "mixer_norm": LayerPart("norm", _norm(c, "norm1"), "")}
        if l.mlp is not None:
            parts["feed_forward"] = LayerPart("feed_forward", _ff_spec(c, i), "mlp.")
            parts["feed_forward_norm"] = LayerPart("norm", _norm(c, "norm2"), "")
        layers.append(LayerSpec(f"l{i}", PartSpec("output_norm_residual", {"residual_mult": c.residual_mult,
                                                                           "feed_forward": l.mlp is not None}), parts))
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_context=1 << 30,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "tensor": "embed",
                                               "norm": _norm(c, "embed.norm")}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=_norm(c, "final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": c.vocab, "hidden_size": W, "tied_to": "embed",
                                    "softcap": c.logit_softcap}),
        embedding_prefix="", final_norm_prefix="", lm_head_prefix="", unused_tensors=tuple(unused))


register_architecture("Tofinex", build_tofinex,
                      "Tofinex decoder (parts that read the residual itself and whose outputs are normalised; "
                      "attention with normalised neighbour-rotated heads, capped scores, a softmax with one key "
                      "more and values blended with the first layer's; dense or sigmoid-routed input-weighted "
                      "feed-forward with a gated shared expert; tied, capped output head)")
