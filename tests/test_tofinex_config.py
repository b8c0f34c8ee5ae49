"""Tofinex without a GPU: the reader of ``config.json`` and its refusals, the description the engine builds
from it, the manifest against names made from the configuration alone, and the plain model's own consistency
(the mechanisms written a second way)."""

import copy
import math

import pytest
import torch

import plain_tofinex as pt
import tofinex_tiny as tt
from mini_infer_b200.config.model_config import ConfigError
from mini_infer_b200.config.registry import build_model_spec, known_architectures
from mini_infer_b200.config.tofinex_config import TofinexConfig
from mini_infer_b200.engine.model import Model


def test_the_architecture_is_registered():
    assert "Tofinex" in known_architectures()


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_reader_and_description(name):
    cfg = tt.CONFIGS[name]
    c = TofinexConfig.from_json_dict(cfg)
    assert (c.vocab, c.width, c.eps) == (cfg["vocab"], cfg["width"], cfg["norm"]["eps"])
    assert c.residual_mult == cfg.get("residual_mult", 1.0) and c.logit_softcap == cfg.get("logit_softcap", 0.0)
    spec = build_model_spec(cfg)
    assert spec.lm_head.get("tied_to") and spec.lm_head.get("softcap") == c.logit_softcap
    first = c.first_blending_layer
    for i, (l, ls) in enumerate(zip(cfg["layers"], spec.layers)):
        m, mixer = l["mixer"], ls.mixer
        assert ls.block.kind == "output_norm_residual" and ls.block.get("residual_mult") == c.residual_mult
        assert ls.block.get("feed_forward") == (l["mlp"] is not None)
        assert mixer.kind == "head_mix_attention" and mixer.get("sink") and mixer.get("window") == 0
        assert (mixer.get("num_heads"), mixer.get("num_kv_heads"), mixer.get("head_dim"), mixer.get("value_dim")) == \
            (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
        assert mixer.get("scale") == m["scale"] and mixer.get("softcap") == (m.get("softcap") or 0.0)
        pos = mixer.get("position")
        if m.get("rot"):
            assert pos.kind == "rope" and pos.get("pairing") == "neighbours" and pos.get("rot_dim") == m["rot"]["dims"]
        else:
            assert pos.kind == "none"
        blend = mixer.get("value_blend")
        assert (blend is not None) == bool(m.get("v_mix"))
        if blend:
            assert blend["first"] == (i == first)
        if l["mlp"] is None:
            assert "feed_forward" not in ls.parts and "feed_forward_norm" not in ls.parts
        elif l["mlp"]["kind"] == "dense":
            assert ls.feed_forward.kind == "gated_mlp" and ls.feed_forward.get("activation") == "silu"
        else:
            ff = ls.feed_forward
            assert ff.kind == "sparse_moe" and ff.get("scoring") == "sigmoid" and ff.get("weight_input")
            assert not ff.get("norm_topk_prob")
            assert ff.get("shared_intermediate_size") == (l["mlp"]["shared"]["ff"] if l["mlp"].get("shared") else 0)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_manifest_matches_names_made_from_the_configuration(name):
    cfg = tt.CONFIGS[name]
    w = tt.make_weights(cfg, 1)
    shapes = {k: tuple(v.shape) for k, v in w.items()}
    decls = {d.name: tuple(d.shape) for d in Model(build_model_spec(dict(cfg, tensor_shapes=shapes))).tensor_decls()}
    assert decls == shapes
    # without a header every blending layer declares its weight
    assert set(d.name for d in Model(build_model_spec(cfg)).tensor_decls()) == set(shapes)


def test_a_checkpoint_without_the_first_blending_weight_is_described_too():
    cfg = tt.CONFIG_A
    w = tt.make_weights(cfg, 1)
    first = TofinexConfig.from_json_dict(cfg).first_blending_layer
    shapes = {k: tuple(v.shape) for k, v in w.items() if k != f"l{first}.mix.vmix"}
    decls = {d.name for d in Model(build_model_spec(dict(cfg, tensor_shapes=shapes))).tensor_decls()}
    assert decls == set(shapes)


class _Header:
    """Names, shapes and types as a checkpoint's header gives them."""

    def __init__(self, weights):
        self.w = weights

    def names(self):
        return list(self.w)

    def shape(self, name):
        return tuple(self.w[name].shape)

    def dtype(self, name):
        return self.w[name].dtype

    def describe(self):
        return "a header"


def test_a_checkpoint_that_stores_every_layer_alike_fits():
    """A blending weight in a layer that blends nothing, a second norm in a layer without a feed-forward and a
    number stored as a vector of one are no errors; any other stray tensor is."""
    from mini_infer_b200.weights.loader import WeightError, check_manifest
    cfg = tt.CONFIG_A
    w = tt.make_weights(cfg, 2)
    w["l0.mix.vmix"] = torch.tensor(0.3, dtype=torch.bfloat16)                 # layer 0 blends nothing
    w["l2.norm2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)             # layer 2 has no feed-forward
    w["l3.mix.vmix"] = w["l3.mix.vmix"].reshape(1)
    spec = build_model_spec(dict(cfg, tensor_shapes={k: tuple(v.shape) for k, v in w.items()}))
    model = Model(spec)
    check_manifest(model.tensor_decls(), _Header(w), allow_unexpected=spec.unused_tensors)
    w["l1.norm3"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    with pytest.raises(WeightError):
        check_manifest(model.tensor_decls(), _Header(w), allow_unexpected=spec.unused_tensors)


def test_one_cache_group_per_geometry():
    assert len(Model(build_model_spec(tt.CONFIG_D)).kv_groups) == 2
    same = copy.deepcopy(tt.CONFIG_D)
    same["layers"][1]["mixer"].update(heads=1, kv_heads=1, dim=8, vdim=8)
    assert len(Model(build_model_spec(same)).kv_groups) == 1


def _broken(change):
    cfg = copy.deepcopy(tt.CONFIG_A)
    change(cfg)
    return cfg


@pytest.mark.parametrize("change", [
    lambda c: c.pop("vocab"), lambda c: c.update(width=0), lambda c: c.pop("norm"), lambda c: c.update(layers=[]),
    lambda c: c["layers"][0].update(type="recurrent"), lambda c: c["layers"][0]["mixer"].pop("scale"),
    lambda c: c["layers"][0]["mixer"].update(heads=3), lambda c: c["layers"][0]["mixer"].update(softcap=-1.0),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"].update(v_mix=1), lambda c: c["layers"][2]["mixer"].update(vdim=11),
    lambda c: c["layers"][0]["mlp"].update(kind="conv"), lambda c: c["layers"][0]["mlp"].pop("ff"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=6), lambda c: c["layers"][1]["mlp"].update(shared={"ff": 0}),
    lambda c: c.update(logit_softcap=-2.0), lambda c: c.update(residual_mult="half"),
])
def test_refusals(change):
    with pytest.raises(ConfigError):
        TofinexConfig.from_json_dict(_broken(change))


# --------------------------------------------------------------------------- #
# the plain model against itself
# --------------------------------------------------------------------------- #

def test_rotation_of_neighbours_is_a_complex_multiplication():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 3, 12, generator=g, dtype=torch.float64)
    got = pt.rotate_neighbours(x, 8, 50.0, first_position=4)
    z = torch.view_as_complex(x[..., :8].reshape(9, 3, 4, 2).contiguous())
    f = torch.tensor([50.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float64)
    a = torch.arange(4, 13, dtype=torch.float64)[:, None] * f[None]
    want = torch.view_as_real(z * torch.polar(torch.ones_like(a), a)[:, None, :]).reshape(9, 3, 8)
    assert float((got[..., :8] - want).abs().max()) < 1e-12 and torch.equal(got[..., 8:], x[..., 8:])
    # a score depends on the distance of the two positions only
    q, k = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    s = [float((pt.rotate_neighbours(q, 8, 50.0, a0 + 5) * pt.rotate_neighbours(k, 8, 50.0, a0)).sum()) for a0 in (0, 3, 40)]
    assert max(s) - min(s) < 1e-9


def test_softmax_with_one_key_more():
    s = torch.tensor([[0.3, -1.0, 2.0, 5.0]], dtype=torch.float64)
    vis = torch.tensor([[True, True, True, False]])
    p = pt.sink_softmax(s, vis)
    e = torch.exp(s[0, :3])
    assert float((p[0, :3] - e / (1 + e.sum())).abs().max()) < 1e-12 and float(p[0, 3]) == 0.0
    # it is the ordinary softmax over the keys and one score of zero more
    full = torch.softmax(torch.cat([s[0, :3], torch.zeros(1, dtype=torch.float64)]), dim=0)
    assert float((p[0, :3] - full[:3]).abs().max()) < 1e-12
    big = pt.sink_softmax(torch.tensor([[800.0, 799.0]], dtype=torch.float64), torch.tensor([[True, True]]))
    assert bool(torch.isfinite(big).all()) and abs(float(big.sum()) - 1.0) < 1e-12


def test_router_and_input_weights():
    g = torch.Generator().manual_seed(2)
    W, E, ff = 12, 4, 6
    w = {"r.router": torch.randn(E, W, generator=g, dtype=torch.float64)}
    for e in range(E):
        w[f"r.e{e}.gate"], w[f"r.e{e}.up"] = (torch.randn(ff, W, generator=g, dtype=torch.float64) for _ in range(2))
        w[f"r.e{e}.down"] = torch.randn(W, ff, generator=g, dtype=torch.float64)
    h = torch.randn(3, W, generator=g, dtype=torch.float64)
    idx, wt, s = pt.router_choice(h, w["r.router"], 2)
    assert torch.equal(s, torch.sigmoid(h @ w["r.router"].T)) and torch.equal(wt, s.gather(1, idx))
    assert all(s[t, idx[t, 0]] >= s[t, idx[t, 1]] >= s[t].sort().values[-3] for t in range(3))
    out, _ = pt.moe(h, w, "r.", {"router": {"top": 2}, "shared": None})
    t = 1
    by_hand = sum(pt.gated_unit(wt[t, j] * h[t:t + 1], w[f"r.e{int(idx[t, j])}.gate"], w[f"r.e{int(idx[t, j])}.up"],
                                w[f"r.e{int(idx[t, j])}.down"])[0] for j in range(2))
    assert float((out[t] - by_hand).abs().max()) < 1e-12


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_a_prefix_gives_the_same_logits_and_blending_reads_the_first_blending_layer(name):
    cfg = tt.CONFIGS[name]
    w = tt.make_weights(cfg, 4)
    toks = tt.random_requests(cfg, [17], 1)["r0"]
    whole = pt.forward(cfg, w, toks)
    assert float((pt.forward(cfg, w, toks[:9]) - whole[:9]).abs().max()) < 1e-9           # causal
    if cfg.get("logit_softcap"):
        assert float(whole.abs().max()) < cfg["logit_softcap"]
    # the first blending layer never reads its own weight; every later one does
    first = TofinexConfig.from_json_dict(cfg).first_blending_layer
    w2 = dict(w)
    w2[f"l{first}.mix.vmix"] = torch.tensor(0.9, dtype=torch.bfloat16)
    assert torch.equal(pt.forward(cfg, w2, toks), whole)
    later = [i for i, l in enumerate(cfg["layers"]) if l["mixer"].get("v_mix") and i != first]
    if later:
        w3 = dict(w)
        w3[f"l{later[0]}.mix.vmix"] = torch.tensor(0.9, dtype=torch.bfloat16)
        assert float((pt.forward(cfg, w3, toks) - whole).abs().max()) > 1e-4
