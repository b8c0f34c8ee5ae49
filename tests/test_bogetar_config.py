"""Bogetar without a GPU: the reader of ``config.json`` and its refusals, the description the engine builds from
it, the manifest against names made from the configuration alone, what each layer keeps between steps, and the
plain model's own consistency (the mechanisms written a second way)."""

import copy

import pytest
import torch

import bogetar_tiny as bt
import plain_bogetar as pb
from mini_infer_b200.cache.needs import KVNeed, StateNeed
from mini_infer_b200.config.bogetar_config import BogetarConfig
from mini_infer_b200.config.model_config import ConfigError
from mini_infer_b200.config.registry import build_model_spec, known_architectures
from mini_infer_b200.engine.model import Model


def test_the_architecture_is_registered():
    assert "Bogetar" in known_architectures()


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_reader_and_description(name):
    cfg = bt.CONFIGS[name]
    c = BogetarConfig.from_json_dict(cfg)
    assert (c.vocab, c.width, c.eps) == (cfg["vocab"], cfg["width"], cfg["norm"]["eps"])
    assert c.norm_groups == cfg["norm"].get("groups", 1) and c.taps == cfg["canon"]["taps"]
    spec = build_model_spec(cfg)
    assert spec.lm_head.get("tied_to") == "embed"
    assert spec.final_norm.kind == "rmsnorm_grouped" and spec.final_norm.get("groups") == c.norm_groups
    for l, ls in zip(cfg["layers"], spec.layers):
        m = l["mixer"]
        assert ls.block.kind == "sandwich_residual" and ls.block.get("input_conv")
        assert ls.block.get("feed_forward") == (l["mlp"] is not None)
        for role in ("mixer_norm", "mixer_out_norm"):
            assert ls.parts[role].spec.kind == "rmsnorm_grouped" and ls.parts[role].spec.get("groups") == c.norm_groups
        assert ls.mixer_conv.kind == "residual_short_conv" and ls.mixer_conv.get("taps") == c.taps
        if l["type"] == "delta":
            assert ls.mixer.kind == "gated_delta" and "mixer_b" not in ls.parts
            assert (ls.mixer.get("num_heads"), ls.mixer.get("num_kv_heads"), ls.mixer.get("head_dim"),
                    ls.mixer.get("value_dim"), ls.mixer.get("conv")) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"])
        else:
            a, r = m["left"], m["right"]
            assert ls.block.get("second_mixer") and ls.block.get("mixer_scale") == m["left_scale"]
            assert ls.block.get("second_mixer_scale") == m["right_scale"]
            left, right = ls.mixer, ls.mixer_b
            assert left.kind == "head_mix_attention" and left.get("key_weights") == "logistic" and left.get("output_gate")
            assert not left.get("head_mix") and left.get("window") == a["mask"]["size"] and left.get("scale") == a["scale"]
            assert left.get("qk_norm") == {"eps": c.eps}
            pos = left.get("position")
            if a.get("rot"):
                assert pos.kind == "rope" and pos.get("rot_dim") == a["rot"]["dims"] and pos.get("theta") == a["rot"]["base"]
            else:
                assert pos.kind == "none"
            assert right.kind == "gated_linear_attention" and right.get("tau") == r["tau"]
            assert right.get("decay_rank") == r["decay_rank"]
        if l["mlp"] is None:
            assert not any(role.startswith("feed_forward") for role in ls.parts)
        else:
            ff, r = ls.feed_forward, l["mlp"]["router"]
            assert ff.kind == "sparse_moe" and ff.get("activation") == "clamped_swish" and not ff.get("norm_topk_prob")
            assert ff.get("limit") == l["mlp"]["expert"]["limit"] and ff.get("top_k") == r["top"]
            g = r.get("groups")
            assert tuple(ff.get("expert_groups")) == ((g["count"], g["keep"]) if g else (1, 1))
            assert ls.feed_forward_conv.get("tensor") == "canon2"


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_manifest_matches_names_made_from_the_configuration(name):
    cfg = bt.CONFIGS[name]
    w = bt.make_weights(cfg, 1)
    shapes = {k: tuple(v.shape) for k, v in w.items()}
    decls = {d.name: tuple(d.shape) for d in Model(build_model_spec(dict(cfg, tensor_shapes=shapes))).tensor_decls()}
    assert decls == shapes


def test_the_decay_rank_comes_from_the_checkpoint_header():
    cfg = copy.deepcopy(bt.CONFIG_A)
    w = bt.make_weights(cfg, 1)
    shapes = {k: tuple(v.shape) for k, v in w.items()}
    for l in cfg["layers"]:
        if l["type"] == "parallel":
            del l["mixer"]["right"]["decay_rank"]
    decls = {d.name: tuple(d.shape) for d in Model(build_model_spec(dict(cfg, tensor_shapes=shapes))).tensor_decls()}
    assert decls == shapes


def test_what_each_layer_keeps_between_steps():
    cfg = bt.CONFIG_A
    model = Model(build_model_spec(cfg))
    taps, W = cfg["canon"]["taps"], cfg["width"]
    states = {owner: need for owner, need in model.state_needs}
    for i, l in enumerate(cfg["layers"]):
        assert states[(i, "mixer_conv")].shape == ((taps - 1) * W,)
        assert ((i, "feed_forward_conv") in states) == (l["mlp"] is not None)
        m = l["mixer"]
        if l["type"] == "delta":
            channels = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
            assert states[(i, "mixer")].shape == (m["heads"] * m["dim"] * m["vdim"] + (m["conv"] - 1) * channels,)
        else:
            r = m["right"]
            assert states[(i, "mixer_b")].shape == (r["heads"] * r["dim"] * r["vdim"],)
            assert isinstance(states[(i, "mixer_b")], StateNeed)
    # one paged group per geometry and window of the attention halves
    needs = sorted((g.need.num_kv_heads, g.need.head_dim, g.need.value_dim, g.need.window) for g in model.kv_groups)
    want = sorted((l["mixer"]["left"]["kv_heads"], l["mixer"]["left"]["dim"], l["mixer"]["left"]["vdim"],
                   l["mixer"]["left"]["mask"]["size"]) for l in cfg["layers"] if l["type"] == "parallel")
    assert needs == want and all(isinstance(g.need, KVNeed) for g in model.kv_groups)


def _bad(change):
    cfg = copy.deepcopy(bt.CONFIG_A)
    change(cfg)
    return cfg


@pytest.mark.parametrize("change", [
    lambda c: c.pop("canon"),
    lambda c: c["norm"].update(groups=5),
    lambda c: c["layers"][0].update(type="attention"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][1]["mixer"]["left"].pop("mask"),
    lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18),
    lambda c: c["layers"][1]["mixer"]["right"].update(tau=0.0),
    lambda c: c["layers"][1]["mixer"].pop("right_scale"),
    lambda c: c["layers"][1]["mlp"].update(kind="dense"),
    lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
    lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"),
])
def test_refusals(change):
    with pytest.raises(ConfigError):
        BogetarConfig.from_json_dict(_bad(change))


# ---- the plain model's own consistency ------------------------------------------------------------------- #

def test_plain_model_is_causal_and_keeps_its_window():
    cfg = bt.CONFIG_A
    w = bt.make_weights(cfg, 3)
    toks = bt.random_requests(cfg, [30], 1)["r0"]
    full = pb.forward(cfg, w, toks)
    assert float((pb.forward(cfg, w, toks[:17]) - full[:17]).abs().max()) < 1e-9


def test_plain_windowed_attention_written_a_second_way():
    torch.manual_seed(0)
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "mask": {"size": 3}, "scale": 0.4,
         "rot": {"base": 100.0, "dims": 4}}
    W, T, eps = 10, 9, 1e-5
    P = {"q": torch.randn(24, W), "k": torch.randn(12, W), "v": torch.randn(10, W), "q.norm": torch.rand(6) + 0.5,
         "k.norm": torch.rand(6) + 0.5, "pb": torch.randn(4), "g": torch.randn(20, W), "o": torch.randn(W, 20)}
    P = {k: v.double() for k, v in P.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    got = pb.windowed_sigmoid_attention(h, P, "", m, eps, pb.same)
    # token by token, the rotation as a complex multiplication
    def prep(x, norm, t):
        x = x / torch.sqrt((x * x).mean() + eps) * norm
        z = torch.complex(x[:2], x[2:4]) * torch.polar(torch.ones(2, dtype=torch.float64),
                                                       t * torch.tensor([1.0, 100.0 ** -0.5], dtype=torch.float64))
        return torch.cat([z.real, z.imag, x[4:]])
    want = torch.zeros(T, W, dtype=torch.float64)
    for t in range(T):
        heads = []
        for hd in range(4):
            q = prep((P["q"] @ h[t])[hd * 6:(hd + 1) * 6], P["q.norm"], t)
            acc = torch.zeros(5, dtype=torch.float64)
            for j in range(max(0, t - 2), t + 1):
                g = hd // 2
                k = prep((P["k"] @ h[j])[g * 6:(g + 1) * 6], P["k.norm"], j)
                acc += torch.sigmoid((q @ k) * 0.4 + P["pb"][hd]) * (P["v"] @ h[j])[g * 5:(g + 1) * 5]
            heads.append(acc)
        want[t] = P["o"] @ (torch.cat(heads) * torch.sigmoid(P["g"] @ h[t]))
    assert float((got - want).abs().max()) < 1e-9


def test_plain_linear_attention_is_a_decayed_sum_over_earlier_tokens():
    torch.manual_seed(1)
    m = {"heads": 2, "dim": 3, "vdim": 4, "tau": 4.0}
    W, T, eps = 7, 6, 1e-6
    P = {k: v.double() for k, v in {"q": torch.randn(6, W), "k": torch.randn(6, W), "v": torch.randn(8, W),
         "g": torch.randn(8, W), "o": torch.randn(W, 8), "norm": torch.rand(4) + 0.5, "a1": torch.randn(2, W),
         "a2": torch.randn(6, 2), "a2.b": torch.randn(6)}.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    got = pb.gated_linear_attention(h, P, "", m, eps, pb.same)
    q, k, v = (h @ P["q"].T) * 3 ** -0.5, h @ P["k"].T, h @ P["v"].T
    alpha = torch.sigmoid(h @ P["a1"].T @ P["a2"].T + P["a2.b"]) ** 0.25
    rows = []
    for t in range(T):
        heads = []
        for hd in range(2):
            o = torch.zeros(4, dtype=torch.float64)
            for j in range(t + 1):
                decay = alpha[j + 1:t + 1, hd * 3:(hd + 1) * 3].prod(dim=0)       # channel by channel since token j
                o += ((q[t, hd * 3:(hd + 1) * 3] * decay) @ k[j, hd * 3:(hd + 1) * 3]) * v[j, hd * 4:(hd + 1) * 4]
            heads.append(o / torch.sqrt((o * o).mean() + eps) * P["norm"])
        y = torch.cat(heads) * (lambda z: z * torch.sigmoid(z))(P["g"] @ h[t])
        rows.append(P["o"] @ y)
    assert float((got - torch.stack(rows)).abs().max()) < 1e-9


def test_plain_delta_rule_forgets_what_it_overwrites():
    """With a write strength of one, no decay and the same unit key twice, the second value replaces the first."""
    S = torch.zeros(3, 2, dtype=torch.float64)
    k = torch.tensor([0.6, 0.0, 0.8], dtype=torch.float64)
    for v in (torch.tensor([1.0, 2.0]), torch.tensor([-3.0, 5.0])):
        u = 1.0 * (v.double() - S.T @ k)
        S = S + k[:, None] * u[None, :]
    assert float((S.T @ k - torch.tensor([-3.0, 5.0], dtype=torch.float64)).abs().max()) < 1e-12


def test_plain_router_keeps_to_the_best_groups():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    h = torch.eye(6, dtype=torch.float64)[:1] * 0 + torch.tensor([[0.0, 0.1, 3.0, -1.0, 2.0, 2.5]], dtype=torch.float64)
    idx, s = pb.route(h, torch.eye(6, dtype=torch.float64), r)
    assert sorted(idx[0].tolist()) == [2, 3]            # group 1 holds the best score; expert 5 is not eligible
    r["groups"]["keep"] = 2
    idx, _ = pb.route(h, torch.eye(6, dtype=torch.float64), r)
    assert sorted(idx[0].tolist()) == [2, 5]
    weights = s[0, idx[0]]
    assert float(weights.sum()) < 1.0                    # the scores as they are, not renormalised
