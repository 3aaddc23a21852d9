"""Livovik without a GPU: the configuration reader, the registry, tensor names, the schedule of layers that run
on another layer's tensors, the cache specs, the random-weights folder, and the plain implementation's own
mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import livovik_tiny as L
import plain_livovik as P
from rllm_b200.config import ConfigError, LivovikConfig, config_from_dict
from rllm_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("name", list(L.TINY))
def test_reader_round_trip_and_registry(name):
    raw = L.TINY[name][0]
    arch, cfg = config_from_dict(raw)
    assert arch.name == "Livovik" and isinstance(cfg, LivovikConfig)
    assert LivovikConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.vocab == raw["vocab"] and cfg.width == raw["width"] and cfg.postln_alpha == raw["postln_alpha"]
    for lay, r in zip(cfg.layers, raw["layers"]):
        m = r["mixer"]
        assert (lay.mixer.heads, lay.mixer.kv_heads, lay.mixer.dim, lay.mixer.vdim) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
        assert lay.mixer.chunk == (m["mask"]["size"] if "mask" in m else None)
        assert lay.mixer.rot_dims == (m["rot"]["dims"] if "rot" in m else 0)
        assert lay.weights_of == r.get("weights_of")


def test_model_structure_follows_the_configuration():
    arch, cfg = config_from_dict(L.LC)
    model = arch.build(cfg)
    # layers 1 and 3 run on layer 0's tensors (3 through 1): one block, three calls, a cache layer each
    assert [(c.block, c.cache_layer) for c in model.schedule] == [(0, 0), (0, 1), (1, 2), (0, 3)]
    names = {n for n, *_ in expected_tensors(model)}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.sink",
            "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.e6.gate", "l0.mlp.shared.sg", "l0.mlp.shared.down",
            "l2.mlp.up", "l2.mlp.down"} <= names
    assert not any(n.startswith(("l1.", "l3.")) for n in names)
    specs = model.cache_specs()
    assert specs[0] == specs[1] == specs[3] and specs[0].chunk == 33 and specs[0].v_dim == 12 and specs[0].head_dim == 20
    assert specs[2].chunk == 64 and specs[2].kv_heads == 5
    # a layer without feed-forward has no second norm; no mask means no block rule
    arch, cfg = config_from_dict(L.LB)
    model = arch.build(cfg)
    names = {n for n, *_ in expected_tensors(model)}
    assert "l1.norm1" in names and "l1.norm2" not in names and not any(n.startswith("l1.mlp") for n in names)
    assert model.cache_specs()[1].chunk is None and model.cache_specs()[1].v_dim is None
    assert "l0.mlp.shared.sg" not in names and "l0.mlp.shared.gate" not in names


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 15), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 64), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 2), "weights_of"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 0), "differs"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].__setitem__("high", 0.5), "scaling"),
])
def test_refusals(edit, what):
    raw = copy.deepcopy(L.LA)
    edit(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert what.split(".")[-1] in str(e.value)


def test_an_entry_on_another_layers_tensors_may_leave_out_what_it_shares():
    raw = copy.deepcopy(L.LC)
    full = config_from_dict(raw)[1]
    raw["layers"][1] = {"type": "attention", "weights_of": 0, "mixer": raw["layers"][1]["mixer"]}      # no mlp key
    raw["layers"][3] = {"weights_of": 1}                                                                   # nothing else
    assert config_from_dict(raw)[1] == full


def test_random_folder_is_read_by_the_plain_reader(tmp_path):
    d = L.make_model_dir(tmp_path, "LB")
    cfg, w = P.read_model_dir(d)
    assert cfg["architecture"] == "Livovik" and w["l0.mix.sink"].shape == (6,) and w["l0.mix.v"].shape == (40, 64)
    lg = P.forward(cfg, w, L.random_prompt(17, cfg["vocab"], 1))
    assert lg.shape == (17, 200) and torch.isfinite(lg).all()


# ------------------------------------------------------------------ the plain implementation against closed forms

def test_plain_softmax_with_sink_and_mask():
    s = torch.tensor([[0.3, -1.0, 2.0, 0.5]], dtype=P.F64)
    allowed = torch.tensor([[True, False, True, True]])
    p = P.softmax_with_sink(s, allowed, 1.25)
    den = math.exp(1.25) + math.exp(0.3) + math.exp(2.0) + math.exp(0.5)
    assert torch.allclose(p, torch.tensor([[math.exp(0.3), 0.0, math.exp(2.0), math.exp(0.5)]], dtype=P.F64) / den)
    assert float(p.sum()) < 1.0
    # a very negative sink leaves the ordinary softmax
    assert abs(float(P.softmax_with_sink(s, allowed, -1e9).sum()) - 1.0) < 1e-12


def test_plain_block_rule_and_frequencies():
    assert P.visible(41, 21, {"size": 21}) and not P.visible(42, 41, {"size": 21}) and P.visible(42, 42, {"size": 21})
    assert not P.visible(3, 4, None) and P.visible(1000, 0, None)
    f = P.rotary_frequencies(8, 10000.0)
    assert f == [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    # wavelengths 2 pi / f = 6.3, 63, 628, 6283 against original 64 (high 4: below 16 kept; low 1: above 64 divided)
    g = P.rotary_frequencies(8, 10000.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
    assert g[0] == f[0] and g[2] == f[2] / 8 and g[3] == f[3] / 8
    s = (64 / (2 * math.pi / f[1]) - 1.0) / 3.0
    assert 0 < s < 1 and abs(g[1] - ((1 - s) * f[1] / 8 + s * f[1])) < 1e-15


def test_plain_rotation_pairs_halves_and_keeps_the_rest():
    x = torch.arange(12, dtype=P.F64).view(1, 1, 12) + 1
    y = P.rotate(x, [3], [0.5, 0.25])                 # dimensions (0, 2) and (1, 3) are pairs
    c, s_, c2, s2 = math.cos(1.5), math.sin(1.5), math.cos(0.75), math.sin(0.75)
    want = [1 * c - 3 * s_, 2 * c2 - 4 * s2, 3 * c + 1 * s_, 4 * c2 + 2 * s2] + list(range(5, 13))
    assert torch.allclose(y.view(-1), torch.tensor(want, dtype=P.F64))
    assert torch.equal(P.rotate(x, [0], [0.5, 0.25]), x)


def test_plain_experts_weight_the_input():
    g = torch.Generator().manual_seed(3)
    W, F, E = 6, 5, 4
    w = {"router": torch.randn(E, W, generator=g, dtype=P.F64)}
    for e in range(E):
        for n, shape in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F))):
            w[f"e{e}.{n}"] = torch.randn(*shape, generator=g, dtype=P.F64)
    h = torch.randn(3, W, generator=g, dtype=P.F64)
    out = P.moe_ffn(h, w, {"router": {"experts": E, "top": 2}})
    s = torch.sigmoid(h @ w["router"].T)
    for t in range(3):
        top = sorted(range(E), key=lambda e: -float(s[t, e]))[:2]
        want = sum(P.gated_expert(s[t, e] * h[t:t + 1], w, f"e{e}.")[0] for e in top)
        assert torch.allclose(out[t], want)
        # not the same as weighting the output: the activation is not homogeneous
        assert not torch.allclose(out[t], sum(s[t, e] * P.gated_expert(h[t:t + 1], w, f"e{e}.")[0] for e in top))
