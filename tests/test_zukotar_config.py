"""Zukotar without a GPU: the configuration reader, the registry, the tensors the model expects,
the order of its layer runs, and the plain implementation's own mechanisms against closed forms."""
import json
import math

import pytest
import torch

import plain_zukotar as P
import zukotar_tiny as Z


def test_registry_finds_the_design_by_its_architecture_string():
    from rllm_b200.config import config_from_dict, registered_architectures
    assert "Zukotar" in registered_architectures()
    arch, cfg = config_from_dict(Z.ZA)
    assert arch.name == "Zukotar" and cfg.width == 96 and cfg.vocab == 160
    assert cfg.layers[1].mixer.window == 21 and cfg.layers[2].mixer.window is None
    assert cfg.layers[1].mixer.rot_dims == 8 and cfg.layers[1].mixer.rot_dim == 16
    assert cfg.layers[1].mlp is None and cfg.layers[2].mlp.groups == 4 and cfg.layers[2].mlp.keep == 2
    assert cfg.layers[0].mlp.groups == 1
    again = type(cfg).from_dict(cfg.to_dict())
    assert again == cfg


@pytest.mark.parametrize("name", list(Z.TINY))
def test_layer_runs_follow_the_loop(name):
    from rllm_b200.config import config_from_dict
    raw = Z.TINY[name][0]
    _, cfg = config_from_dict(raw)
    assert cfg.layer_runs() == P.layer_runs(raw)
    model_runs = [r for r in cfg.layer_runs()]
    n = len(raw["layers"])
    loop = raw.get("loop")
    assert len(model_runs) == n + (0 if not loop else (loop["times"] - 1) * (loop["stop"] - loop["start"]))


def test_every_run_of_a_layer_has_a_cache_layer_of_its_own():
    from rllm_b200.config import config_from_dict
    from rllm_b200.parts import LatentCacheSpec, StateSpec
    arch, cfg = config_from_dict(Z.ZA)
    model = arch.build(cfg)
    specs = model.cache_specs()
    assert len(specs) == 7 and len({c.cache_layer for c in model.schedule if c.cache_layer >= 0}) == 7
    kinds = [type(s) for s in specs]
    assert kinds == [StateSpec, LatentCacheSpec] * 3 + [LatentCacheSpec]
    assert specs[1] == specs[3] == LatentCacheSpec(64, 21) and specs[6] == LatentCacheSpec(32, None)
    # a pass begins with its own row of the loop's table, added by a block without a cache
    begins = [c for c in model.schedule if c.cache_layer < 0]
    assert [model.blocks[c.block].index for c in begins] == [0, 1, 2]
    assert model.schedule[0].cache_layer < 0 and model.schedule[3].cache_layer < 0


def test_expected_tensors_and_sizes_the_checkpoint_alone_knows(tmp_path):
    from rllm_b200.config import config_from_dict
    from rllm_b200.weights import WeightError, expected_tensors, load_weights, write_random_model
    arch, cfg = config_from_dict(Z.ZC)
    names = {n: s.shape for n, s, *_ in expected_tensors(arch.build(cfg))}
    assert names["embed"] == (120, 72) and names["loop.step"] == (2, 72) and names["final.norm"] == (72,)
    assert names["l0.mix.q"] == (3 * 16, 72) and names["l0.mix.dkv"] == (40, 72) and names["l0.mix.g"] == (3, 72)
    assert names["l0.mix.uk"] == (36, 36) and names["l0.mix.uv"] == (60, 36) and names["l0.mix.dkv.norm"] == (36,)
    assert names["l1.mix.a1"] == (8, 72) and names["l1.mix.a2"] == (72, 8) and names["l1.mix.a2.b"] == (72,)
    assert names["l1.mix.norm"] == (44,) and names["l1.mlp.e8.down"] == (72, 28) and names["l1.mlp.router"] == (9, 72)
    assert "lm_head.weight" not in names and "l0.norm2b" in names
    # a folder written with one bottleneck width loads into a model whose configuration names none
    d = write_random_model(Z.ZC, 3, str(tmp_path / "m"))
    raw = json.loads(json.dumps(Z.ZC))
    del raw["layers"][1]["mixer"]["decay_rank"]
    arch, cfg = config_from_dict(raw)
    model = arch.build(cfg)
    assert dict((n, s.shape) for n, s, *_ in expected_tensors(model))["l1.mix.a1"] == (-1, 72)
    load_weights(model, d, torch.float32, "cpu")
    gla = model.blocks[1].mixer
    assert gla.w_in.shape == (2 * 2 * (36 + 44) + 8, 72) and gla.w_a2.shape == (72, 8)
    # any other wrong size is still an error
    raw["layers"][0]["mixer"]["kv_rank"] = 32
    arch, cfg = config_from_dict(raw)
    with pytest.raises(WeightError) as e:
        load_weights(arch.build(cfg), d, torch.float32, "cpu")
    assert any(n == "l0.mix.uk" for n, *_ in e.value.wrong_shape)


@pytest.mark.parametrize("change,msg", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][2]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(count=5), "groups"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, msg):
    from rllm_b200.config import ConfigError, config_from_dict
    raw = json.loads(json.dumps(Z.ZA))
    change(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert msg in str(e.value)


# ----------------------------------------------------------------- the plain implementation itself

def test_plain_rotation_turns_pairs_and_leaves_the_rest():
    x = torch.arange(12, dtype=P.DT).reshape(1, 12).repeat(3, 1)
    y = P.rotate_interleaved(x, torch.tensor([0, 1, 5]), 100.0, 8)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, 8:], x[:, 8:])
    a = 5 * 100.0 ** (-2.0 * 1 / 8)
    assert math.isclose(float(y[2, 2]), 2 * math.cos(a) - 3 * math.sin(a), rel_tol=1e-12)
    assert math.isclose(float(y[2, 3]), 3 * math.cos(a) + 2 * math.sin(a), rel_tol=1e-12)
    assert torch.allclose((y[:, :8] ** 2).sum(-1), (x[:, :8] ** 2).sum(-1))


def test_plain_gla_equals_its_unrolled_sum():
    """o_t = sum_{j<=t} (q_t . (prod_{j<i<=t} alpha_i) k_j) v_j, written out, against the recurrence."""
    torch.manual_seed(0)
    T, W, H, d, v, r = 7, 10, 2, 3, 4, 2
    m = {"heads": H, "dim": d, "vdim": v, "tau": 3.0}
    w = {"q": torch.randn(H * d, W), "k": torch.randn(H * d, W), "v": torch.randn(H * v, W), "g": torch.randn(H * v, W),
         "a1": torch.randn(r, W), "a2": torch.randn(H * d, r), "a2.b": torch.randn(H * d), "norm": torch.rand(v) + 0.5,
         "o": torch.randn(W, H * v)}
    w = {"x." + k: t.to(P.DT) for k, t in w.items()}
    h = torch.randn(T, W, dtype=P.DT)
    got = P.gla(h, w, "x.", m, 1e-5)
    q = (h @ w["x.q"].T).reshape(T, H, d) / math.sqrt(d)
    k = (h @ w["x.k"].T).reshape(T, H, d)
    val = (h @ w["x.v"].T).reshape(T, H, v)
    al = torch.sigmoid((h @ w["x.a1"].T) @ w["x.a2"].T + w["x.a2.b"]).pow(1 / 3.0).reshape(T, H, d)
    o = torch.zeros(T, H, v, dtype=P.DT)
    for t in range(T):
        for j in range(t + 1):
            decay = torch.ones(H, d, dtype=P.DT)
            for i in range(j + 1, t + 1):
                decay = decay * al[i]
            o[t] += ((q[t] * decay * k[j]).sum(-1))[:, None] * val[j]
    o = P.rms_norm(o, w["x.norm"], 1e-5).reshape(T, H * v)
    g = h @ w["x.g"].T
    want = (o * g * torch.sigmoid(g)) @ w["x.o"].T
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-9)


def test_plain_router_keeps_to_the_best_groups_and_does_not_renormalise():
    z = torch.tensor([[0.0, 5.0, 0.1, 0.2, 4.0, 4.5, 4.4, 0.3]], dtype=P.DT)     # 4 groups of 2
    w_router = torch.eye(8, dtype=P.DT)
    idx, wt = P.route(z, w_router, {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}})
    s = torch.softmax(z, -1)[0]
    # groups by their largest score: {0,1} (5.0), {4,5} (4.5), {6,7} (4.4), {2,3}; expert 6 is shut out
    assert idx[0].tolist() == [1, 5, 4] and torch.allclose(wt[0], s[[1, 5, 4]]) and float(wt.sum()) < 1.0
    idx, _ = P.route(z, w_router, {"experts": 8, "top": 3})
    assert idx[0].tolist() == [1, 5, 6]


def test_plain_window_edge_and_full_model_shapes():
    """A key that would win every score is seen at distance window - 1 and not at distance window."""
    cfg, w = Z.ZB, None
    torch.manual_seed(1)
    m = Z.latent(2, 4, 4, 3, 6, 1.0, 100.0, 4, 5)
    W = 8
    w = {"x." + k: torch.randn(*s, dtype=P.DT) * 0.3 for k, s in
         {"q": (16, W), "dkv": (10, W), "dkv.norm": (6,), "uk": (8, 6), "uv": (6, 6), "g": (2, W), "o": (W, 6)}.items()}
    h = torch.randn(12, W, dtype=P.DT)
    base = P.latent_attention(h, w, "x.", m, 1e-6)
    h2 = h.clone()
    h2[3] = h2[3] * 50                      # position 3 changes: seen by 3..7 only
    moved = (P.latent_attention(h2, w, "x.", m, 1e-6) - base).abs().sum(-1) > 1e-9
    assert moved.tolist() == [False] * 3 + [True] * 5 + [False] * 4
