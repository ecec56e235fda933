"""The Runopel design without a GPU: its configuration, its description as parts, the cache and state plan the decoder
derives from it, the retention rule of a windowed cache, and the plain implementation against itself and against
hand-made cases (the recurrence against its unrolled sum, a window's edge, the streams, the limits, the router)."""
import json
import math

import pytest
import torch

import plain_runopel as plain
import runopel_models as tm

F = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, dtype=F, generator=torch.Generator().manual_seed(seed))


def test_config_round_trip_and_refusals():
    from hipinfer_b200.config import ConfigError, config_from_dict

    for name, cfg in tm.MODELS.items():
        c = config_from_dict(cfg)
        assert c.architecture == "Runopel" and c.to_dict()["layers"] == cfg["layers"], name
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c
    assert config_from_dict(tm.C).streams is None and config_from_dict(tm.B).streams == 1

    def broken(change):
        bad = json.loads(json.dumps(tm.A))
        change(bad)
        with pytest.raises(ConfigError):
            config_from_dict(bad)

    broken(lambda d: d["layers"][0]["mixer"].update(groups=3))              # 4 heads in 3 groups
    broken(lambda d: d["layers"][0]["mixer"].update(norm_groups=5))         # 64 channels in 5 parts
    broken(lambda d: d["layers"][1]["mlp"]["router"].update(top=6))         # six of five experts
    broken(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10))        # more rotated dimensions than the rotated part has
    broken(lambda d: d["layers"][1]["mixer"]["mask"].update(size=0))
    broken(lambda d: d["layers"][2].update(type="convolution"))
    broken(lambda d: d["layers"][3]["mlp"].update(kind="sparse"))
    broken(lambda d: d["layers"][0]["mlp"].pop("limit"))
    broken(lambda d: d.pop("norm"))


def test_spec_caches_and_states():
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.models.decoder import DecoderModel
    from hipinfer_b200.parts.registry import BuildContext

    def build(cfg):
        return DecoderModel(get_architecture("Runopel").build_spec(config_from_dict(cfg)), BuildContext.meta())

    # A: two latent layers with equal windows share one group of pages; the recurrent layers hold a state and K - 1 inputs
    m = build(tm.A)
    assert [(g.kind, g.n_layers) for g in m.cache_groups] == [("window", 2)]
    assert [p.write if p else None for p in m.cache_plan] == [None, True, None, True]
    assert {k: v[0] for k, v in m.state_specs.items()} == {(0, "S"): (4, 8, 16), (0, "conv"): (3, 96), (2, "S"): (2, 16, 24),
                                                           (2, "conv"): (1, 80)}
    # B: a window of one token and a layer without a mask are caches of different kinds; one tap carries no inputs
    m = build(tm.B)
    assert sorted((g.kind, g.n_layers) for g in m.cache_groups) == [("full", 1), ("window", 1)]
    assert m.state_specs[(1, "conv")][0] == (0, 120) and m.state_specs[(3, "conv")][0] == (6, 128)
    # D: streams and experts by name; a layer without a feed-forward has neither its norm nor its stream weights
    names = {s.name: tuple(s.shape) for s in build(tm.D).param_specs()}
    assert names["l0.hc1.mix"] == (4, 4) and names["l0.hc2.in"] == (4,) and names["l1.mlp.router"] == (3, 50)
    assert names["l1.mlp.e2.down"] == (50, 22) and names["l1.mix.in"] == (2 * 18 + 2 * 7 + 3, 50) and names["l1.mix.conv"] == (32, 5)
    assert names["l0.mix.dkv"] == (20 + 6, 50) and names["l0.mix.uk"] == (2 * 10, 20) and names["l0.mlp.gate.b"] == (30,)
    assert "l2.norm2" not in names and "l2.hc2.in" not in names and "l2.mlp.gate" not in names
    # C: no streams at all: no stream weights anywhere
    assert not [n for n in (s.name for s in build(tm.C).param_specs()) if ".hc" in n]


def test_window_retention_rule():
    from hipinfer_b200.cache import CacheGroupSpec, CacheManager

    spec = CacheGroupSpec("g", "window", 1, 1, 8, 40, (("c", 1, 8),), ())
    cm = CacheManager([spec], 16, 12, 1)
    cm.add_request("x")
    cm.append("x", 100)                # the next query, at 100, sees 61..100: pages wholly below 61 are dead
    cm.release_behind_window("x")
    table = cm.block_table("x", 0)
    assert table[:3] == [-1] * 3 and table[3] >= 0
    cm.append("x", 60)                 # next query at 160 sees 121..160
    cm.release_behind_window("x")
    table = cm.block_table("x", 0)
    assert table[:7] == [-1] * 7 and table[7] >= 0
    cm.free_request("x")
    cm.check()


@pytest.mark.parametrize("which", ["a", "b", "d"])
def test_plain_model_whole_against_token_by_token(which):
    cfg = tm.MODELS[which]
    w = tm.draw_weights(cfg, 3, torch.float32)
    toks = torch.randint(0, cfg["vocab"], (50,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(cfg, w, toks)
    # causality: a prefix's logits are the whole sequence's first rows
    part = plain.forward(cfg, w, toks[:31])
    assert float((whole[:31] - part).abs().max()) < 1e-9 * float(whole.abs().max())
    layers = []
    plain.forward(cfg, w, toks[:5], layers_out=layers)
    assert len(layers) == len(cfg["layers"]) and layers[0].shape == (5, cfg["width"])


def test_decisive_routers_choose_by_token_alone():
    cfg = tm.MODELS["c"]
    w = tm.draw_weights(cfg, 3, torch.bfloat16)
    code = 16
    toks = list(range(40))
    chosen = {}
    real_route = plain.route

    def spy(h, router, top):
        s, order = real_route(h, router, top)
        z = torch.sort(h @ router.T, dim=-1, descending=True).values
        chosen.setdefault("gaps", []).append(float(((z[:, :-1] - z[:, 1:]) / z.abs().amax(-1, keepdim=True)).min()))
        return s, order

    plain.route = spy
    try:
        plain.forward(cfg, w, toks)
    finally:
        plain.route = real_route
    assert len(chosen["gaps"]) == 2 and min(chosen["gaps"]) > 0.02
    assert len({tuple(w["embed"][t, :code].tolist()) for t in toks}) > 30


def test_scan_is_the_unrolled_sum():
    """y_t = sum_(s <= t) (prod_(s < r <= t) a_r) dt_s (C_t . B_s) x_s + D x_t, with a_r = exp(-exp(A) dt_r)."""
    T, H, P, N, G = 9, 4, 3, 5, 2
    x, B, C = rnd(T, H, P, seed=1), rnd(T, G, N, seed=2), rnd(T, G, N, seed=3)
    dt = plain.softplus(rnd(T, H, seed=4))
    A_log, D = rnd(H, seed=5) * 0.5, rnd(H, seed=6)
    y = plain.state_space_scan(x, B, C, dt, A_log, D, G)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            want = D[h] * x[t, h]
            for s in range(t + 1):
                decay = math.exp(-math.exp(float(A_log[h])) * float(dt[s + 1:t + 1, h].sum()))
                want = want + decay * dt[s, h] * (C[t, g] @ B[s, g]) * x[s, h]
            assert torch.allclose(y[t, h], want, atol=1e-12)


def test_convolution_taps_and_softplus():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=F)                    # the last tap is the current token's
    out = plain.causal_conv(x, w, torch.tensor([0.5], dtype=F))
    assert out[:, 0].tolist() == [1.5, 12.5, 123.5, 1230.5]
    z = torch.tensor([-800.0, -1.0, 0.0, 30.0, 900.0], dtype=F)
    sp = plain.softplus(z)
    assert sp[0] == 0.0 and sp[4] == 900.0 and abs(float(sp[2]) - math.log(2.0)) < 1e-15 and abs(float(sp[1]) - math.log1p(math.exp(-1.0))) < 1e-15


def test_gate_comes_before_the_grouped_norm():
    m = dict(heads=2, vdim=4, state=3, groups=1, norm_groups=2)
    W = 6
    w = {"in": rnd(2 * 8 + 2 * 3 + 2, W, seed=1), "conv": rnd(8 + 6, 2, seed=2), "conv.b": rnd(14, seed=3), "dt_bias": rnd(2, seed=4),
         "A_log": rnd(2, seed=5), "D": rnd(2, seed=6), "norm": torch.ones(8, dtype=F), "o": torch.eye(8, dtype=F)}
    y = plain.mamba2(rnd(5, W, seed=7), w, m, 0.0)
    # with a unit weight and no eps each half of a row has a root mean square of exactly one
    assert torch.allclose((y.reshape(5, 2, 4) ** 2).mean(-1), torch.ones(5, 2, dtype=F))


def test_window_edge_rotation_and_shared_rotated_key():
    seen = plain.window_mask(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True] and seen[1].tolist() == [True, True, False, False, False, False]
    assert plain.window_mask(3, 1).tolist() == [[True, False, False], [False, True, False], [False, False, True]]
    assert plain.window_mask(3).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    t = rnd(4, 2, 12, seed=1)
    pos = torch.tensor([0, 1, 5, 9])
    a = plain.rotate_pairs(t, pos, 8, 100.0)
    assert torch.allclose(a.norm(dim=-1), t.norm(dim=-1)) and torch.equal(a[..., 8:], t[..., 8:]) and torch.equal(a[0], t[0])
    assert torch.allclose(a[1, 0, 0], t[1, 0, 0] * math.cos(1.0) - t[1, 0, 1] * math.sin(1.0))
    assert torch.allclose(a[2, 1, 3], t[2, 1, 3] * math.cos(5 * 100.0 ** -0.25) + t[2, 1, 2] * math.sin(5 * 100.0 ** -0.25))
    # a key just outside the window with a huge score changes nothing; just inside it takes the whole weight
    m = dict(heads=1, dim=2, rot_dim=2, vdim=2, kv_rank=2, scale=1.0, rot=dict(base=10.0, dims=2), mask=dict(size=3))
    w = {"q": torch.zeros(4, 3, dtype=F), "dkv": torch.zeros(4, 3, dtype=F), "dkv.norm": torch.ones(2, dtype=F),
         "uk": torch.eye(2, dtype=F) * 50.0, "uv": torch.eye(2, dtype=F), "o": torch.eye(2, dtype=F)}
    w["q"][0, 0] = 1.0                                               # q = (h0, 0 | 0, 0)
    w["dkv"][0, 1], w["dkv"][1, 2] = 1.0, 1.0                        # the latent is (h1, h2), normed
    h = torch.tensor([[1.0, 1.0, 0.0], [1.0, 0.0, 1.0], [1.0, 0.0, 1.0], [1.0, 0.0, 1.0]], dtype=F)
    out = plain.latent_attention(h, w, m, 0.0)
    # token 0's key (sqrt2, 0) * 50 scores high with every query; row 2 still sees it (2 - 0 < 3), row 3 does not
    assert out[2, 0] > 1.4 and abs(float(out[3, 0])) < 1e-9


def test_streams_limits_and_router_by_hand():
    # dense: the gate is capped from above only, the other branch on both sides, and one is added to it
    w = {"gate": torch.eye(2, dtype=F), "gate.b": torch.zeros(2, dtype=F), "up": torch.eye(2, dtype=F), "up.b": torch.zeros(2, dtype=F),
         "down": torch.eye(2, dtype=F), "down.b": torch.tensor([0.25, 0.0], dtype=F)}
    out = plain.dense_ff(torch.tensor([[9.0, -9.0]], dtype=F), w, 2.0)
    sg = lambda g: g / (1.0 + math.exp(-1.702 * g))
    assert torch.allclose(out, torch.tensor([[sg(2.0) * 3.0 + 0.25, sg(-9.0) * -1.0]], dtype=F))
    # routed: the score multiplies the expert's INPUT and is not renormalised
    h = torch.tensor([[1.0, 2.0]], dtype=F)
    e = {"router": torch.tensor([[0.0, 0.0], [1.0, 0.0], [-1.0, 0.0]], dtype=F)}
    for i in range(3):
        e[f"e{i}.gate"], e[f"e{i}.up"], e[f"e{i}.down"] = torch.eye(2, dtype=F) * (i + 1), torch.eye(2, dtype=F), torch.eye(2, dtype=F)
    s, order = plain.route(h, e["router"], 2)
    assert order.tolist() == [[1, 0]] and abs(float(s[0, 1]) - 1 / (1 + math.exp(-1.0))) < 1e-15 and float(s[0, 0]) == 0.5
    want = torch.zeros(2, dtype=F)
    for i in (1, 0):
        v = s[0, i] * h[0]
        want = want + plain.silu(v * (i + 1)) * v
    assert torch.allclose(plain.routed_ff(h, e, 3, 2)[0], want)
    # equal scores: the lower index wins
    assert plain.route(h, torch.zeros(3, 2, dtype=F), 2)[1].tolist() == [[0, 1]]
    # streams: with mix = identity, in = out = (1, 0) the model is the plain residual on stream 0 plus an untouched copy
    cfg = tm.model(30, 8, [tm.ssm(1, 4, 3, mlp=tm.dense(6))], streams=2, mult=0.5)
    wt = tm.draw_weights(cfg, 1, torch.float32)
    for q in ("hc1", "hc2"):
        wt[f"l0.{q}.in"], wt[f"l0.{q}.out"], wt[f"l0.{q}.mix"] = torch.tensor([1.0, 0.0]), torch.tensor([1.0, 0.0]), torch.eye(2)
    one = dict(cfg)
    one.pop("streams")
    layers2, layers1 = [], []
    plain.forward(cfg, wt, [3, 7, 1], layers_out=layers2)
    plain.forward(one, wt, [3, 7, 1], layers_out=layers1)
    x0 = wt["embed"].double()[[3, 7, 1]]
    assert torch.allclose(layers2[0], layers1[0] + x0)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from hipinfer_b200.config import config_from_dict, load_config
    from hipinfer_b200.weights import write_random_model
    from hipinfer_b200.weights.safetensors_io import ModelFiles

    write_random_model(config_from_dict(tm.D), str(tmp_path / "m"), seed=4)
    assert load_config(str(tmp_path / "m")) == config_from_dict(tm.D)
    files = ModelFiles(str(tmp_path / "m"))
    assert "l1.mlp.e1.up" in files.names() and "l2.mix.A_log" in files.names() and files.info("l0.hc1.mix")[1] == (4, 4)
    files.close()
