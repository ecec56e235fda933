"""The Mavinex design without a GPU: its configuration, its description as parts, the cache and state plan the decoder
derives from it, and the plain implementation against itself and against hand-made cases (the recurrence against its
unrolled sum, a window's edge, the sink, both frequency rules pinned to values worked out by hand, the router)."""
import json
import math

import pytest
import torch

import mavinex_models as tm
import plain_mavinex as plain

F = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, dtype=F, generator=torch.Generator().manual_seed(seed))


def test_config_round_trip_and_refusals():
    from hipinfer_b200.config import ConfigError, config_from_dict

    for name, cfg in tm.MODELS.items():
        c = config_from_dict(cfg)
        assert c.architecture == "Mavinex" and c.to_dict()["layers"] == cfg["layers"], name
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c
    c = config_from_dict(tm.A)
    assert c.postln_alpha == 2.0 and c.embedding_scale == 8.0 and [c.weights_layer(i) for i in range(4)] == [0, 0, 2, 0]
    assert config_from_dict(tm.B).layers[1].mixer.window is None and config_from_dict(tm.B).layers[0].mixer.window == 1

    def broken(change, base=tm.A):
        bad = json.loads(json.dumps(base))
        change(bad)
        with pytest.raises(ConfigError):
            config_from_dict(bad)

    broken(lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3))            # 4 heads in 3 groups
    broken(lambda d: d["layers"][0]["mlp"]["router"].update(top=6))                 # six of five experts
    broken(lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=18))        # more rotated dimensions than the head has
    broken(lambda d: d["layers"][2]["mixer"]["rot"].update(dims=7))
    broken(lambda d: d["layers"][2]["mixer"]["mask"].update(size=0))
    broken(lambda d: d["layers"][2].update(type="convolution"))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda d: d["layers"][0]["mixer"]["right"].pop("dt_rank"))
    broken(lambda d: d["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("high"))
    broken(lambda d: d["layers"][1].update(weights_of=9))                           # no such layer
    broken(lambda d: d["layers"][1].update(weights_of=2))                           # a layer of another kind
    broken(lambda d: (d["layers"][0].update(weights_of=1), d["layers"][1].update(weights_of=0)))     # round in a circle
    broken(lambda d: d.pop("norm"))


def test_spec_caches_states_and_tensors():
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.models.decoder import DecoderModel
    from hipinfer_b200.parts.registry import BuildContext

    def build(cfg):
        return DecoderModel(get_architecture("Mavinex").build_spec(config_from_dict(cfg)), BuildContext.meta())

    # A: one side-by-side layer run three times with a cache and a state of its own each time, and one latent layer
    m = build(tm.A)
    assert len(m.spec.layers) == 2 and [s.layer for s in m.spec.order] == [0, 0, 1, 0]
    assert sorted((g.kind, g.n_layers) for g in m.cache_groups) == [("window", 1), ("window_keep_first", 3)]
    assert all(p is not None and p.write for p in m.cache_plan)
    assert {k: v[0] for k, v in m.state_specs.items()} == {(i, n): s for i in (0, 1, 3) for n, s in
                                                           (("right.S", (48, 8)), ("right.conv", (3, 48)))}
    names = {s.name: tuple(s.shape) for s in m.param_specs()}
    assert not [n for n in names if n.startswith("l1.") or n.startswith("l3.")]
    assert names["l0.mix.left.q"] == (64, 64) and names["l0.mix.left.k"] == (32, 64) and names["l0.mix.left.v"] == (48, 64)
    assert names["l0.mix.left.q.norm"] == (64,) and names["l0.mix.left.k.norm"] == (32,) and names["l0.mix.left.g"] == (96, 64)
    assert names["l0.mix.left.o"] == (64, 96) and names["l0.mix.right.in"] == (96, 64) and names["l0.mix.right.x"] == (5 + 16, 48)
    assert names["l0.mix.right.dt"] == (48, 5) and names["l0.mix.right.A_log"] == (48, 8) and names["l0.mix.right.conv"] == (48, 4)
    assert names["l0.mix.left.out"] == names["l0.mix.right.out"] == names["l0.norm1"] == names["l0.norm2"] == (64,)
    assert names["l0.mlp.router"] == (5, 64) and names["l0.mlp.router.b"] == (5,) and names["l0.mlp.e4.down"] == (64, 32)
    assert names["l2.mix.q"] == (3 * 24, 64) and names["l2.mix.dkv"] == (48, 64) and names["l2.mix.g"] == (3, 64)
    assert names["l2.mix.sink"] == (3,) and names["l2.mix.uv"] == (72, 40) and names["head"] == (160, 64) and names["final.norm"] == (64,)
    # B: a window of one token and a layer without a mask are caches of different kinds; one tap carries no inputs; a layer
    # without a feed-forward has no second norm
    m = build(tm.B)
    assert sorted((g.kind, g.n_layers) for g in m.cache_groups) == [("full", 1), ("full", 2), ("window", 1), ("window_keep_first", 1)]
    assert m.state_specs[(2, "right.conv")][0] == (0, 24) and m.state_specs[(4, "right.conv")][0] == (6, 80)
    names = {s.name for s in m.param_specs()}
    assert "l2.norm1" in names and "l2.norm2" not in names and "l2.mlp.router" not in names and "l3.mix.q" not in names


def test_band_frequencies_are_pinned_to_hand_values():
    """dims 8, base 10000, factor 4, low 1, high 4, original 64: f = 1, 0.1, 0.01, 0.001; wavelengths 6.28, 62.8, 628, 6283.
    Kept below 16, divided by 4 above 64, between: s = (64 / 62.83 - 1) / 3 = 0.0061977, f = (1 - s) 0.025 + s 0.1."""
    f = plain.band_frequencies(8, 10000.0, tm.bands(4.0, 64))
    s = (64.0 / (2 * math.pi / 0.1) - 1.0) / 3.0
    want = [1.0, (1 - s) * 0.025 + s * 0.1, 0.0025, 0.00025]
    assert max(abs(float(a) - b) / b for a, b in zip(f, want)) < 1e-12 and abs(want[1] - 0.02546483) < 1e-7
    assert torch.equal(plain.band_frequencies(8, 10000.0), torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=F))


def test_yarn_frequencies_are_pinned_to_hand_values():
    """dims 8, base 10000, factor 2, original 64, fast 4, slow 1: the pair index that turns t times in 64 positions is
    8 ln(64 / (2 pi t)) / (2 ln 10000) = 0.4059 (t = 4) and 1.0080 (t = 1): lo = 0, hi = 2; ramps 0, 0.5, 1, 1; the
    magnitude is 0.1 ln 2 + 1."""
    f, mag = plain.yarn_frequencies(8, 10000.0, tm.yarn(2.0, 64, fast=4.0, slow=1.0))
    want = [1.0, 0.5 * 0.05 + 0.5 * 0.1, 0.005, 0.0005]
    assert max(abs(float(a) - b) / b for a, b in zip(f, want)) < 1e-12
    assert abs(mag - 1.0693147) < 1e-7
    assert abs(8 * math.log(64 / (2 * math.pi * 4)) / (2 * math.log(10000.0)) - 0.4059) < 1e-4
    # a ramp whose ends meet: the divisor is held at 0.001, every later pair is scaled whole
    f, _ = plain.yarn_frequencies(8, 10000.0, tm.yarn(2.0, 64, fast=1.0, slow=1.0))
    assert abs(float(f[0]) - 1.0) < 1e-12 and abs(float(f[2]) - 0.005) < 1e-12


def test_engine_and_plain_frequencies_agree():
    from hipinfer_b200.kernels import ops

    for dims, base, sc in ((64, 200000.0, tm.bands(6.0, 2048)), (16, 100.0, tm.bands(3.0, 50, low=2.0, high=5.0)), (6, 10000.0, None)):
        f, mag = ops.rope_frequencies(dims, base, dict(sc, kind="wavelength_bands") if sc else None)
        assert mag == 1.0 and float((f - plain.band_frequencies(dims, base, sc)).abs().max()) < 1e-15
    for dims, base, sc in ((32, 10000.0, tm.yarn(3.0, 256)), (8, 100.0, tm.yarn(40.0, 16, fast=4.0, slow=2.0)), (64, 1e6, tm.yarn(8.0, 4096))):
        f, mag = ops.rope_frequencies(dims, base, dict(sc, kind="yarn"))
        pf, pm = plain.yarn_frequencies(dims, base, sc)
        assert abs(mag - pm) < 1e-15 and float((f - pf).abs().max()) < 1e-15


def test_rotation_pairings():
    t = rnd(3, 2, 8, seed=1)
    pos = torch.tensor([0, 5, 9])
    f = plain.band_frequencies(4, 100.0)
    a, b = plain.rotate(t, pos, f, 4, "interleaved"), plain.rotate(t, pos, f, 4, "half", 1.5)
    assert torch.equal(a[0], t[0]) and torch.equal(a[..., 4:], t[..., 4:]) and torch.equal(b[..., 4:], t[..., 4:])
    ang = 5 * float(f[1])
    assert abs(float(a[1, 0, 2]) - (float(t[1, 0, 2]) * math.cos(ang) - float(t[1, 0, 3]) * math.sin(ang))) < 1e-12
    assert abs(float(b[1, 0, 1]) - 1.5 * (float(t[1, 0, 1]) * math.cos(ang) - float(t[1, 0, 3]) * math.sin(ang))) < 1e-12
    assert abs(float(b[1, 0, 3]) - 1.5 * (float(t[1, 0, 3]) * math.cos(ang) + float(t[1, 0, 1]) * math.sin(ang))) < 1e-12


def test_selective_scan_is_its_unrolled_sum():
    T, I, N = 9, 3, 4
    x, B, C = rnd(T, I, seed=1), rnd(T, N, seed=2), rnd(T, N, seed=3)
    dt, A_log, D = plain.softplus(rnd(T, I, seed=4)), rnd(I, N, seed=5), rnd(I, seed=6)
    y = plain.selective_scan(x, dt, B, C, A_log, D)
    A = -torch.exp(A_log)
    for t in (0, 4, 8):
        for c in range(I):
            want = D[c] * x[t, c]
            for s in range(t + 1):
                decay = torch.exp(A[c] * dt[s + 1:t + 1, c].sum())
                want = want + (decay * dt[s, c] * x[s, c] * B[s] * C[t]).sum()
            assert abs(float(y[t, c] - want)) < 1e-10


def test_convolution_sees_zeros_before_the_sequence():
    x, w, b = rnd(6, 2, seed=1), rnd(2, 3, seed=2), rnd(2, seed=3)
    y = plain.causal_conv(x, w, b)
    assert torch.allclose(y[0], b + x[0] * w[:, 2]) and torch.allclose(y[2], b + x[0] * w[:, 0] + x[1] * w[:, 1] + x[2] * w[:, 2])


def test_the_sink_joins_the_denominator_once_and_the_window_has_hard_edges():
    s = torch.tensor([[1.0, 2.0, 0.5]], dtype=F)
    seen = torch.tensor([[True, True, False]])
    w = plain.softmax_with_sink(s, seen, 0.7)
    den = math.exp(1.0) + math.exp(2.0) + math.exp(0.7)
    assert torch.allclose(w, torch.tensor([[math.exp(1.0) / den, math.exp(2.0) / den, 0.0]], dtype=F))
    assert abs(float(plain.softmax_with_sink(s, seen).sum()) - 1.0) < 1e-12
    seen = plain.visible(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True] and seen[1].tolist() == [True, True, False, False, False, False]
    assert plain.visible(4).tolist() == torch.tril(torch.ones(4, 4)).bool().tolist()


def test_router_chooses_by_logit_and_weighs_by_softmax_over_the_chosen():
    h = torch.eye(3, dtype=F)
    router = torch.tensor([[1.0, 0.0, 2.0], [3.0, 0.0, 2.0], [2.0, 0.0, 0.0], [0.5, 0.0, 2.0]], dtype=F)
    bias = torch.tensor([0.0, 0.0, 0.0, 0.1], dtype=F)
    chosen, weight = plain.route(h, router, bias, 2)
    assert chosen.tolist() == [[1, 2], [3, 0], [3, 0]]        # row 1: logits 0, 0, 0, 0.1; ties go to the lower index
    assert torch.allclose(weight[0], torch.softmax(torch.tensor([3.0, 2.0], dtype=F), 0))
    assert torch.allclose(weight[2], torch.softmax(torch.tensor([2.1, 2.0], dtype=F), 0))


def test_a_layer_that_runs_again_uses_the_same_tensors():
    """Layers 1 and 3 of model A have no tensors of their own: the plain logits change when layer 0's tensors change, and
    a model with copies of those tensors under l1 and l3 in place of the references gives the same logits."""
    w = tm.draw_weights(tm.A, 3, torch.float32)
    toks = list(range(20))
    ref = plain.forward(tm.A, w, toks)
    flat = json.loads(json.dumps(tm.A))
    for i in (1, 3):
        flat["layers"][i].pop("weights_of")
    w2 = dict(w)
    for k, v in w.items():
        if k.startswith("l0."):
            w2["l1." + k[3:]] = v
            w2["l3." + k[3:]] = v
    assert torch.equal(plain.forward(flat, w2, toks), ref)
    w2["l3.mix.left.o"] = w2["l3.mix.left.o"] * 1.5
    assert not torch.equal(plain.forward(flat, w2, toks), ref)
