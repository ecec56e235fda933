"""The Mavinex design through the engine: the step function, the cache and state manager, trace replay, the scheduler
and the Python entry point, in 32-bit and in bfloat16, against the plain implementation of tests/plain_mavinex.py, on
four small configurations of the tests' own (tests/mavinex_models.py)."""
import math

import pytest
import torch

import tiny
import mavinex_models as tm

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [1, 2, 5, 40, 90, 130, 33, 64], "b": [3, 1, 70, 16, 17, 100, 48, 2], "c": [600, 7, 129, 64, 200, 65, 1, 150],
           "d": [120, 31, 57, 2, 64, 90, 16, 100]}
TOL = {"float32": 3e-5, "bfloat16": 2.5e-2}


def _close(got, ref, dtype, what, sens=None):
    """32-bit: every position within the bound. bfloat16: a position's bound is the general one or, where that is larger,
    six times the sensitivity to rounding of the position and its two neighbours on either side (tests/mavinex_models.py: a
    norm that divides by nearly nothing, sums that cancel; the estimate is one draw of rounding noise, and what makes a
    position sensitive also holds a token earlier or later through the recurrent state); up to 3 % of a request's positions
    (at least one) may lie over their bound, none over four times."""
    scale = float(ref.abs().max())
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    bad = (got.double() - ref.double()).abs().amax(-1) / scale
    bound = torch.full_like(bad, TOL[dtype])
    if dtype == "bfloat16" and sens is not None:
        near = torch.nn.functional.max_pool1d(sens[:bad.shape[0]].double()[None, None], 5, 1, 2)[0, 0]
        bound = torch.maximum(bound, 6.0 * near)
    over = int((bad > bound).sum())
    allowed = 0 if dtype == "float32" else max(1, (3 * got.shape[0]) // 100)
    if over > allowed or bool((bad > 4 * bound).any()):
        worst = int((bad / bound).argmax())
        raise AssertionError(f"{what}: {over} of {got.shape[0]} positions over their bound (allowed {allowed}), the worst "
                             f"{float(bad[worst]):.3e} at {worst} (bound {float(bound[worst]):.1e}); first wrong position "
                             f"{int((bad > bound).nonzero()[0])}")


def _plain(cfg, w, reqs, dtype):
    """({id: plain logits}, {id: sensitivity per position, bfloat16 only})"""
    ref = {rid: tm.PlainMavinex(cfg, w).forward(toks) for rid, toks in reqs.items()}
    sens = {rid: tm.sensitivity(cfg, w, toks, ref[rid]) if dtype == "bfloat16" else None for rid, toks in reqs.items()}
    return ref, sens


@pytest.fixture(scope="module", params=[(m, d) for m in ("a", "b", "c", "d") for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    from hipinfer_b200.engine.runner import ModelRunner

    which, dtype = request.param
    folder, cfg, w = tm.make_folder(tmp_path_factory.mktemp(f"mavinex_{which}_{dtype}"), which, seed=7,
                                    dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    requests = {f"r{i}": tiny.random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(LENGTHS[which])}
    ref, sens = _plain(cfg, w, requests, dtype)
    longest = -(-max(LENGTHS[which]) // 64) * 64
    # pages for four live requests of the longest kind and four state slots: both are used again
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=4 * longest // 16, max_num_seqs=4)
    yield dict(which=which, dtype=dtype, folder=folder, cfg=cfg, weights=w, requests=requests, ref=ref, sens=sens, runner=runner,
               stepper=tiny.RunnerStepper(runner))
    assert not runner.live_requests()
    runner.cache.check()
    assert runner.cache.free_pages() == [p.num_pages for p in runner.cache.pools]


def _check(setup, plan, what):
    got = tiny.run_plan(setup["stepper"], setup["requests"], plan)
    for rid, ref in setup["ref"].items():
        _close(got[rid], ref, setup["dtype"], f"{what} {setup['which']} {setup['dtype']} {rid}", setup["sens"][rid])
    return got


def test_whole_prompts(setup):
    _check(setup, tiny.plan_whole(setup["requests"]), "whole")


def test_whole_prompts_with_the_recurrence_in_short_pieces(setup, monkeypatch):
    """Prompts of a few dozen tokens already run the selective recurrence in pieces (of 8 tokens), in a batch of unequal
    requests too; the states the pieces leave are the ones that the single tokens after them start from."""
    from hipinfer_b200.kernels import ops

    monkeypatch.setattr(ops, "SEL_PIECE_TOKENS", 8)
    _check(setup, tiny.plan_whole(setup["requests"]), "whole in pieces")
    _check(setup, tiny.plan_tail_decode(setup["requests"], 5), "pieces then single tokens")
    _check(setup, tiny.plan_mixed(setup["requests"], 11), "mixed in pieces")


def test_last_tokens_one_by_one(setup):
    _check(setup, tiny.plan_tail_decode(setup["requests"], 48), "tail")


def test_every_token_alone(setup):
    short = {r: t for r, t in setup["requests"].items() if len(t) <= 70}
    got = tiny.run_plan(setup["stepper"], short, [[(r, 1)] for r, t in short.items() for _ in t])
    for rid in short:
        _close(got[rid], setup["ref"][rid], setup["dtype"], f"token by token {rid}", setup["sens"][rid])


@pytest.mark.parametrize("sizes", [(7, 2, 16, 3, 2, 33, 5, 2, 64, 1, 9), (2,), (15, 17, 1, 31), (64, 2, 63, 66)])
def test_portions(setup, sizes):
    _check(setup, tiny.plan_portions(setup["requests"], sizes), f"portions {sizes}")


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mixed_batches(setup, seed):
    _check(setup, tiny.plan_mixed(setup["requests"], seed), f"mixed{seed}")


def test_mixed_batches_with_long_portions(setup):
    _check(setup, tiny.plan_mixed_long(setup["requests"], 1, long=(65, 140)), "mixed long")


def test_a_request_in_a_batch_equals_the_request_alone(setup):
    """Beyond rounding nothing of a row depends on the batch (a routed layer runs single rows and sorted portions on
    different kernels, so the sums' order may differ)."""
    reqs = setup["requests"]
    alone = tiny.run_plan(setup["stepper"], reqs, tiny.plan_whole(reqs))
    ids = list(reqs)
    together = tiny.run_plan(setup["stepper"], reqs, [[(r, len(reqs[r])) for r in ids[:4]], [(r, len(reqs[r])) for r in ids[4:]]])
    tol = 1e-5 if setup["dtype"] == "float32" else 2e-2
    for rid in ids:
        scale = float(alone[rid].abs().max())
        assert float((alone[rid] - together[rid]).abs().max()) <= tol * scale, rid


def test_a_state_slot_and_pages_used_again_start_clean(setup):
    """The same request after others have used and returned every slot and page gives the same bits as on a fresh engine
    state (the recurrent state is zeroed at admission; pages hold what the request itself wrote)."""
    reqs, st = setup["requests"], setup["stepper"]
    first = tiny.run_plan(st, {"r3": reqs["r3"]}, [[("r3", len(reqs["r3"]))]])["r3"]
    others = {r: reqs[r] for r in ("r4", "r5", "r0", "r2", "r7")}
    tiny.run_plan(st, others, tiny.plan_mixed(others, 5))
    again = tiny.run_plan(st, {"r3": reqs["r3"]}, [[("r3", len(reqs["r3"]))]])["r3"]
    assert torch.equal(first, again)


def test_long_decoding_past_every_window(setup):
    """A short prompt, then hundreds of single tokens: windows pass over decoded tokens, pages are given back while the
    request runs, decode-only steps replay from CUDA graphs."""
    cfg = setup["cfg"]
    n = min(cfg["max_positions"], 330 if setup["which"] != "c" else 560)
    toks = tiny.random_tokens(n, cfg["vocab"], 77)
    ref, sens = _plain(cfg, setup["weights"], {"long": toks}, setup["dtype"])
    got = tiny.run_plan(setup["stepper"], {"long": toks}, [[("long", 6)]] + [[("long", 1)]] * (n - 6))["long"]
    _close(got, ref["long"], setup["dtype"], "long decoding", sens["long"])
    r = setup["runner"]
    assert r.steps_run > 0


def test_two_requests_decode_together_through_graph_replays(setup):
    reqs = setup["requests"]
    a, b = "r4", "r5"
    ha, hb = len(reqs[a]) // 2, len(reqs[b]) // 3 + 1
    plan = [[(a, ha), (b, hb)]] + [[(a, 1), (b, 1)]] * min(len(reqs[a]) - ha, len(reqs[b]) - hb)
    fed_a, fed_b = ha + len(plan) - 1, hb + len(plan) - 1
    sub = {a: reqs[a][:fed_a], b: reqs[b][:fed_b]}
    got = tiny.run_plan(setup["stepper"], sub, plan)
    _close(got[a], setup["ref"][a][:fed_a], setup["dtype"], "pair a", setup["sens"][a])
    _close(got[b], setup["ref"][b][:fed_b], setup["dtype"], "pair b", setup["sens"][b])


def test_trace_replay_program(setup, tmp_path):
    """bin/trace_run as a child process on the same folder: portions, single tokens, a batch, few pages."""
    reqs = {r: setup["requests"][r] for r in ("r2", "r3", "r6", "r7")}
    tr = tiny.TraceRun(setup["folder"], setup["dtype"], tmp_path / "out", 2 * 64 * -(-max(len(t) for t in reqs.values()) // 64))
    try:
        got = tiny.run_plan(tr, reqs, tiny.plan_mixed(reqs, 3, max_live=2))
    finally:
        tr.close()
    for rid in reqs:
        _close(got[rid], setup["ref"][rid], setup["dtype"], f"trace_run {rid}", setup["sens"][rid])


def test_greedy_generation_through_the_entry_point_and_scheduler(setup):
    """Engine.generate and three requests through the scheduler at once, against greedy decoding with the plain model; a
    different token is accepted only where the plain logits nearly tie."""
    from hipinfer_b200 import Engine

    cfg, n_new = setup["cfg"], 12
    model = tm.PlainMavinex(cfg, setup["weights"])

    def plain_greedy(prompt):
        model.reset()
        logits = model.forward(prompt)[-1]
        out, steps = [], []
        for _ in range(n_new):
            steps.append(logits)
            out.append(int(logits.argmax()))
            logits = model.forward([out[-1]])[-1]
        return out, steps

    def same(got, want, steps, what):
        for i, (g, w) in enumerate(zip(got, want)):
            if g != w:
                top = torch.topk(steps[i], 2).values
                gap = float(top[0] - top[1]) / float(steps[i].abs().max())
                assert gap < (0.02 if setup["dtype"] == "bfloat16" else 1e-3), f"{what}: token {i} is {g}, plain {w} (gap {gap:.5f})"
                return
        assert len(got) == len(want)

    eng = Engine(setup["folder"], dtype=setup["dtype"], max_batch=3, max_seq=min(256, cfg["max_positions"]), max_prefill=32)
    try:
        prompts = [tiny.random_tokens(n, cfg["vocab"], 900 + n) for n in (9, 70, 33)]
        want = [plain_greedy(p) for p in prompts]
        same(eng.generate(prompts[0], n_new), want[0][0], want[0][1], "generate")
        ids = [eng.add_request(p, n_new) for p in prompts]        # portions of 32 tokens beside decoding requests
        done = eng.run()
        for i, rid in enumerate(ids):
            same(done[rid], want[i][0], want[i][1], f"scheduler request {i}")
    finally:
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layers", ["side by side only", "latent only", "one layer", "no feed-forward", "one layer six times"])
def test_models_of_one_kind_of_layer(layers, dtype, tmp_path):
    """A model of side-by-side layers only, one without any state (latent attention only, with and without a window), a
    single layer, layers without feed-forward, and one layer's tensors run six times: whole, in portions, token by token
    and mixed."""
    from hipinfer_b200.engine.runner import ModelRunner

    one = tm.parallel(tm.attention(2, 1, 16, 16, window=20), tm.scan(32, 4, 4), mlp=tm.moe(32, 4, 2))
    cfg = tm.model(90, 64, {
        "side by side only": [tm.parallel(tm.attention(2, 2, 32, 16, window=30, scaling=tm.bands(2.0, 16)), tm.scan(96, 16, 4), mlp=tm.moe(48, 2, 1)),
                              tm.parallel(tm.attention(4, 1, 16, 16), tm.scan(64, 8, 8, conv=3), mlp=tm.moe(32, 4, 2))],
        "latent only": [tm.latent(2, 16, 16, 16, 32, window=30, scaling=tm.yarn(2.0, 16), mlp=tm.moe(32, 2, 1)),
                        tm.latent(4, 8, 4, 8, 48, mlp=tm.moe(32, 3, 2))],
        "one layer": [tm.latent(4, 16, 16, 16, 32, window=40, mlp=tm.moe(32, 2, 2))],
        "no feed-forward": [tm.parallel(tm.attention(2, 1, 16, 32, window=12), tm.scan(32, 16, 2)), tm.latent(2, 16, 8, 16, 24, window=12),
                            tm.parallel(tm.attention(1, 1, 32, 8), tm.scan(16, 8, 4, conv=2))],
        "one layer six times": [one] + [tm.repeat(one, 0)] * 5}[layers],
        alpha={"side by side only": 2.0, "latent only": 1.0, "one layer": 0.3, "no feed-forward": 1.5, "one layer six times": 2.5}[layers],
        embed_scale=4.0, max_positions=200)
    folder, cfg, w = tm.make_folder(tmp_path / "m", cfg, seed=3, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    reqs = {"a": tiny.random_tokens(150, 90, 1), "b": tiny.random_tokens(37, 90, 2)}
    ref, sens = _plain(cfg, w, reqs, dtype)
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=24, max_num_seqs=2)
    st = tiny.RunnerStepper(runner)
    for plan in (tiny.plan_whole(reqs), tiny.plan_portions(reqs, (5, 2, 40, 1, 17)), tiny.plan_tail_decode(reqs, 20),
                 tiny.plan_mixed(reqs, 4, max_live=2)):
        got = tiny.run_plan(st, reqs, plan)
        for rid in reqs:
            _close(got[rid], ref[rid], dtype, f"{layers} {rid}", sens[rid])
    assert not runner.live_requests()


def test_pages_behind_the_window_are_given_back(tmp_path):
    """A latent layer and an attention layer with windows of 40 keep caches of 128 tokens of pages each: a request of 300
    tokens runs through them, in portions and token by token, because the pages that no later query sees return to the
    pool on the way."""
    from hipinfer_b200.engine.runner import ModelRunner

    cfg = tm.model(90, 64, [tm.latent(2, 16, 16, 16, 32, window=40, mlp=tm.moe(48, 2, 1)),
                            tm.parallel(tm.attention(2, 1, 16, 16, window=40), tm.scan(32, 8, 4)),
                            tm.latent(2, 16, 16, 16, 32, window=40)], alpha=2.0, max_positions=400)
    folder, cfg, w = tm.make_folder(tmp_path / "m", cfg, seed=5, dtype=torch.float32)
    toks = tiny.random_tokens(300, 90, 4)
    ref = tm.PlainMavinex(cfg, w).forward(toks)
    runner = ModelRunner.from_folder(folder, dtype="float32", page_size=16, num_pages=8, max_num_seqs=1)     # 128 tokens of pages
    got = tiny.run_plan(tiny.RunnerStepper(runner), {"x": toks}, [[("x", 50)], [("x", 30)]] + [[("x", 1)]] * 40 + [[("x", 60)]] * 3)
    _close(got["x"], ref, "float32", "300 tokens through 128 tokens of pages")
    assert not runner.live_requests()


def _random_config(seed):
    """A configuration drawn from sizes that resemble real layers in the small: both kinds of layer, with and without a
    feed-forward, in a random order, some of them run again with the tensors of an earlier one."""
    import random

    rng = random.Random(seed)
    pick = rng.choice
    width = pick([64, 96, 128, 160, 192, 256])
    kinds = ["latent", "parallel"] + [pick(["latent", "parallel"]) for _ in range(rng.randint(1, 3))]
    rng.shuffle(kinds)
    layers = []
    for kind in kinds:
        e = pick([2, 4, 8, 16])
        mlp = pick([None, tm.moe(pick([32, 64, 96, 128]), e, pick([t for t in (1, 2, 4) if t <= e]))])
        window = pick([None, 1, 16, 33, 64, 96, 128, 1000])
        if kind == "latent":
            rd = pick([8, 16, 32, 64])
            layers.append(tm.latent(pick([1, 2, 3, 4, 6, 8]), pick([16, 32, 48, 64, 96, 128]), rd, pick([16, 32, 48, 64, 96, 128]),
                                    pick([32, 64, 96, 128, 192, 256]), window=window, mlp=mlp, base=pick([100.0, 10000.0, 1000000.0]),
                                    scaling=pick([None, tm.yarn(pick([2.0, 8.0, 40.0]), pick([16, 64, 256]), pick([32.0, 4.0]), pick([1.0, 2.0]))])))
        else:
            kv = pick([1, 2, 4])
            dim = pick([16, 32, 64, 80, 128])
            layers.append(tm.parallel(
                tm.attention(kv * pick([1, 2, 3]), kv, dim, pick([16, 32, 64, 80, 128]), window=window, rot_dims=pick([dim, dim // 2, 0]),
                             base=pick([100.0, 10000.0, 500000.0]), scaling=pick([None, tm.bands(pick([2.0, 8.0, 32.0]), pick([16, 64, 256]))])),
                tm.scan(pick([32, 64, 96, 160, 256]), pick([4, 8, 16, 24, 64]), pick([1, 4, 8, 12, 16]), conv=pick([2, 3, 4])), mlp=mlp))
    for i in range(len(layers)):
        if rng.random() < 0.4:
            layers.insert(rng.randint(i + 1, len(layers)), tm.repeat(layers[i], i)) if layers[i].get("weights_of") is None and \
                not any(L.get("weights_of") is not None and L["weights_of"] >= i for L in layers) else None
    return tm.model(pick([64, 97, 300, 576]), width, layers, alpha=pick([1.0, 0.5, 2.0, 3.0]), embed_scale=pick([1.0, 8.0, 16.0]),
                    eps=pick([1e-5, 1e-6]), max_positions=512)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(12)))
def test_random_configurations(seed, dtype, tmp_path):
    """A dozen configurations drawn at random (sizes on either side of every kernel's size steps): whole prompts, the last
    tokens one by one, portions, and a mixed batch, against the plain model."""
    from hipinfer_b200.engine.runner import ModelRunner

    cfg = _random_config(seed)
    folder, cfg, w = tm.make_folder(tmp_path / "m", cfg, seed=seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    reqs = {"a": tiny.random_tokens(170, cfg["vocab"], 1), "b": tiny.random_tokens(41, cfg["vocab"], 2), "c": tiny.random_tokens(1, cfg["vocab"], 3)}
    ref, sens = _plain(cfg, w, reqs, dtype)
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=30, max_num_seqs=3)
    st = tiny.RunnerStepper(runner)
    for plan in (tiny.plan_whole(reqs), tiny.plan_tail_decode(reqs, 24), tiny.plan_portions(reqs, (17, 2, 40, 1, 33)),
                 tiny.plan_mixed(reqs, seed, max_live=3)):
        got = tiny.run_plan(st, reqs, plan)
        for rid in reqs:
            _close(got[rid], ref[rid], dtype, f"random configuration {seed} {rid}", sens[rid])
    assert not runner.live_requests()
