"""Each mechanism of the Runopel design alone: the kernel against the plain function of tests/plain_runopel.py, in 32-bit
and in bfloat16, at sizes the vectorised paths take and at sizes they do not, with inputs made so that a fault shows (a
token far back that a slow decay still carries, a key one position outside the window with a huge score, scores that
tie, values beyond the limits)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_runopel as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.2e-2}


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, what="", tol=None):
    got, want = got.double().cpu(), want.double()
    err, ref = float((got - want).abs().max()), float(want.abs().max())
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    assert err <= (tol or TOL[dtype]) * ref, f"{what}: {err:.3e} > {tol or TOL[dtype]:.0e} * {ref:.3e}"


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def batch_of(lengths, ctx=None, slots=None):
    """What the kernels read of a step: requests of `lengths` rows each, after `ctx` cached tokens."""
    ctx = ctx or [0] * len(lengths)
    starts = [sum(lengths[:r]) for r in range(len(lengths))]
    return SimpleNamespace(n_requests=len(lengths), max_q_len=max(lengths), req_q_start=i32(starts), req_q_len=i32(lengths),
                           req_ctx_len=i32(ctx), req_state_slot=i32(slots or range(len(lengths))), h_q_len=list(lengths),
                           h_ctx_len=list(ctx), h_q_start=starts,
                           row_request=i32(r for r, n in enumerate(lengths) for _ in range(n)),
                           positions=i32(c + i for c, n in zip(ctx, lengths) for i in range(n)),
                           max_pos=max(c + n for c, n in zip(ctx, lengths)) - 1)


# ------------------------------------------------------------------------------------------ residual streams
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,W", [(1, 50), (2, 176), (3, 64), (8, 1000), (1, 128), (2, 2048), (4, 4096), (2, 4100)])
def test_streams_read_norm_and_write_back(dtype, S, W):
    from hipinfer_b200.kernels import ops

    T, eps, m = 7, 1e-5, 0.6
    x = rnd(T, S, W, seed=1) * 2 + 0.5
    a, b, M = rnd(S, seed=2) + 0.5, rnd(S, seed=3) + 1.0, torch.eye(S) + 0.4 * rnd(S, S, seed=4)
    w, w2, y = (1 + 0.3 * rnd(W, seed=5)).to(dtype), (1 + 0.3 * rnd(W, seed=6)).to(dtype), rnd(T, W, seed=7)
    xd = x.reshape(T, S * W).to(DEV)
    out = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.streams_norm(xd, a.to(DEV), w.to(DEV), eps, out, S)
    u = torch.einsum("s,tsw->tw", a.double(), x.double())
    close(out, plain.rms_div(u, eps) * w.double(), dtype, "read + norm")
    rows = [5, 0, 3]
    out3 = torch.empty(3, W, dtype=dtype, device=DEV)
    ops.streams_norm(xd, None, w.to(DEV), eps, out3, S, i32(rows))
    close(out3, plain.rms_div(x.double().sum(1)[rows], eps) * w.double(), dtype, "plain sum of chosen rows")
    # the write-back alone, and fused with the next reader's norm: the same streams bit for bit
    new = torch.einsum("sk,tsw->tkw", M.double(), x.double()) + m * b.double()[None, :, None] * y.double()[:, None, :]
    x1, x2 = xd.clone(), xd.clone()
    ops.streams_update(x1, y.to(DEV), b.to(DEV), M.contiguous().to(DEV), m, S)
    close(x1.view(T, S, W), new, torch.float32, "write-back")
    nxt = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.streams_update(x2, y.to(DEV), b.to(DEV), M.contiguous().to(DEV), m, S, a.to(DEV), w2.to(DEV), eps, nxt)
    assert torch.equal(x1, x2)
    close(nxt, plain.rms_div(torch.einsum("s,tsw->tw", a.double(), new), eps) * w2.double(), dtype, "fused next norm")
    # without learned weights: x + m y
    x3 = xd.clone()
    ops.streams_update(x3, y.to(DEV), None, None, m, S)
    close(x3.view(T, S, W), x.double() + m * y.double()[:, None, :], torch.float32, "plain residual")
    xs = torch.empty(T, S * W, dtype=torch.float32, device=DEV)
    ops.streams_expand(y.to(DEV), xs, S)
    assert torch.equal(xs.view(T, S, W).cpu(), y[:, None, :].expand(T, S, W))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I,group", [(64, 16), (56, 56), (7, 7), (4096, 16), (30, 6)])
def test_gate_with_biases_and_limits(dtype, I, group):
    from hipinfer_b200.kernels import ops

    L = 1.25
    g, u = rnd(6, I, seed=1) * 3, rnd(6, I, seed=2) * 3                       # a good part lies beyond the limits
    bg, bu = rnd(I, seed=3).to(dtype), rnd(I, seed=4).to(dtype)
    il = lambda p, q, n: torch.stack([p.reshape(n, I // group, group), q.reshape(n, I // group, group)], 2).reshape(n, 2 * I)
    out = torch.empty(6, I, dtype=dtype, device=DEV)
    ops.glu_bias(il(g, u, 6).to(DEV), il(bg[None], bu[None], 1)[0].contiguous().to(DEV), out, group, "clamped_sigmoid", L, 1.702)
    gg = torch.clamp(g.double() + bg.double(), max=L)
    uu = torch.clamp(u.double() + bu.double(), min=-L, max=L)
    close(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), dtype)
    assert float((g + bg.float() < -L).float().mean()) > 0.05                 # the gate has no lower limit: such values are in the test


# ------------------------------------------------------------------------------------------ the state-space mixer
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,K", [(40, 4), (130, 1), (7, 2), (300, 7), (33, 8), (50, 9), (20, 16)])
def test_causal_convolution_carries_its_last_inputs(dtype, C, K):
    """Two requests, cut into portions of 1 to 70 rows (also shorter than the filter): every portion continues from the
    carried inputs of the one before; slots are used in another order than the requests."""
    from hipinfer_b200.kernels import ops

    lens, off = [150, 9], 3
    w, b = (rnd(C, K, seed=1) * 0.6).to(dtype), rnd(C, seed=2).to(dtype)
    xs = [rnd(n, off + C + 2, seed=10 + r) for r, n in enumerate(lens)]
    want = [torch.nn.functional.silu(plain.causal_conv(x[:, off:off + C].double(), w.double(), b.double())) for x in xs]
    carried = torch.zeros(4, K - 1, C, dtype=torch.float32, device=DEV)
    cuts = {0: [1, 1, 2, 70, 1, 5, 64, 6], 1: [2, 1, 1, 5]}
    fed, got = [0, 0], [[], []]
    while any(cuts.values()):
        live = [r for r in (0, 1) if cuts[r]]
        ns = [cuts[r].pop(0) for r in live]
        bt = batch_of(ns, slots=[3 - 2 * r for r in live])
        rows = torch.cat([xs[r][fed[r]:fed[r] + n] for r, n in zip(live, ns)]).to(DEV)
        out = torch.empty(rows.shape[0], C, dtype=torch.float32, device=DEV)
        ops.ssd_conv(rows, off, w.to(DEV), b.to(DEV), carried, bt, out)
        o = 0
        for r, n in zip(live, ns):
            got[r].append(out[o:o + n].cpu())
            fed[r] += n
            o += n
    for r in (0, 1):
        close(torch.cat(got[r]), want[r], torch.float32, f"request {r}")


@pytest.mark.parametrize("H,P,N,G", [(4, 16, 8, 2), (3, 6, 7, 1), (2, 64, 128, 1), (6, 40, 56, 3), (1, 128, 16, 1), (2, 10, 5, 2)])
def test_recurrence_against_the_plain_scan(H, P, N, G, monkeypatch):
    """Whole, in portions and token by token, each request in one walk: the same bits (a token's arithmetic does not depend
    on where a portion starts), and the plain scan's values. Head 0 hardly decays and token 0 is huge: it is still there
    300 tokens on."""
    from hipinfer_b200.kernels import ops

    monkeypatch.setattr(ops, "SSD_PIECE_TOKENS", 0)
    T = 320
    x, B, C = rnd(T, H, P, seed=1), rnd(T, G, N, seed=2), rnd(T, G, N, seed=3)
    x[0] *= 30.0
    dt_raw, dt_bias = rnd(T, H, seed=4), rnd(H, seed=5)
    a_log = torch.linspace(-6.0, 1.0, H) if H > 1 else torch.tensor([-6.0])
    d = 1.0 + 0.5 * rnd(H, seed=6)
    want = plain.state_space_scan(x.double(), B.double(), C.double(), plain.softplus(dt_raw.double() + dt_bias.double()),
                                  a_log.double(), d.double(), G).reshape(T, H * P)
    assert float(want[300:, :P].abs().mean()) > 3 * float(want[300:, -P:].abs().mean()) or H == 1     # token 0 shows in head 0
    xbc = torch.cat([x.reshape(T, -1), B.reshape(T, -1), C.reshape(T, -1)], 1).to(DEV)
    wide = torch.cat([rnd(T, 5, seed=7), dt_raw], 1).to(DEV)                   # dt as a view of wider rows
    outs = []
    for cuts in ([T], [1, 2, 15, 16, 17, 64, 100, 105], [1] * 40 + [T - 40]):
        state = torch.zeros(2, H, N, P, dtype=torch.float32, device=DEV)
        y = torch.empty(T, H * P, dtype=torch.float32, device=DEV)
        t = 0
        for n in cuts:
            ops.ssd_scan(xbc[t:t + n], wide[t:t + n, 5:], dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), state, batch_of([n], slots=[1]),
                         y[t:t + n], H, P, N, G)
            t += n
        assert float(state[0].abs().max()) == 0.0
        outs.append(y.cpu())
    close(outs[0], want, torch.float32, "whole", tol=3e-5)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("piece", [4, 16, 64])
@pytest.mark.parametrize("H,P,N,G", [(4, 16, 8, 2), (3, 6, 7, 1), (2, 64, 128, 1), (6, 40, 56, 3)])
def test_recurrence_in_pieces(H, P, N, G, piece, monkeypatch):
    """Long portions in pieces (each from zero, the starting states one after another, each again for y): three requests of
    unequal length in one step, one of a single token, one that ends in the middle of a piece, each after a first portion
    that left a state; against the plain scan and against the walk in one go, outputs and states. Head 0 hardly decays and
    a request's first token is huge, so a starting state that was lost or decayed wrongly shows in every later piece."""
    from hipinfer_b200.kernels import ops

    first, lens = [5, 3, 2], [1, 3 * piece + piece // 2 + 1, 5 * piece]
    total = [a + b for a, b in zip(first, lens)]
    gen = lambda n, sd: (rnd(n, H, P, seed=sd), rnd(n, G, N, seed=sd + 1), rnd(n, G, N, seed=sd + 2), rnd(n, H, seed=sd + 3))
    data = [gen(n, 10 * r) for r, n in enumerate(total)]
    for x, *_ in data:
        x[0] *= 30.0
    dt_bias, d = rnd(H, seed=5), 1.0 + 0.5 * rnd(H, seed=6)
    a_log = torch.linspace(-6.0, 1.0, H)
    want = [plain.state_space_scan(x.double(), B.double(), C.double(), plain.softplus(dtr.double() + dt_bias.double()), a_log.double(),
                                   d.double(), G).reshape(-1, H * P) for x, B, C, dtr in data]
    rows = lambda part: (torch.cat([torch.cat([x.reshape(len(x), -1), B.reshape(len(x), -1), C.reshape(len(x), -1)], 1)[part(r)]
                                    for r, (x, B, C, _) in enumerate(data)]).to(DEV),
                         torch.cat([dtr[part(r)] for r, (*_, dtr) in enumerate(data)]).to(DEV))
    res = {}
    for label, size in (("one walk", 0), ("pieces", piece)):
        monkeypatch.setattr(ops, "SSD_PIECE_TOKENS", size)
        state = torch.zeros(4, H, N, P, dtype=torch.float32, device=DEV)
        ys = []
        for part, ln in ((lambda r: slice(0, first[r]), first), (lambda r: slice(first[r], None), lens)):
            xbc, dtr = rows(part)
            y = torch.empty(sum(ln), H * P, dtype=torch.float32, device=DEV)
            ops.ssd_scan(xbc, dtr, dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), state, batch_of(ln, slots=[3, 0, 2]), y, H, P, N, G)
            ys.append(y.cpu())
        res[label] = (ys[1], state.cpu())
        t = 0
        for r, n in enumerate(lens):
            close(ys[1][t:t + n], want[r][first[r]:], torch.float32, f"{label}, request {r}", tol=3e-5)
            t += n
        assert float(state[1].abs().max()) == 0.0
    close(res["pieces"][0], res["one walk"][0].double(), torch.float32, "pieces against one walk", tol=1e-5)
    close(res["pieces"][1], res["one walk"][1].double(), torch.float32, "states", tol=1e-5)


def test_recurrence_of_two_requests_in_one_step():
    from hipinfer_b200.kernels import ops

    H, P, N, G, lens = 4, 32, 16, 2, [37, 1, 90]
    T = sum(lens)
    x, B, C, dt_raw = rnd(T, H, P, seed=1), rnd(T, G, N, seed=2), rnd(T, G, N, seed=3), rnd(T, H, seed=4)
    dt_bias, a_log, d = rnd(H, seed=5).bfloat16(), (rnd(H, seed=6) - 1).bfloat16(), rnd(H, seed=7).bfloat16()    # 16-bit constants
    xbc = torch.cat([x.reshape(T, -1), B.reshape(T, -1), C.reshape(T, -1)], 1)
    state = torch.zeros(5, H, N, P, dtype=torch.float32, device=DEV)
    y = torch.empty(T, H * P, dtype=torch.float32, device=DEV)
    ops.ssd_scan(xbc.to(DEV), dt_raw.to(DEV), dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), state, batch_of(lens, slots=[4, 0, 2]), y, H, P, N, G)
    t = 0
    for n in lens:
        sl = slice(t, t + n)
        want = plain.state_space_scan(x[sl].double(), B[sl].double(), C[sl].double(), plain.softplus(dt_raw[sl].double() + dt_bias.double()),
                                      a_log.double(), d.double(), G).reshape(n, H * P)
        close(y[sl], want, torch.float32, f"request of {n}", tol=3e-5)
        t += n
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,parts", [(64, 1), (288, 2), (20, 5), (1024, 8), (6, 6)])
def test_gate_then_grouped_norm(dtype, inner, parts):
    from hipinfer_b200.kernels import ops

    T, eps = 5, 1e-5
    y, zz = rnd(T, inner, seed=1) * 2, rnd(T, inner + 9, seed=2) * 2
    w = (1 + 0.3 * rnd(inner, seed=3)).to(dtype)
    out = torch.empty(T, inner, dtype=dtype, device=DEV)
    ops.ssd_gate_norm(y.to(DEV), zz.to(DEV)[:, 4:4 + inner], w.to(DEV), out, parts, eps)
    v = y.double() * plain.silu(zz[:, 4:4 + inner].double())
    want = plain.rms_div(v.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w.double()
    close(out, want, dtype)


# ------------------------------------------------------------------------------------------ routed feed-forward
def _routed(dtype, W, F, E, top, seed=0):
    from hipinfer_b200.parts.registry import BuildContext, build_part
    from hipinfer_b200.parts.spec import PartSpec

    part = build_part("feed_forward", PartSpec("routed", dict(hidden_size=W, experts=E, top=top, expert_size=F)),
                      BuildContext(dtype, DEV, 16, 256), "l0.")
    w = {s.name: (rnd(*s.shape, seed=seed + i) * ((3.0 if s.name.endswith("router") else 1.2) / math.sqrt(s.shape[1]))).to(dtype)
         for i, s in enumerate(part.param_specs())}
    part.load({k: v.to(DEV) for k, v in w.items()})
    return part, {k[len("l0.mlp."):]: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,F,E,top,T", [(64, 32, 5, 2, 9), (50, 22, 3, 3, 7), (128, 96, 16, 4, 200), (160, 64, 6, 1, 130), (48, 40, 1, 1, 5),
                                         (2200, 24, 3, 2, 19), (4360, 16, 2, 1, 11), (2112, 72, 4, 2, 40), (96, 160, 3, 2, 30)])
def test_routed_feed_forward_row_by_row_grouped_and_sorted(dtype, W, F, E, top, T, monkeypatch):
    """The scores multiply the experts' inputs and are not renormalised; single rows one by one (no sorting), single rows
    grouped by expert (rounds of up to 8, 16 and 32 rows, rows wider than a segment of shared memory, experts without a
    row, feature counts that end inside a tile; widths the warp-MMA form takes and widths it does not) and
    portions (sorted by expert, an ordinary product per expert) give the plain sum."""
    from hipinfer_b200.parts import routed_ff

    part, w = _routed(dtype, W, F, E, top)
    h = (rnd(T, W, seed=50) * 1.5).to(dtype)
    want = plain.routed_ff(h.double(), w, E, top)
    for what, q_len, grouped_from in (("one by one", 1, 10 ** 9), ("grouped", 1, 1), ("sorted", T, 1)):
        monkeypatch.setattr(routed_ff, "GROUPED_MIN_PAIRS", grouped_from)
        y = torch.full((T, W), 0.25, dtype=torch.float32, device=DEV)            # the result is ADDED
        part.forward(h.to(DEV), y, SimpleNamespace(max_q_len=q_len, dump=None))
        close(y - 0.25, want, dtype, what)


def test_router_ties_go_to_the_lower_index():
    from hipinfer_b200.kernels import ops

    W, E = 40, 6
    router = rnd(E, W, seed=1)
    router[4] = router[1]                                                          # experts 1 and 4 always tie
    h = rnd(30, W, seed=2)
    expert, score = ops.moe_route(h.to(DEV), router.to(DEV), 3)
    s, chosen = plain.route(h.double(), router.double(), 3)
    assert torch.equal(expert.cpu().long(), chosen)
    close(score, torch.gather(s, 1, chosen), torch.float32)
    e = expert.cpu()
    both = ((e == 1).any(1) & (e == 4).any(1)).nonzero().flatten().tolist()
    assert both and all(e[t].tolist().index(1) < e[t].tolist().index(4) for t in both)


# ------------------------------------------------------------------------------------------ latent attention in a window
def _plain_window_rows(q, keys, values, positions, scale, window):
    """q [T, H, D] rows at `positions` of ONE sequence with keys [n, D'] (shared by the heads, D' >= D) and values [n, E]."""
    n = keys.shape[0]
    j = torch.arange(n)
    out = []
    for t, p in enumerate(positions):
        seen = (j <= p) & ((p - j < window) if window else (j >= 0))
        s = (q[t] @ keys.T) * scale
        s = s.masked_fill(~seen[None], float("-inf"))
        out.append(torch.softmax(s, -1) @ values)
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,Dr,window,ps", [(6, 48, 16, 70, 16), (3, 40, 8, 24, 16), (2, 20, 6, 5, 8), (4, 32, 32, 1, 16), (4, 96, 32, 200, 16)])
def test_single_rows_in_the_latent_s_space_see_exactly_the_window(dtype, H, R, Dr, window, ps):
    """Rows of two requests over one plane of [latent | rotated key part] rows, the values its first columns. The key just
    inside the window has a large score and the key just outside a larger one: one position off in either direction and
    the result is another vector. Pages before the window are given back (-1 in the block table)."""
    from hipinfer_b200.kernels import ops

    Dk, lens = R + Dr, [window + 150, max(window - 3, 2)]
    rows = [(0, lens[0] - 1), (1, lens[1] - 1), (0, window + 40), (0, window - 1), (0, window), (1, 0)]      # (request, position)
    keys = [rnd(n, Dk, seed=3 + r) * 0.5 for r, n in enumerate(lens)]
    q = rnd(len(rows), H, Dk, seed=9) * 0.5
    for t, (r, p) in enumerate(rows):
        u = q[t, 0] / q[t, 0].norm()
        if p - window + 1 >= 0:
            keys[r][p - window + 1] = 6.0 * u                                      # just inside
        if p - window >= 0:
            keys[r][p - window] = 9.0 * u                                          # just outside
    n_pages = [-(-n // ps) for n in lens]
    order = torch.randperm(sum(n_pages) + 2, generator=torch.Generator().manual_seed(1)).tolist()
    plane = torch.zeros(len(order), 1, ps, Dk, dtype=dtype)
    bt = torch.full((2, max(n_pages)), -1, dtype=torch.int32)
    it = iter(order)
    for r in range(2):
        for lp in range(n_pages[r]):
            page = next(it)
            bt[r, lp] = page
            m = min(ps, lens[r] - lp * ps)
            plane[page, 0, :m] = keys[r][lp * ps:lp * ps + m].to(dtype)
    keys = [k.to(dtype).double() for k in keys]
    qd = q.to(dtype)
    batch = SimpleNamespace(block_tables=[bt.to(DEV)], row_request=i32(r for r, _ in rows), positions=i32(p for _, p in rows),
                            req_q_len=i32([1, 1]), h_q_len=[1, 1], max_q_len=1, max_pos=max(lens) - 1, n_requests=2, extra={})
    scale = 1.0 / math.sqrt(Dk)
    want = torch.stack([_plain_window_rows(qd[t:t + 1].double(), keys[r], keys[r][:, :R], [p], scale, window)[0] for t, (r, p) in enumerate(rows)])
    dplane = plane.to(DEV)
    out = torch.empty(len(rows), H * R, dtype=torch.float32, device=DEV)
    ops.attention_masked(qd.reshape(len(rows), H * Dk).to(DEV), dplane, dplane, batch, 0, out, H, 1, Dk, R, ps, scale, "window", window=window)
    close(out.view(len(rows), H, R), want, dtype, "rows")


@pytest.mark.parametrize("H,D,E,window,ctx,n", [(6, 64, 32, 70, 300, 130), (2, 32, 32, 24, 0, 100), (4, 64, 64, 1, 40, 64), (3, 96, 64, 200, 500, 17)])
def test_a_portion_s_rows_see_exactly_the_window(H, D, E, window, ctx, n):
    """The tensor-core kernel over keys and values made from the first kept page on: rows [first, ctx + n) only."""
    from hipinfer_b200.kernels import ops

    if not ops.masked_flash_supported(D, E):
        pytest.skip("sizes the kernel does not take")
    ps = 16
    first = (max(0, ctx - window + 1) // ps) * ps
    total = ctx + n
    keys, values = rnd(total, H, D, seed=1) * 0.5, rnd(total, H, E, seed=2)
    q = rnd(n, H, D, seed=3) * 0.5
    for t in (0, 1, n // 2, n - 1):
        p = ctx + t
        u = q[t, 0] / q[t, 0].norm()
        if p - window + 1 >= 0:
            keys[p - window + 1, 0] = 6.0 * u
        if p - window >= 0:
            keys[p - window, 0] = 9.0 * u
    kb, vb, qb = keys.bfloat16(), values.bfloat16(), q.bfloat16()
    scale = 1.0 / math.sqrt(D)
    want = torch.stack([_plain_window_rows(qb[:, h:h + 1].double(), kb[:, h].double(), vb[:, h].double(), range(ctx, total), scale, window)[:, 0]
                        for h in range(H)], 1)
    batch = batch_of([3, n], ctx=[0, ctx])                                       # the request is the second of the step
    qall = torch.cat([torch.zeros(3, H * D, dtype=torch.bfloat16), qb.reshape(n, H * D)]).to(DEV)
    out = torch.zeros(3 + n, H * E, dtype=torch.bfloat16, device=DEV)
    ops.attention_flash_tokens(qall, kb[first:].reshape(-1, H * D).contiguous().to(DEV), vb[first:].reshape(-1, H * E).contiguous().to(DEV),
                               batch, 1, out, H, H, D, E, scale, window=window, first_pos=first)
    close(out[3:].view(n, H, E), want, torch.bfloat16, "portion")
    assert float(out[:3].float().abs().max()) == 0.0
