"""Each mechanism of the Mavinex design alone: the kernel against the plain function of tests/plain_mavinex.py, in 32-bit
and in bfloat16, at sizes the vectorised paths take and at sizes they do not, with inputs made so that a fault shows (a
token far back that a slow decay still carries, a key one position outside the window with a huge score, a sink that
takes all the weight, logits that tie)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_mavinex as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.2e-2}
F = torch.float64


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


# ------------------------------------------------------------------------------------------ the norm after the sum
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,alpha", [(50, 2.0), (64, 1.0), (176, 0.5), (1000, 3.0), (2048, 2.0), (4100, 1.0)])
def test_residual_sum_then_norm(dtype, W, alpha):
    """x <- rms(alpha x + y) (1 + w), with a plain result, with two side-by-side results that are normed and averaged, with
    both, and without the closing norm (the sum alone); the rounded copy is the new x rounded once."""
    from hipinfer_b200.kernels import ops

    T, eps, pe = 9, 1e-5, 1e-6
    x, y, a, b = rnd(T, W, seed=1) * 3, rnd(T, W, seed=2), rnd(T, W, seed=3) * 5, rnd(T, W, seed=4) * 0.01
    wa, wb, w = (1 + 0.3 * rnd(W, seed=5)).to(dtype), (1 + 0.3 * rnd(W, seed=6)).to(dtype), 0.2 * rnd(W, seed=7)
    pair64 = 0.5 * (plain.rms(a.double(), pe) * wa.double() + plain.rms(b.double(), pe) * wb.double())
    one_plus = (1.0 + w).to(DEV)
    for what, yy, use_pair in (("plain", y, False), ("pair", None, True), ("both", y, True)):
        u = (yy.double() if yy is not None else 0) + (pair64 if use_pair else 0)
        pair = ops.NormedPair(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 0.5, pe) if use_pair else None
        xd, rounded = x.to(DEV).clone(), torch.empty(T, W, dtype=dtype, device=DEV)
        ops.residual_norm(xd, None if yy is None else yy.to(DEV), pair, alpha, one_plus, eps, rounded)
        want = plain.rms(alpha * x.double() + u, eps) * (1.0 + w.double())
        close(xd, want, torch.float32, what)
        assert torch.equal(rounded, xd.to(dtype))
        xd = x.to(DEV).clone()
        ops.residual_norm(xd, None if yy is None else yy.to(DEV), pair, alpha)
        close(xd, alpha * x.double() + u, torch.float32, what + ", the sum alone")


def test_norm_part_with_a_weight_stored_around_zero():
    from hipinfer_b200.parts.registry import BuildContext, build_part
    from hipinfer_b200.parts.spec import PartSpec

    W, eps = 96, 1e-6
    w = (0.3 * rnd(W, seed=1)).bfloat16()
    x = rnd(5, W, seed=2) * 4
    for dtype in (torch.float32, torch.bfloat16):
        part = build_part("norm", PartSpec("rmsnorm", dict(name="n", size=W, eps=eps, one_plus=True)), BuildContext(dtype, DEV))
        part.load({"n": w.to(DEV)})
        close(part.forward(x.to(DEV)), plain.rms(x.double(), eps) * (1.0 + w.double()), dtype)
        close(part.forward(x.to(DEV), rows=i32([3, 0])), (plain.rms(x.double(), eps) * (1.0 + w.double()))[[3, 0]], dtype, "rows")


# ------------------------------------------------------------------------------------------ rotation tables
@pytest.mark.parametrize("dims,base,sc", [(64, 200000.0, dict(kind="wavelength_bands", factor=6.0, low=1.0, high=4.0, original=2048)),
                                          (16, 10000.0, dict(kind="wavelength_bands", factor=4.0, low=2.0, high=8.0, original=40)),
                                          (32, 10000.0, dict(kind="yarn", factor=3.0, original=256, fast=32.0, slow=1.0)),
                                          (8, 100.0, dict(kind="yarn", factor=40.0, original=16, fast=4.0, slow=2.0)),
                                          (12, 5000.0, None)])
def test_rotation_tables_with_rescaled_frequencies(dims, base, sc):
    from hipinfer_b200.kernels import ops

    table = ops.shared_rope_table(dims, base, 3000, DEV, sc).cpu()
    plain_sc = {k: v for k, v in sc.items() if k != "kind"} if sc else None
    if sc and sc["kind"] == "yarn":
        f, mag = plain.yarn_frequencies(dims, base, plain_sc)
    else:
        f, mag = plain.band_frequencies(dims, base, plain_sc), 1.0
    f32 = f.float().double()                                             # the engine keeps the frequencies in 32-bit
    for p in (0, 1, 17, 500, 2999):
        ang = (torch.tensor(float(p)).float() * f32.float()).double()    # and the angle is a 32-bit product
        assert float((table[p, :, 0].double() - torch.cos(ang) * mag).abs().max()) < 2e-7 * mag
        assert float((table[p, :, 1].double() - torch.sin(ang) * mag).abs().max()) < 2e-7 * mag
    if sc:
        assert float((f - plain.band_frequencies(dims, base)).abs().max()) > 0, "the scaling moves no frequency: nothing tested"


# ------------------------------------------------------------------------------------------ attention: row norm, rotation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,rot", [(6, 2, 64, 96, 64), (3, 1, 10, 6, 6), (4, 4, 32, 32, 16), (2, 1, 128, 24, 0)])
def test_whole_row_norm_then_interleaved_rotation_and_cache_write(dtype, H, G, D, E, rot):
    """q and k are divided by the root mean square of their WHOLE rows (all heads at once) and multiplied by a weight per
    column before the rotation of pairs (2i, 2i + 1); a norm per head instead would give other numbers (checked)."""
    from hipinfer_b200.kernels import ops

    T, ps, eps, base = 11, 8, 1e-5, 5000.0
    sc = dict(kind="wavelength_bands", factor=4.0, low=1.0, high=4.0, original=32)
    proj = rnd(T, 3 + H * D + G * D + G * E, seed=1)
    proj[:, 3:3 + D] *= 6.0                                               # one head much larger than the others
    wq, wk = 1 + 0.3 * rnd(H * D, seed=2), 1 + 0.3 * rnd(G * D, seed=3)
    pos = torch.tensor([0, 1, 2, 3, 40, 41, 42, 500, 501, 7, 8])
    slots = torch.randperm(4 * ps, generator=torch.Generator().manual_seed(4))[:T].to(torch.int32)
    table = ops.shared_rope_table(rot, base, 600, DEV, sc)
    q = torch.empty(T, H * D, dtype=dtype, device=DEV)
    kc, vc = torch.zeros(4, G, ps, D, dtype=dtype, device=DEV), torch.zeros(4, G, ps, E, dtype=dtype, device=DEV)
    o = (3, 3 + H * D, 3 + H * D + G * D)
    ops.rope_norm_store(proj.to(DEV), o, pos.to(torch.int32).to(DEV), slots.to(DEV), table, rot, "interleaved", False, 0.0, q, kc, vc,
                        H, G, D, E, ps, row_norm=(wq.to(DEV), wk.to(DEV)), row_norm_eps=eps)
    f = plain.band_frequencies(rot, base, {k: v for k, v in sc.items() if k != "kind"}) if rot else torch.zeros(0, dtype=F)
    p64 = proj.double()
    qn = (plain.rms(p64[:, o[0]:o[1]], eps) * wq.double()).reshape(T, H, D)
    kn = (plain.rms(p64[:, o[1]:o[2]], eps) * wk.double()).reshape(T, G, D)
    want_q, want_k = plain.rotate(qn, pos, f, rot, "interleaved"), plain.rotate(kn, pos, f, rot, "interleaved")
    close(q.view(T, H, D), want_q, dtype, "q", tol=None if dtype == torch.bfloat16 else 1e-4)
    per_head = plain.rms(p64[:, o[0]:o[1]].reshape(T, H, D), eps)
    assert float((per_head - plain.rms(p64[:, o[0]:o[1]], eps).reshape(T, H, D)).abs().max()) > 0.3
    for t in range(T):
        page, off = int(slots[t]) // ps, int(slots[t]) % ps
        close(kc[page, :, off], want_k[t], dtype, f"k of row {t}", tol=None if dtype == torch.bfloat16 else 1e-4)
        close(vc[page, :, off], p64[t, o[2]:].reshape(G, E), dtype, f"v of row {t}")


def _paged_kv(keys, values, ps, dtype, seed):
    """Planes [page, kv head, ps, width] of requests' keys [n, G, D] and values [n, G, E] on shuffled pages, and block tables."""
    n_pages = [-(-k.shape[0] // ps) for k in keys]
    order = torch.randperm(sum(n_pages) + 2, generator=torch.Generator().manual_seed(seed)).tolist()
    G, D, E = keys[0].shape[1], keys[0].shape[2], values[0].shape[2]
    kc, vc = torch.zeros(len(order), G, ps, D, dtype=dtype), torch.zeros(len(order), G, ps, E, dtype=dtype)
    bt = torch.full((len(keys), max(n_pages)), -1, dtype=torch.int32)
    it = iter(order)
    for r in range(len(keys)):
        for lp in range(n_pages[r]):
            page = next(it)
            bt[r, lp] = page
            m = min(ps, keys[r].shape[0] - lp * ps)
            kc[page, :, :m] = keys[r][lp * ps:lp * ps + m].transpose(0, 1).to(dtype)
            vc[page, :, :m] = values[r][lp * ps:lp * ps + m].transpose(0, 1).to(dtype)
    return kc.to(DEV), vc.to(DEV), bt.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,window", [(6, 2, 64, 96, 120), (4, 1, 32, 32, 24), (2, 2, 16, 24, 1), (8, 2, 64, 64, 200), (3, 1, 10, 6, 37)])
def test_grouped_heads_see_exactly_the_window_in_decoding_and_in_a_portion(dtype, H, G, D, E, window):
    """Keys of kv head 0 just inside the window get a large score with head 0's query and the key just outside a larger
    one; values wider or narrower than keys; a gate per element. Single rows over the pages (positions at the window's
    edge, at a page's edge, the first tokens, far behind the window) and the same rows as ONE portion behind a cached
    context: one position off in either direction and the result is another vector."""
    from hipinfer_b200.kernels import ops

    ps, n = 16, window + 170
    ctx = window + 23                                           # the portion is rows [ctx, n)
    keys, vals = rnd(n, G, D, seed=1) * 0.5, rnd(n, G, E, seed=2)
    q = rnd(n, H, D, seed=3) * 0.5
    marked = sorted({0, 1, window - 1, window, window + 1, ctx - 1, ctx, ctx + 1, ctx + 15, ctx + 16, n - 1} & set(range(n)))
    for p in marked[::2]:                                       # every second one, so that marks do not sit in each other's windows
        u = q[p, 0] / q[p, 0].norm()
        if p - window + 1 >= 0:
            keys[p - window + 1, 0] = 6.0 * u
        if p - window >= 0:
            keys[p - window, 0] = 9.0 * u
    gate = rnd(n, 3 + H * E, seed=4) * 2
    kc, vc, bt = _paged_kv([keys], [vals], ps, dtype, 5)
    scale = 1.0 / math.sqrt(D)
    kd, vd, qd = keys.to(dtype).double(), vals.to(dtype).double(), q.to(dtype).double()
    seen = plain.visible(n, window)

    def want_rows(rows):
        out = []
        for p in rows:
            heads = [plain.softmax_with_sink((kd[:, h // (H // G)] @ qd[p, h])[None] * scale, seen[p][None])[0] @ vd[:, h // (H // G)]
                     for h in range(H)]
            out.append(torch.cat(heads) * torch.sigmoid(gate[p, 3:].double()))
        return torch.stack(out)

    # decoding: every marked row alone
    batch = SimpleNamespace(block_tables=[bt], row_request=i32([0] * len(marked)), positions=i32(marked), req_q_len=i32([1]),
                            h_q_len=[1], max_q_len=1, max_pos=n - 1, n_requests=1, extra={})
    out = torch.empty(len(marked), H * E, dtype=dtype, device=DEV)
    ops.attention_masked(q[marked].reshape(len(marked), H * D).to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, scale, "window",
                         window=window, gate=gate[marked].to(DEV), gate_offset=3)
    close(out, want_rows(marked), dtype, "single rows")
    # a portion: rows ctx .. n - 1 in one step behind ctx cached tokens
    rows = list(range(ctx, n))
    batch = batch_of([len(rows)], ctx=[ctx])
    batch.block_tables, batch.extra = [bt], {}
    out = torch.empty(len(rows), H * E, dtype=dtype, device=DEV)
    ops.attention_masked(q[ctx:].reshape(len(rows), H * D).to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, scale, "window",
                         window=window, gate=gate[ctx:].to(DEV), gate_offset=3)
    close(out, want_rows(rows), dtype, "portion")


# ------------------------------------------------------------------------------------------ the selective recurrence
def _scan_inputs(T, I, N, seed):
    x, dt_raw, bc, z = rnd(T, I, seed=seed), rnd(T, I, seed=seed + 1), rnd(T, 2 * N, seed=seed + 2), rnd(T, I, seed=seed + 3)
    g = torch.Generator().manual_seed(seed + 4)
    a_log = torch.rand(I, N, generator=g) * 5.0 - 4.0
    return x, dt_raw, bc, z, a_log, rnd(I, seed=seed + 5) * 0.7, 1 + 0.5 * rnd(I, seed=seed + 6)


def _scan_plain(x, dt_raw, bc, z, a_log, dt_bias, d, N):
    dt = plain.softplus(dt_raw.double() + dt_bias.double())
    y = plain.selective_scan(x.double(), dt, bc[:, :N].double(), bc[:, N:].double(), a_log.double(), d.double())
    return y * plain.silu(z.double())


@pytest.mark.parametrize("I,N", [(48, 8), (18, 7), (30, 5), (24, 1), (96, 16), (320, 24), (64, 40), (256, 128), (40, 200), (80, 3)])
def test_selective_recurrence_against_the_plain_scan(I, N):
    """Three requests of unequal lengths in one step, then single tokens that go on from the states the step left; a slot
    that another request used before starts clean only because the caller zeroes it (checked: the state is carried)."""
    from hipinfer_b200.kernels import ops

    lens, tail = [70, 1, 33], 5
    ins = [_scan_inputs(n + tail, I, N, 10 * r) for r, n in enumerate(lens)]
    a_log, dt_bias, d = ins[0][4], ins[0][5], ins[0][6]
    want = [_scan_plain(x, dr, bc, z, a_log, dt_bias, d, N) for x, dr, bc, z, *_ in ins]
    state = torch.zeros(5, I, N, dtype=torch.float32, device=DEV)
    slots = [3, 0, 4]
    cat = lambda k, lo, hi: torch.cat([ins[r][k][lo(r):hi(r)] for r in range(3)]).to(DEV)
    first = (lambda r: 0), (lambda r: lens[r])
    out = torch.empty(sum(lens), I, dtype=torch.float32, device=DEV)
    ops.selective_scan(cat(0, *first), cat(1, *first), cat(2, *first), cat(3, *first), dt_bias.to(DEV), a_log.to(DEV), d.to(DEV),
                       state, batch_of(lens, slots=slots), out)
    o = 0
    for r, n in enumerate(lens):
        close(out[o:o + n], want[r][:n], torch.float32, f"request {r}", tol=1e-4)
        o += n
    assert float(state[1].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0 and float(state[3].abs().max()) > 0.0
    for j in range(tail):
        step = (lambda r: lens[r] + j), (lambda r: lens[r] + j + 1)
        out1 = torch.empty(3, I, dtype=torch.float32, device=DEV)
        ops.selective_scan(cat(0, *step), cat(1, *step), cat(2, *step), cat(3, *step), dt_bias.to(DEV), a_log.to(DEV), d.to(DEV),
                           state, batch_of([1, 1, 1], slots=slots), out1)
        for r in range(3):
            close(out1[r], want[r][lens[r] + j], torch.float32, f"request {r}, single token {j}", tol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_recurrence_is_the_same_however_the_tokens_are_cut(dtype):
    """One launch over 75 tokens, portions of 2, 16, 17, 1 and 39, and one token a launch give the same bits: a token's
    arithmetic does not depend on where a portion or a chunk starts. Views of wider rows are read in place."""
    from hipinfer_b200.kernels import ops

    T, I, N = 75, 40, 12
    x, dt_raw, bc, z, a_log, dt_bias, d = _scan_inputs(T, I, N, 3)
    wide = torch.cat([rnd(T, 3, seed=9), x, z, bc, dt_raw], 1).to(DEV)      # x, z, B | C, dt as views of one wide row
    xv, zv, bcv, dtv = wide[:, 3:3 + I], wide[:, 3 + I:3 + 2 * I], wide[:, 3 + 2 * I:3 + 2 * I + 2 * N], wide[:, 3 + 2 * I + 2 * N:]
    consts = [t.to(dtype).to(DEV) for t in (dt_bias, a_log, d)]

    def run(cuts):
        state = torch.zeros(1, I, N, dtype=torch.float32, device=DEV)
        out = torch.empty(T, I, dtype=dtype, device=DEV)
        o = 0
        for n in cuts:
            ops.selective_scan(xv[o:o + n], dtv[o:o + n], bcv[o:o + n], zv[o:o + n], *consts, state, batch_of([n]), out[o:o + n])
            o += n
        return out, state

    whole, s0 = run([T])
    want = _scan_plain(x, dt_raw, bc, z, a_log.to(dtype), dt_bias.to(dtype), d.to(dtype), N)
    close(whole, want, dtype, tol=1e-4 if dtype == torch.float32 else None)
    for cuts in ([2, 16, 17, 1, 39], [1] * T):
        got, s1 = run(cuts)
        assert torch.equal(got, whole) and torch.equal(s0, s1)


@pytest.mark.parametrize("I,N", [(48, 8), (18, 7), (96, 16), (40, 200)])
@pytest.mark.parametrize("piece", [4, 16, 64])
def test_selective_recurrence_in_pieces(I, N, piece, monkeypatch):
    """Portions long enough run in pieces (every piece from a zero state, the starting states in order, every piece again
    for the results): unequal requests, one that ends inside a piece, one of a single token, states that an earlier portion
    left; against the plain scan and against the walk in one go. The states the pieces leave are those the next tokens
    start from."""
    from hipinfer_b200.kernels import ops

    lens, then = [3 * piece + 5, 1, 4 * piece, 3 * piece - 1], 3 * piece + 2
    ins = [_scan_inputs(n + then + 2, I, N, 10 * r) for r, n in enumerate(lens)]
    a_log, dt_bias, d = ins[0][4], ins[0][5], ins[0][6]
    want = [_scan_plain(x, dr, bc, z, a_log, dt_bias, d, N) for x, dr, bc, z, *_ in ins]
    consts = [t.to(DEV) for t in (dt_bias, a_log, d)]
    slots = [2, 0, 3, 1]

    def run(piece_tokens):
        monkeypatch.setattr(ops, "SEL_PIECE_TOKENS", piece_tokens)
        state = torch.zeros(4, I, N, dtype=torch.float32, device=DEV)
        outs, lo = [], [0] * 4
        for ns in (lens, [then] * 4, [1] * 4, [1] * 4):
            cat = lambda k: torch.cat([ins[r][k][lo[r]:lo[r] + ns[r]] for r in range(4)]).to(DEV)
            out = torch.empty(sum(ns), I, dtype=torch.float32, device=DEV)
            ops.selective_scan(cat(0), cat(1), cat(2), cat(3), *consts, state, batch_of(ns, slots=slots), out)
            outs.append(out.cpu())
            lo = [a + b for a, b in zip(lo, ns)]
        return outs, state.cpu()

    (got, state), (whole, state_w) = run(piece), run(0)
    lo = [0] * 4
    for k, ns in enumerate((lens, [then] * 4, [1] * 4, [1] * 4)):
        o = 0
        for r in range(4):
            close(got[k][o:o + ns[r]], want[r][lo[r]:lo[r] + ns[r]], torch.float32, f"step {k}, request {r}", tol=1e-4)
            close(got[k][o:o + ns[r]], whole[k][o:o + ns[r]], torch.float32, f"step {k}, request {r}: pieces against one walk", tol=1e-4)
            o += ns[r]
        lo = [a + b for a, b in zip(lo, ns)]
    close(state, state_w, torch.float32, "the states left", tol=1e-4)


def test_a_slow_decay_carries_a_far_token_and_a_fast_one_forgets_it():
    """Channel 0 decays by exp(-e^-9 dt) a token: what token 0 wrote is still there 600 tokens on. Channel 1 decays by
    exp(-e^3 dt): it holds the last token alone. The inputs of all tokens between are zero, so the result names the token."""
    from hipinfer_b200.kernels import ops

    T, I, N = 601, 2, 4
    x, dt_raw, z = torch.zeros(T, I), torch.full((T, I), 0.5), torch.full((T, I), 30.0)       # silu(30) = 30
    bc = torch.zeros(T, 2 * N)
    x[0], x[T - 1] = torch.tensor([2.0, 2.0]), torch.tensor([0.0, 3.0])
    bc[0, :N] = 1.0
    bc[T - 1, :N], bc[T - 1, N:] = 1.0, 1.0
    a_log = torch.tensor([[-9.0] * N, [3.0] * N])
    dt_bias, d = torch.zeros(I), torch.zeros(I)
    state = torch.zeros(1, I, N, dtype=torch.float32, device=DEV)
    out = torch.empty(T, I, dtype=torch.float32, device=DEV)
    ops.selective_scan(x.to(DEV), dt_raw.to(DEV), bc.to(DEV), z.to(DEV), dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), state, batch_of([T]), out)
    want = _scan_plain(x, dt_raw, bc, z, a_log, dt_bias, d, N)
    close(out, want, torch.float32, tol=1e-4)
    dt = float(plain.softplus(torch.tensor(0.5, dtype=F)))
    far = 2.0 * dt * math.exp(-math.exp(-9.0) * dt * (T - 1)) * N * 30.0
    assert abs(float(out[T - 1, 0]) - far) < 1e-3 * far and far > 50.0                         # token 0 is still nearly whole
    assert abs(float(out[T - 1, 1]) - 3.0 * dt * N * 30.0) < 1e-3 * 3.0 * dt * N * 30.0        # nothing of token 0 is left


@pytest.mark.parametrize("M,K,N", [(200, 128, 96), (70, 16, 256), (300, 12, 64), (8, 128, 96)])
def test_a_32_bit_product_through_two_rounded_halves(M, K, N):
    """32-bit rows times a bfloat16 weight: as the sum of two bfloat16 matrices on the tensor cores where the sizes allow,
    on the plain kernel otherwise; either way far closer than rounding the rows to bfloat16 would be."""
    from hipinfer_b200.kernels import ops

    wide = rnd(M, K + 5, seed=1)
    a, w = wide[:, 5:], (rnd(N, K, seed=2) / math.sqrt(K)).bfloat16()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear_split32(wide.to(DEV)[:, 5:], ops.Weight(w.to(DEV)), out)
    want = a.double() @ w.double().T
    close(out, want, torch.float32, tol=3e-5)
    assert float((a.bfloat16().double() @ w.double().T - want).abs().max()) > 1e-3 * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,I,N,R,K", [(64, 48, 8, 5, 4), (50, 18, 7, 2, 5), (128, 256, 16, 8, 3), (48, 24, 12, 3, 1), (96, 80, 3, 1, 7), (64, 40, 6, 4, 11)])
def test_selective_mixer_part(dtype, W, I, N, R, K):
    """The whole mixer through its part: a portion of two requests, then single tokens from the states and the carried
    convolution inputs it left."""
    from hipinfer_b200.parts.registry import BuildContext, build_part
    from hipinfer_b200.parts.spec import PartSpec

    part = build_part("mixer", PartSpec("selective_scan", dict(hidden_size=W, inner=I, state=N, dt_rank=R, conv=K)), BuildContext(dtype, DEV), "p.")
    g = torch.Generator().manual_seed(5)
    w = {}
    for s in part.param_specs():
        leaf = s.name[len("p.mix."):]
        t = torch.randn(s.shape, generator=g)
        w[leaf] = ({"A_log": torch.rand(s.shape, generator=g) * 5 - 4, "D": 1 + 0.5 * t, "conv": (1.2 / math.sqrt(K)) * t, "conv.b": 0.5 * t, "dt.b": 0.5 * t}
                   .get(leaf, t * (1.2 / math.sqrt(s.shape[-1])))).to(dtype)
    part.load({"p.mix." + k: v.to(DEV) for k, v in w.items()})
    lens, tail = [37, 6], 3
    hs = [(rnd(n + tail, W, seed=20 + r) * 1.5).to(dtype) for r, n in enumerate(lens)]
    m = dict(inner=I, state=N, dt_rank=R, conv=K)
    want = [plain.selective_mixer(h.double(), {k: v.double() for k, v in w.items()}, m) for h in hs]
    state = {k: torch.zeros((2,) + shape, dtype=dt, device=DEV) for k, (shape, dt) in part.state_need().items()}
    y = torch.full((sum(lens), W), 0.25, dtype=torch.float32, device=DEV)            # the result is ADDED
    b = batch_of(lens)
    b.dump = None
    part.forward(torch.cat([h[:n] for h, n in zip(hs, lens)]).to(DEV), y, b, None, state)
    close(y[:lens[0]] - 0.25, want[0][:lens[0]], dtype, "portion 0", tol=None if dtype == torch.bfloat16 else 1e-4)
    close(y[lens[0]:] - 0.25, want[1][:lens[1]], dtype, "portion 1", tol=None if dtype == torch.bfloat16 else 1e-4)
    for j in range(tail):
        y = torch.zeros(2, W, dtype=torch.float32, device=DEV)
        b = batch_of([1, 1])
        b.dump = None
        part.forward(torch.stack([hs[r][lens[r] + j] for r in range(2)]).to(DEV), y, b, None, state)
        for r in range(2):
            close(y[r], want[r][lens[r] + j], dtype, f"request {r}, single token {j}", tol=None if dtype == torch.bfloat16 else 1e-4)


# ------------------------------------------------------------------------------------------ latent attention
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,Dr,rot", [(136, 32, 32), (20, 6, 4), (64, 64, 64)])
def test_latents_into_the_cache_with_either_pairing(dtype, R, Dr, rot):
    from hipinfer_b200.kernels import ops

    T, ps, eps, base = 9, 8, 1e-5, 10000.0
    sc = dict(kind="yarn", factor=4.0, original=32, fast=8.0, slow=1.0)
    proj = rnd(T, 2 + R + Dr, seed=1)
    wc = (1 + 0.3 * rnd(R, seed=2)).to(dtype)
    pos = torch.tensor([0, 1, 2, 30, 31, 32, 400, 5, 6])
    slots = torch.randperm(3 * ps, generator=torch.Generator().manual_seed(3))[:T].to(torch.int32)
    table = ops.shared_rope_table(rot, base, 512, DEV, sc)
    f, mag = plain.yarn_frequencies(rot, base, {k: v for k, v in sc.items() if k != "kind"})
    for pairing in ("half", "interleaved"):
        cache = torch.zeros(3, 1, ps, R + Dr, dtype=dtype, device=DEV)
        ops.latent_prepare(proj.to(DEV), (0, 2, 2 + R), None, wc.to(DEV), pos.to(torch.int32).to(DEV), slots.to(DEV), table, rot, eps,
                           torch.empty(T, 0, dtype=dtype, device=DEV), cache, 0, R, Dr, ps, pairing)
        c = plain.rms(proj[:, 2:2 + R].double(), eps) * wc.double()
        kr = plain.rotate(proj[:, 2 + R:].double(), pos, f, rot, pairing, mag)
        for t in range(T):
            row = cache[int(slots[t]) // ps, 0, int(slots[t]) % ps]
            close(row[:R], c[t], dtype, f"{pairing}: latent of row {t}")
            close(row[R:], kr[t], dtype, f"{pairing}: rotated key part of row {t}", tol=None if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_head_by_head_with_a_half_paired_tail_and_a_gate_per_head(dtype):
    from hipinfer_b200.kernels import ops

    T, H, K, N, tail, rot, base = 7, 3, 20, 12, 8, 6, 100.0
    a = rnd(T, 2 + H * (K + tail), seed=1)
    wt = rnd(H, K, N, seed=2).to(dtype)
    pos = torch.tensor([0, 3, 9, 100, 101, 1, 2])
    table = ops.shared_rope_table(rot, base, 512, DEV)
    out = torch.empty(T, H * (N + tail), dtype=dtype, device=DEV)
    ops.heads_linear(a[:, 2:].to(DEV), K + tail, wt.to(DEV), out, N + tail, tail=tail, rot=rot, positions=pos.to(torch.int32).to(DEV),
                     table=table, pairing="half")
    a3 = a[:, 2:].double().reshape(T, H, K + tail)
    want = torch.cat([torch.einsum("thk,hkn->thn", a3[..., :K], wt.double()),
                      plain.rotate(a3[..., K:], pos, plain.band_frequencies(rot, base), rot, "half")], -1)
    close(out.view(T, H, N + tail), want, dtype, "tail", tol=None if dtype == torch.bfloat16 else 1e-4)
    gate = rnd(T, 4 + H, seed=3) * 2
    out = torch.empty(T, H * N, dtype=dtype, device=DEV)
    ops.heads_linear(a3[..., :K].reshape(T, H * K).float().to(DEV), K, wt.to(DEV), out, N, gate=gate.to(DEV), gate_offset=4, gate_per_head=True)
    want = torch.einsum("thk,hkn->thn", a3[..., :K].float().double(), wt.double()) * torch.sigmoid(gate[:, 4:].double())[:, :, None]
    close(out.view(T, H, N), want, dtype, "a gate per head")


def _paged_plane(rows_per_request, ps, dtype, seed):
    """One plane with one head: every request's rows on shuffled pages. (plane, block tables)"""
    n_pages = [-(-r.shape[0] // ps) for r in rows_per_request]
    order = torch.randperm(sum(n_pages) + 2, generator=torch.Generator().manual_seed(seed)).tolist()
    plane = torch.zeros(len(order), 1, ps, rows_per_request[0].shape[1], dtype=dtype)
    bt = torch.full((len(rows_per_request), max(n_pages)), -1, dtype=torch.int32)
    it = iter(order)
    for r, rows in enumerate(rows_per_request):
        for lp in range(n_pages[r]):
            page = next(it)
            bt[r, lp] = page
            m = min(ps, rows.shape[0] - lp * ps)
            plane[page, 0, :m] = rows[lp * ps:lp * ps + m].to(dtype)
    return plane.to(DEV), bt.to(DEV)


def _plain_sink_rows(q, keys, values, positions, scale, window, sink):
    """q [T, H, D] rows at `positions` of ONE sequence with keys [n, D] (shared by the heads) and values [n, E]."""
    n = keys.shape[0]
    j = torch.arange(n)
    out = []
    for t, p in enumerate(positions):
        seen = (j <= p) & ((p - j < window) if window else (j >= 0))
        s = (q[t] @ keys.T) * scale
        out.append(torch.stack([plain.softmax_with_sink(s[h][None], seen[None], None if sink is None else sink[h])[0] @ values
                                for h in range(q.shape[1])]))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,Dr,window,ps", [(6, 48, 16, 70, 16), (3, 40, 8, 24, 16), (2, 20, 6, 5, 8), (4, 32, 32, 1, 16), (4, 96, 32, 200, 16)])
def test_single_rows_with_a_sink_see_exactly_the_window(dtype, H, R, Dr, window, ps):
    """Rows of two requests over one plane of [latent | rotated key part] rows, the values its first columns, a sink per
    head in the denominator. The key just inside the window has a large score and the key just outside a larger one: one
    position off in either direction and the result is another vector. One head's sink is far above every score: that
    head's result is nearly zero; without the sink it is not."""
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
    plane, bt = _paged_plane(keys, ps, dtype, 1)
    keys = [k.to(dtype).double() for k in keys]
    qd = q.to(dtype)
    sink = rnd(H, seed=11) * 2
    sink[H - 1] = 60.0
    batch = SimpleNamespace(block_tables=[bt], row_request=i32(r for r, _ in rows), positions=i32(p for _, p in rows),
                            req_q_len=i32([1, 1]), h_q_len=[1, 1], max_q_len=1, max_pos=max(lens) - 1, n_requests=2, extra={})
    scale = 1.0 / math.sqrt(Dk)
    for use_sink in (True, False):
        want = torch.stack([_plain_sink_rows(qd[t:t + 1].double(), keys[r], keys[r][:, :R], [p], scale, window, sink.double() if use_sink else None)[0]
                            for t, (r, p) in enumerate(rows)])
        out = torch.empty(len(rows), H * R, dtype=torch.float32, device=DEV)
        ops.attention_masked(qd.reshape(len(rows), H * Dk).to(DEV), plane, plane, batch, 0, out, H, 1, Dk, R, ps, scale, "window", window=window,
                             sink=sink.to(DEV) if use_sink else None)
        close(out.view(len(rows), H, R), want, dtype, f"rows, sink {use_sink}")
        last = float(out.view(len(rows), H, R)[:, H - 1].abs().max())
        assert (last < 1e-6) if use_sink else (last > 1e-3)


@pytest.mark.parametrize("H,D,E,window,ctx,n", [(6, 64, 32, 70, 300, 130), (2, 32, 32, 24, 0, 100), (4, 64, 64, 1, 40, 64), (3, 96, 64, 200, 500, 17)])
def test_a_portion_s_rows_with_a_sink_and_a_gate_per_head(H, D, E, window, ctx, n):
    """The tensor-core kernel over keys and values made from the first kept page on, with the sink in the denominator and one
    gate number per head in its epilogue."""
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
    sink, gate = rnd(H, seed=4) * 2, rnd(3 + n, 2 + H, seed=5) * 2
    scale = 1.0 / math.sqrt(D)
    want = torch.stack([_plain_sink_rows(qb[:, h:h + 1].double(), kb[:, h].double(), vb[:, h].double(), range(ctx, total), scale, window,
                                         sink[h:h + 1].double())[:, 0] for h in range(H)], 1)
    want = want * torch.sigmoid(gate[3:, 2:].double())[:, :, None]
    batch = batch_of([3, n], ctx=[0, ctx])                                       # the request is the second of the step
    qall = torch.cat([torch.zeros(3, H * D, dtype=torch.bfloat16), qb.reshape(n, H * D)]).to(DEV)
    out = torch.zeros(3 + n, H * E, dtype=torch.bfloat16, device=DEV)
    ops.attention_flash_tokens(qall, kb[first:].reshape(-1, H * D).contiguous().to(DEV), vb[first:].reshape(-1, H * E).contiguous().to(DEV),
                               batch, 1, out, H, H, D, E, scale, window=window, first_pos=first, sink=sink.to(DEV), gate=gate.to(DEV),
                               gate_offset=2, gate_per_head=True)
    close(out[3:].view(n, H, E), want, torch.bfloat16, "portion")
    assert float(out[:3].float().abs().max()) == 0.0


# ------------------------------------------------------------------------------------------ experts
def _routed(dtype, W, Fs, E, top):
    from hipinfer_b200.parts.registry import BuildContext, build_part
    from hipinfer_b200.parts.spec import PartSpec

    part = build_part("feed_forward", PartSpec("routed", dict(hidden_size=W, experts=E, top=top, expert_size=Fs, score="softmax_chosen",
                                                              weight_at="output", router_bias=True)), BuildContext(dtype, DEV), "p.")
    g = torch.Generator().manual_seed(7)
    w = {}
    for s in part.param_specs():
        leaf = s.name[len("p.mlp."):]
        t = torch.randn(s.shape, generator=g)
        w[leaf] = (t * 0.7 if leaf == "router.b" else t * ((3.0 if leaf == "router" else 1.2) / math.sqrt(s.shape[-1]))).to(dtype)
    part.load({"p.mlp." + k: v.to(DEV) for k, v in w.items()})
    return part, {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,Fs,E,top,T", [(64, 32, 5, 2, 9), (50, 22, 3, 3, 7), (128, 96, 16, 4, 200), (160, 64, 6, 1, 130), (48, 40, 1, 1, 5),
                                          (2112, 72, 4, 2, 40), (96, 160, 3, 2, 30)])
def test_experts_weighted_by_a_softmax_over_the_chosen_logits(dtype, W, Fs, E, top, T, monkeypatch):
    """The largest logits (with their bias) choose, the weights are the softmax over the chosen logits alone and multiply
    the experts' results; single rows one by one, single rows grouped by expert, and portions sorted by expert give the
    plain sum. In bfloat16 rows whose choice hangs on a nearly tied pair of logits are left out of the comparison."""
    from hipinfer_b200.parts import routed_ff

    part, w = _routed(dtype, W, Fs, E, top)
    h = (rnd(T, W, seed=50) * 1.5).to(dtype)
    want = plain.experts(h.double(), w, top)
    z = torch.sort(h.double() @ w["router"].T + w["router.b"], -1, descending=True).values
    sure = torch.ones(T, dtype=torch.bool) if top == E else (z[:, top - 1] - z[:, top]) > 1e-3 * z.abs().max()
    assert int(sure.sum()) >= T - 2
    for what, q_len, grouped_from in (("one by one", 1, 10 ** 9), ("grouped", 1, 1), ("sorted", T, 1)):
        monkeypatch.setattr(routed_ff, "GROUPED_MIN_PAIRS", grouped_from)
        y = torch.full((T, W), 0.25, dtype=torch.float32, device=DEV)            # the result is ADDED
        part.forward(h.to(DEV), y, SimpleNamespace(max_q_len=q_len, dump=None))
        close((y - 0.25).cpu()[sure], want[sure], dtype, what)


def test_router_logits_with_a_bias_ties_and_weights():
    from hipinfer_b200.kernels import ops

    W, E = 40, 6
    router, bias = rnd(E, W, seed=1), rnd(E, seed=3)
    router[4], bias[4] = router[1], bias[1]                                        # experts 1 and 4 always tie
    h = rnd(30, W, seed=2)
    expert, weight = ops.moe_route(h.to(DEV), router.to(DEV), 3, bias.to(DEV), "softmax_chosen")
    chosen, want = plain.route(h.double(), router.double(), bias.double(), 3)
    assert torch.equal(expert.cpu().long(), chosen)
    close(weight, want, torch.float32)
    assert float((weight.sum(-1) - 1).abs().max()) < 1e-6
    e = expert.cpu()
    both = ((e == 1).any(1) & (e == 4).any(1)).nonzero().flatten().tolist()
    assert both and all(e[t].tolist().index(1) < e[t].tolist().index(4) for t in both)
    # the bias moves the choice: without it other experts win somewhere
    no_bias, _ = ops.moe_route(h.to(DEV), router.to(DEV), 3, None, "softmax_chosen")
    assert not torch.equal(no_bias, expert)
    # negative logits everywhere: the largest still win (no score is mistaken for "taken")
    expert, weight = ops.moe_route(h.to(DEV), router.to(DEV), 3, (bias - 50.0).to(DEV), "softmax_chosen")
    assert torch.equal(expert.cpu().long(), chosen)
    close(weight, want, torch.float32, tol=1e-4)
