"""A plain, slow statement of the Mavinex decoder on the CPU, one function per mechanism, written from the design's
equations and sharing no code with the engine. Everything is float64 torch on whole sequences (the recurrence token by
token); nothing is paged, batched, cached or fused. The GPU tests compare the engine with these functions.

Notation: T tokens at positions p = 0..T-1 of one sequence, W the model's width, a the residual multiplier.

  rms(x)            x / sqrt(mean(x^2) + eps)
  layer             x <- rms(a x + mixer(x)) (1 + n1);  x <- rms(a x + ff(x)) (1 + n2)       the sublayers read x itself
  side by side      mixer(h) = (rms(att(h)) wl + rms(ssm(h)) wr) / 2
  att               q = rms(Wq h) nq, k = rms(Wk h) nk over the whole rows; split into H and G heads of D; rotated on the
                    first `dims` dimensions of each head, pairs (2i, 2i + 1); score = q . k * scale over the keys j with
                    0 <= i - j < window; softmax; values E wide; heads concatenated, times sigmoid(Wg h), then Wo
  ssm               [x | z] = Win h;  x <- silu(conv(x) + b) (K taps, causal, zeros before the start);
                    [dl | B | C] = Wx x;  dt = softplus(Wdt dl + bd);  S[c, n] <- exp(-exp(Alog[c, n]) dt_c) S[c, n] + dt_c x_c B_n;
                    y_c = sum_n S[c, n] C_n + D_c x_c;  Wo (y silu(z))
  latent            q = Wq h per head [D plain | Dr rotated];  [c_raw | kr_raw] = Wdkv h;  c = rms(c_raw) nc;  the rotated
                    parts rotated with pairs (i, i + dims / 2) and YaRN frequencies, cos and sin times a magnitude;
                    k_h = Wuk_h c, v_h = Wuv_h c;  score = (q_plain . k_h + q_rot . kr) * scale inside the window;  softmax
                    whose denominator also holds exp(sink_h);  head h times sigmoid(Wg h)_h;  Wo
  experts           z = Wr h + br;  the `top` largest z choose;  weights = softmax over the chosen z;
                    out = sum_e weight_e Wd_e (silu(Wg_e h) * (Wu_e h))
  output            logits = head (rms(x) (1 + nf))
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(t, eps):
    return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs()))


def band_frequencies(dims, base, sc=None):
    """f_i = base^(-2i / dims); with sc {factor, low, high, original}: by wavelength l = 2 pi / f, f is kept below
    original / high, divided by factor above original / low, and blended linearly in original / l between."""
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    if not sc:
        return f
    out = f.clone()
    for i in range(dims // 2):
        wl = 2.0 * math.pi / float(f[i])
        if wl < sc["original"] / sc["high"]:
            continue
        if wl > sc["original"] / sc["low"]:
            out[i] = f[i] / sc["factor"]
        else:
            s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * f[i] / sc["factor"] + s * f[i]
    return out


def yarn_frequencies(dims, base, sc=None):
    """(frequencies, magnitude). With sc {factor, original, fast, slow}: a ramp over the pair index between the pair that
    turns `fast` times within `original` positions and the one that turns `slow` times blends f_i / factor (ramp 1) with
    f_i (ramp 0); the magnitude 0.1 ln(factor) + 1 multiplies cos and sin."""
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    if not sc:
        return f, 1.0
    turn = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(turn(sc["fast"])), 0), min(math.ceil(turn(sc["slow"])), dims - 1)
    out = f.clone()
    for i in range(dims // 2):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / sc["factor"] * r + f[i] * (1.0 - r)
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(t, positions, freqs, dims, pairing, magnitude=1.0):
    """t [T, ..., D]: the first `dims` dimensions of the last axis rotated by each row's position; pairing "interleaved":
    pairs (2i, 2i + 1); "half": pairs (i, i + dims / 2). cos and sin are multiplied by `magnitude`."""
    out = t.clone()
    shape = (-1,) + (1,) * (t.dim() - 2)
    for i in range(dims // 2):
        ang = positions.to(F) * freqs[i]
        c, s = (torch.cos(ang) * magnitude).view(shape), (torch.sin(ang) * magnitude).view(shape)
        ia, ib = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
        u, v = t[..., ia], t[..., ib]
        out[..., ia] = u * c - v * s
        out[..., ib] = v * c + u * s
    return out


def visible(T, window=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def softmax_with_sink(scores, seen, sink=None):
    """Rows of softmax over the seen keys; with `sink` the denominator also holds exp(sink) (no key, no value)."""
    s = scores.masked_fill(~seen, float("-inf"))
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, torch.as_tensor(sink, dtype=F))
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(torch.as_tensor(sink, dtype=F) - top)
    return e / den


def window_attention(h, w, m, eps):
    """w: q, k, v, q.norm, k.norm, g, o; m: heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling}, mask {size} or none."""
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    f = band_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = rotate((rms(h @ w["q"].T, eps) * w["q.norm"]).reshape(T, H, D), pos, f, m["rot"]["dims"], "interleaved")
    k = rotate((rms(h @ w["k"].T, eps) * w["k.norm"]).reshape(T, G, D), pos, f, m["rot"]["dims"], "interleaved")
    v = (h @ w["v"].T).reshape(T, G, E)
    seen = visible(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, E, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = softmax_with_sink((q[:, hd] @ k[:, g].T) * m["scale"], seen) @ v[:, g]
    return (out.reshape(T, H * E) * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def causal_conv(x, weight, bias):
    """x [T, C], weight [C, K] (the last column multiplies the current token), bias [C]; zeros before the sequence."""
    T, C = x.shape
    K = weight.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=F), x], 0)
    out = bias.expand(T, C).clone()
    for j in range(K):
        out = out + padded[j:j + T] * weight[:, j]
    return out


def selective_scan(x, dt, B, C, A_log, D):
    """x, dt [T, I] (dt after softplus), B, C [T, N], A_log [I, N], D [I]; the state starts at zero. y [T, I]."""
    T, I = x.shape
    A = -torch.exp(A_log)
    S = torch.zeros(I, A.shape[1], dtype=F)
    y = torch.zeros(T, I, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


def selective_mixer(h, w, m):
    """w: in, conv, conv.b, x, dt, dt.b, A_log, D, o; m: inner, state, dt_rank, conv."""
    I, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w["in"].T
    x, z = silu(causal_conv(xz[:, :I], w["conv"], w["conv.b"])), xz[:, I:]
    low = x @ w["x"].T
    dt = softplus(low[:, :R] @ w["dt"].T + w["dt.b"])
    y = selective_scan(x, dt, low[:, R:R + N], low[:, R + N:], w["A_log"], w["D"])
    return (y * silu(z)) @ w["o"].T


def side_by_side(h, w, m, eps):
    a = window_attention(h, sub(w, "left."), m["left"], eps)
    b = selective_mixer(h, sub(w, "right."), m["right"])
    return 0.5 * (rms(a, eps) * w["left.out"] + rms(b, eps) * w["right.out"])


def latent_attention(h, w, m, eps):
    """w: q, dkv, dkv.norm, uk, uv, sink, g, o; m: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling}, mask."""
    H, D, Dr, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    f, mag = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = (h @ w["q"].T).reshape(T, H, D + Dr)
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], pos, f, m["rot"]["dims"], "half", mag)
    ckr = h @ w["dkv"].T
    c = rms(ckr[:, :R], eps) * w["dkv.norm"]
    kr = rotate(ckr[:, R:], pos, f, m["rot"]["dims"], "half", mag)
    k = (c @ w["uk"].T).reshape(T, H, D)
    v = (c @ w["uv"].T).reshape(T, H, E)
    seen = visible(T, (m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ w["g"].T)
    out = torch.zeros(T, H, E, dtype=F)
    for hd in range(H):
        s = (q_plain[:, hd] @ k[:, hd].T + q_rot[:, hd] @ kr.T) * m["scale"]
        out[:, hd] = softmax_with_sink(s, seen, w["sink"][hd]) @ v[:, hd] * gate[:, hd:hd + 1]
    return out.reshape(T, H * E) @ w["o"].T


def route(h, router, bias, top):
    """(chosen experts [T, top], weights [T, top]): the largest logits (ties: the lower index), softmax over the chosen."""
    z = h @ router.T + bias
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), -1)


def experts(h, w, top):
    """w: router, router.b, e<i>.gate / up / down. The weight multiplies the expert's result."""
    chosen, weight = route(h, w["router"], w["router.b"], top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j, e in enumerate(chosen[t].tolist()):
            out[t] += weight[t, j] * ((silu(h[t] @ w[f"e{e}.gate"].T) * (h[t] @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T)
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def weights_layer(cfg, i):
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg, tensors, tokens, layers_out=None, round_to=None):
    """Logits [T, vocab] of one sequence from position 0. cfg: the config.json dictionary; tensors: name -> tensor.
    layers_out (a list): the residual rows after every layer are appended.
    round_to (a dtype): every sublayer's input and result are rounded to it; the difference to the exact logits measures
    how sensitive each position is to rounding."""
    rd = (lambda t: t) if round_to is None else (lambda t: t.to(round_to).to(F))
    eps, a = cfg["norm"]["eps"], float(cfg.get("postln_alpha", 1.0))
    x = tensors["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, L in enumerate(cfg["layers"]):
        t = sub(tensors, f"l{weights_layer(cfg, i)}.")
        if L["type"] == "parallel":
            y = side_by_side(rd(x), sub(t, "mix."), L["mixer"], eps)
        elif L["type"] == "latent_attention":
            y = latent_attention(rd(x), sub(t, "mix."), L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = rms(a * x + rd(y), eps) * (1.0 + t["norm1"])
        if L.get("mlp") is not None:
            x = rms(a * x + rd(experts(rd(x), sub(t, "mlp."), L["mlp"]["router"]["top"])), eps) * (1.0 + t["norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * (1.0 + tensors["final.norm"].to(F))) @ tensors["head"].to(F).T
