"""A plain, slow statement of the Runopel decoder on the CPU, one function per mechanism, written from the design's
equations and sharing no code with the engine. Everything is float64 torch on whole sequences (the recurrence token by
token); nothing is paged, batched, cached or fused. The GPU tests compare the engine with these functions.

Notation: T tokens at positions p = 0..T-1 of one sequence, W the model's width, S residual streams, m the residual
multiplier; for the state-space mixer H heads of P value channels, N state channels, G groups, K convolution taps; for
latent attention H heads, D plain and Dr rotated query/key dimensions, E value size, R the latent's size.

  rms               y = x / sqrt(mean(x^2) + eps)   (times a weight where one is named)
  layer, one stream x <- x + m * mixer(rms(x) * w1);  x <- x + m * ff(rms(x) * w2)
  layer, S streams  u = sum_s a_s x_s;  y = sublayer(rms(u) * w);  x_t <- sum_s M[s, t] x_s + m * b_t * y  (all t at once);
                    all streams start as the embedding, the model's output reads their sum
  state space       [z | x | B | C | dt] = Win h;  (x, B, C) <- silu(conv(x, B, C) + bias), causal, K taps per channel,
                    zeros before the sequence;  dt <- softplus(dt + dt_bias)
                    per head h (group g = h // (H / G)):  S_t = exp(-exp(A_h) dt) S_(t-1) + dt B_t x_t^T   (N x P)
                    y_t = S_t^T C_t + D_h x_t;  y <- y * silu(z);  rms in equal parts of the row, times a weight;  Wo
  latent attention  q = Wq h, per head [D plain | Dr rotated];  [c_raw | kr_raw] = Wdkv h;  c = rms(c_raw) * wc;
                    q_rot, kr rotated (pairs (2i, 2i + 1), angle p * base^(-2i / dims));  k_h = Wuk_h c, v_h = Wuv_h c
                    score = (q_plain . k_h + q_rot . kr) * scale over the keys j with 0 <= i - j < window;  softmax;  Wo
  dense ff          g = min(Wg h + bg, L);  u = clamp(Wu h + bu, -L, L);  Wd (g sigmoid(1.702 g) (u + 1)) + bd
  routed ff         s = sigmoid(Wr h);  the `top` largest s choose experts;  out = sum_e expert_e(s_e h),
                    expert(v) = Wd (silu(Wg v) * (Wu v))
  output            logits = embed @ (rms(x) * w) * logit_scale
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_div(t, eps):
    return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs()))


def rotate_pairs(t, positions, dims, base):
    """t [T, ..., D]: pairs (2i, 2i + 1), i < dims / 2, of the last axis rotated by each row's position."""
    out = t.clone()
    shape = (-1,) + (1,) * (t.dim() - 2)
    for i in range(dims // 2):
        ang = positions.to(F) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        u, v = t[..., 2 * i], t[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def causal_conv(x, weight, bias):
    """x [T, C], weight [C, K] (the last column multiplies the current token), bias [C]; zeros before the sequence."""
    T, C = x.shape
    K = weight.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=F), x], 0)
    out = bias.expand(T, C).clone()
    for j in range(K):
        out = out + padded[j:j + T] * weight[:, j]
    return out


def state_space_scan(x, B, C, dt, A_log, D, groups):
    """x [T, H, P], B and C [T, G, N], dt [T, H] (after softplus), A_log and D [H]; the state starts at zero."""
    T, H, P = x.shape
    N = B.shape[-1]
    per = H // groups
    y = torch.zeros(T, H, P, dtype=F)
    for h in range(H):
        g = h // per
        S = torch.zeros(N, P, dtype=F)
        for t in range(T):
            S = torch.exp(-torch.exp(A_log[h]) * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def mamba2(h, w, m, eps):
    """w: in, conv, conv.b, dt_bias, A_log, D, norm, o; m: heads, vdim, state, groups, norm_groups."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = H * P, h.shape[0]
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = state_space_scan(x, B, C, dt, w["A_log"], w["D"], G).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms_div(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def window_mask(T, window=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def latent_attention(h, w, m, eps):
    """w: q, dkv, dkv.norm, uk, uv, o; m: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, mask {size} or none."""
    H, D, Dr, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = (h @ w["q"].T).reshape(T, H, D + Dr)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    ckr = h @ w["dkv"].T
    c = rms_div(ckr[:, :R], eps) * w["dkv.norm"]
    kr = rotate_pairs(ckr[:, R:], pos, m["rot"]["dims"], m["rot"]["base"])
    k = (c @ w["uk"].T).reshape(T, H, D)
    v = (c @ w["uv"].T).reshape(T, H, E)
    size = (m.get("mask") or {}).get("size")
    seen = window_mask(T, size)
    out = torch.zeros(T, H, E, dtype=F)
    for hd in range(H):
        s = (q_plain[:, hd] @ k[:, hd].T + q_rot[:, hd] @ kr.T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, hd]
    return out.reshape(T, H * E) @ w["o"].T


def dense_ff(h, w, limit):
    g = torch.clamp(h @ w["gate"].T + w["gate.b"], max=limit)
    u = torch.clamp(h @ w["up"].T + w["up.b"], min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T + w["down.b"]


def route(h, router, top):
    """Scores sigmoid(Wr h) and, per row, the indices of the `top` largest (ties: the lower index)."""
    s = torch.sigmoid(h @ router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return s, order


def routed_ff(h, w, experts, top):
    """w: router, e<i>.gate / up / down. The score multiplies the expert's input."""
    s, chosen = route(h, w["router"], top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            v = s[t, e] * h[t]
            out[t] += (silu(v @ w[f"e{e}.gate"].T) * (v @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, layers_out=None, round_to=None):
    """Logits [T, vocab] of one sequence from position 0. cfg: the config.json dictionary; tensors: name -> tensor.
    layers_out (a list): the residual stream (the sum of the streams) after every layer is appended.
    round_to (a dtype): every sublayer's input and result are rounded to it; the difference to the exact logits measures
    how sensitive each position is to rounding."""
    rd = (lambda t: t) if round_to is None else (lambda t: t.to(round_to).to(F))
    eps = cfg["norm"]["eps"]
    m = float(cfg.get("residual_mult", 1.0))
    S = cfg.get("streams")
    embed = tensors["embed"].to(F)
    x0 = embed[torch.as_tensor(tokens, dtype=torch.long)]
    xs = [x0.clone() for _ in range(S)] if S else [x0]
    for i, L in enumerate(cfg["layers"]):
        t = sub(tensors, f"l{i}.")
        mix_w, mlp_w = sub(t, "mix."), sub(t, "mlp.")
        if L["type"] == "mamba2":
            mixer = lambda h: mamba2(h, mix_w, L["mixer"], eps)
        elif L["type"] == "latent_attention":
            mixer = lambda h: latent_attention(h, mix_w, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        subs = [(mixer, "norm1", "hc1.")]
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                ff = lambda h: dense_ff(h, mlp_w, mlp["limit"])
            else:
                ff = lambda h: routed_ff(h, mlp_w, mlp["router"]["experts"], mlp["router"]["top"])
            subs.append((ff, "norm2", "hc2."))
        for fn, norm, hc in subs:
            if S:
                c = sub(t, hc)
                u = sum(c["in"][s] * xs[s] for s in range(S))
                y = rd(fn(rd(rms_div(u, eps) * t[norm])))
                xs = [sum(c["mix"][s, k] * xs[s] for s in range(S)) + m * c["out"][k] * y for k in range(S)]
            else:
                xs = [xs[0] + m * rd(fn(rd(rms_div(xs[0], eps) * t[norm])))]
        if layers_out is not None:
            layers_out.append(sum(xs))
    x = sum(xs)
    return (rms_div(x, eps) * tensors["final.norm"].to(F)) @ embed.T * float(cfg.get("logit_scale", 1.0))
