"""The state-space mixer with a scalar decay per head (Mamba-2, the state-space duality form).

With H heads of P value channels, N state channels in G groups (head h reads group h // (H / G)), K convolution taps:

    [z (H P) | x (H P) | B (G N) | C (G N) | dt (H)] = Win h
    (x, B, C) <- silu(conv(x, B, C) + bias)      causal, one filter of K taps per channel, zeros before the sequence
    dt <- softplus(dt + dt_bias)                  no clamp
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T          S is N x P per head, starts at zero
    y_t = S_t^T C_t + D_h x_t
    y <- y * silu(z), then the row in `norm_groups` equal parts, each divided by its own root mean square (eps inside the
    root), times a weight; then Wo. The gate comes before the norm.

The input projection is one product whose 32-bit result feeds the convolution and the recurrence directly; step sizes,
decays, the state and the norm are 32-bit (csrc/ssd.cu). A request's state slot holds the state S and the last K - 1 raw
inputs of the convolution (`state_need`), zeroed at admission; there is no cache.

params: hidden_size, heads, vdim, state, groups, norm_groups, conv, eps, and the tensor names in, conv, conv_bias, dt_bias,
a_log, d, norm, o (`<key>_name`, relative to the prefix).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Mixer, register_part, to_compute

_DEFAULT_NAMES = dict({"in": "mix.in"}, conv="mix.conv", conv_bias="mix.conv.b", dt_bias="mix.dt_bias", a_log="mix.A_log",
                      d="mix.D", norm="mix.norm", o="mix.o")


class Mamba2Mixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden, self.heads, self.vdim = int(p["hidden_size"]), int(p["heads"]), int(p["vdim"])
        self.n_state, self.groups, self.norm_groups = int(p["state"]), int(p["groups"]), int(p["norm_groups"])
        self.taps, self.eps = int(p["conv"]), float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise ValueError(f"state-space mixer: {self.heads} heads in {self.groups} groups, {self.inner} channels in "
                             f"{self.norm_groups} norm groups")
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items()}
        self.w_in = self.wo = None

    def param_specs(self):
        n, W, H = self.names, self.hidden, self.heads
        return [ParamSpec(n["in"], (2 * self.inner + 2 * self.groups * self.n_state + H, W)),
                ParamSpec(n["conv"], (self.channels, self.taps)), ParamSpec(n["conv_bias"], (self.channels,), init="zeros"),
                ParamSpec(n["dt_bias"], (H,), init="zeros"), ParamSpec(n["a_log"], (H,), init="zeros"),
                ParamSpec(n["d"], (H,), init="ones"), ParamSpec(n["norm"], (self.inner,), init="ones"),
                ParamSpec(n["o"], (W, self.inner))]

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items()}
        self.w_in, self.wo = ops.Weight(t["in"]), ops.Weight(t["o"])
        self.conv_w = t["conv"]
        self.conv_b = t["conv_bias"].to(self.conv_w.dtype)
        self.dt_bias = t["dt_bias"]
        self.a_log, self.d_skip = t["a_log"].to(self.dt_bias.dtype), t["d"].to(self.dt_bias.dtype)
        self.norm_w = t["norm"]

    def weight_bytes(self):
        small = (self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_w)
        return self.w_in.nbytes + self.wo.nbytes + sum(w.numel() * w.element_size() for w in small)

    def state_need(self):
        return {"S": ((self.heads, self.n_state, self.vdim), torch.float32),
                "conv": ((self.taps - 1, self.channels), torch.float32)}

    def forward(self, xn, x, batch, cache, state):
        T, inner, dev = xn.shape[0], self.inner, xn.device
        proj = torch.empty(T, inner + self.channels + self.heads, dtype=torch.float32, device=dev)
        ops.linear_rows32(xn, self.w_in, proj)
        xbc = torch.empty(T, self.channels, dtype=torch.float32, device=dev)
        ops.ssd_conv(proj, inner, self.conv_w, self.conv_b, state["conv"], batch, xbc)
        y = torch.empty(T, inner, dtype=torch.float32, device=dev)
        ops.ssd_scan(xbc, proj[:, inner + self.channels:], self.dt_bias, self.a_log, self.d_skip, state["S"], batch, y,
                     self.heads, self.vdim, self.n_state, self.groups)
        yn = torch.empty(T, inner, dtype=self.ctx.dtype, device=dev)
        ops.ssd_gate_norm(y, proj[:, :inner], self.norm_w, yn, self.norm_groups, self.eps)
        planes.record(batch, "attention", yn)
        ops.linear_into_stream(yn, self.wo, x)
        return None


register_part("mixer", "mamba2", Mamba2Mixer)
