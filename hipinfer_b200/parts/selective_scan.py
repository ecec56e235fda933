"""The selective state-space mixer with a decay per (channel, state) pair (the Mamba-1 form).

With `inner` channels, N states a channel, a step-size rank R and K convolution taps:

    [x (inner) | z (inner)] = Win h
    x <- silu(conv(x) + bias)                     causal, one filter of K taps per channel, zeros before the sequence
    [dt_low (R) | B (N) | C (N)] = Wx x
    dt = softplus(Wdt dt_low + dt_bias)            one step size per channel
    S[c, n] <- exp(-exp(A_log[c, n]) dt_c) S[c, n] + dt_c x_c B_n          S starts at zero
    y_c = sum_n S[c, n] C_n + D_c x_c;   y <- y * silu(z);   then Wo

The input projection's 32-bit result feeds the convolution directly; step sizes, decays, their exponentials, the state and
the sums over it are 32-bit (csrc/selective_scan.cu); the convolved x is rounded only for the product with Wx, the
recurrence reads it in 32-bit. A request's state slot holds S and the last K - 1 raw inputs of the convolution
(`state_need`), zeroed at admission; there is no cache.

params: hidden_size, inner, state, dt_rank, conv, and the tensor names in, conv, conv_bias, x, dt, dt_bias, a_log, d, o
(`<key>_name`, relative to the prefix).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Mixer, register_part, to_compute

_DEFAULT_NAMES = dict({"in": "mix.in"}, conv="mix.conv", conv_bias="mix.conv.b", x="mix.x", dt="mix.dt", dt_bias="mix.dt.b",
                      a_log="mix.A_log", d="mix.D", o="mix.o")


class SelectiveScanMixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden, self.inner, self.n_state = int(p["hidden_size"]), int(p["inner"]), int(p["state"])
        self.dt_rank, self.taps = int(p["dt_rank"]), int(p["conv"])
        if min(self.inner, self.n_state, self.dt_rank, self.taps) < 1:
            raise ValueError("selective state-space mixer: every size must be positive")
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items()}
        self.w_in = self.w_x = self.w_dt = self.wo = None

    def param_specs(self):
        n, W, I, N, R = self.names, self.hidden, self.inner, self.n_state, self.dt_rank
        return [ParamSpec(n["in"], (2 * I, W)), ParamSpec(n["conv"], (I, self.taps)), ParamSpec(n["conv_bias"], (I,), init="zeros"),
                ParamSpec(n["x"], (R + 2 * N, I)), ParamSpec(n["dt"], (I, R)), ParamSpec(n["dt_bias"], (I,), init="zeros"),
                ParamSpec(n["a_log"], (I, N), init="zeros"), ParamSpec(n["d"], (I,), init="ones"), ParamSpec(n["o"], (W, I))]

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items()}
        self.w_in, self.w_x, self.w_dt, self.wo = (ops.Weight(t[k]) for k in ("in", "x", "dt", "o"))
        self.conv_w = t["conv"]
        self.conv_b = t["conv_bias"].to(self.conv_w.dtype)
        self.a_log = t["a_log"]
        self.dt_bias, self.d_skip = t["dt_bias"].to(self.a_log.dtype), t["d"].to(self.a_log.dtype)

    def weight_bytes(self):
        small = (self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip)
        return (self.w_in.nbytes + self.w_x.nbytes + self.w_dt.nbytes + self.wo.nbytes
                + sum(w.numel() * w.element_size() for w in small))

    def state_need(self):
        return {"S": ((self.inner, self.n_state), torch.float32), "conv": ((self.taps - 1, self.inner), torch.float32)}

    def forward(self, xn, x, batch, cache, state):
        T, I, N, R, dev = xn.shape[0], self.inner, self.n_state, self.dt_rank, xn.device
        proj = torch.empty(T, 2 * I, dtype=torch.float32, device=dev)
        ops.linear_rows32(xn, self.w_in, proj)
        xc = torch.empty(T, I, dtype=torch.float32, device=dev)
        ops.ssd_conv(proj, 0, self.conv_w, self.conv_b, state["conv"], batch, xc)
        dbc = torch.empty(T, R + 2 * N, dtype=torch.float32, device=dev)
        ops.linear_rows32(xc if self.ctx.dtype == torch.float32 else ops.convert(xc, self.ctx.dtype), self.w_x, dbc)
        dt = torch.empty(T, I, dtype=torch.float32, device=dev)
        ops.linear_split32(dbc[:, :R], self.w_dt, dt)         # the low-rank step sizes keep 16 bits or more into their product
        y = torch.empty(T, I, dtype=self.ctx.dtype, device=dev)
        ops.selective_scan(xc, dt, dbc[:, R:], proj[:, I:], self.dt_bias, self.a_log, self.d_skip, state["S"], batch, y)
        planes.record(batch, "attention", y)
        ops.linear_into_stream(y, self.wo, x)
        return None


register_part("mixer", "selective_scan", SelectiveScanMixer)
