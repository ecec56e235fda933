"""The dense feed-forward: SwiGLU. act = silu(xn Wg^T) * (xn Wu^T), silu(g) = g / (1 + e^-g)
(src/kernels.cuh:100-105), out = act Wd^T added into the residual stream
(src/api.cu:1708-1718). Gate and up are one matrix with rows interleaved in groups of 16
(16 gate rows, 16 up rows, ...), so that a tile of the product holds matching pairs and the
activation can be applied in the product's epilogue; the reference stores its weights the
same way for the same reason (scripts/export.py:97-101). The loader side of that choice is
here: `load` interleaves, nothing outside this file sees the layout.

params: hidden_size, intermediate_size, and the three tensor names.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Part, register_part, to_compute

GROUP = 16


class SwiGLU(Part):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        if self.inter % GROUP:
            raise ValueError(f"SwiGLU: intermediate_size {self.inter} must be a multiple of {GROUP} "
                             f"(gate and up rows are interleaved in groups of {GROUP})")
        self.names = {k: prefix + params.get(k + "_name", f"mlp.{k}_proj.weight") for k in ("gate", "up", "down")}
        self.wgu = self.wdown = None

    def param_specs(self):
        return [ParamSpec(self.names["gate"], (self.inter, self.hidden)),
                ParamSpec(self.names["up"], (self.inter, self.hidden)),
                ParamSpec(self.names["down"], (self.hidden, self.inter))]

    def load(self, tensors):
        g, u = to_compute(tensors[self.names["gate"]], self.ctx), to_compute(tensors[self.names["up"]], self.ctx)
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        I, H = self.inter, self.hidden
        gu = torch.stack([g.to(dt).reshape(I // GROUP, GROUP, H), u.to(dt).reshape(I // GROUP, GROUP, H)], 1)
        self.wgu = ops.Weight(gu.reshape(2 * I, H).contiguous())
        self.wdown = ops.Weight(to_compute(tensors[self.names["down"]], self.ctx))

    def weight_bytes(self):
        return self.wgu.nbytes + self.wdown.nbytes

    takes_lazy_norm = True
    takes_norm_feed = True     # forward() accepts norm_feed=: buffers of the norm that reads x next (see parts/block.py)

    def forward(self, xn, x, batch, norm_feed=None):
        act = torch.empty(xn.shape[0], self.inter, dtype=self.ctx.dtype, device=xn.device)
        if isinstance(xn, ops.LazyNorm):     # a few rows: the norm in the gate/up product's prologue
            if not ops.norm_linear_swiglu(xn, self.wgu, act, GROUP):
                ops.linear_swiglu(xn.materialize(), self.wgu, act, GROUP)
        else:
            ops.linear_swiglu(xn, self.wgu, act, GROUP)
        planes.record(batch, "activation", act)
        if ops.linear_add_rows(act, self.wdown, x, norm_feed):            # a few rows: added in the product's epilogue
            return None
        return ops.linear_deferred(act, self.wdown, x, accumulate=True)   # the next norm may add it


class GatedFF(Part):
    """A gated dense feed-forward with a choice of activation: out = Wdown (act(Wgate h) * (Wup h)), act "silu" or
    "gelu_tanh" (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))). Gate and up are one product; its 32-bit result feeds
    the activation, which is rounded once. Any intermediate size: rows are interleaved in groups of 16 where the size
    is a multiple of 16 (the layout the fused kernels of SwiGLU read), else the gate rows come first.

    params: hidden_size, intermediate_size, activation, gate_name, up_name, down_name."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.act = params.get("activation", "silu")
        if self.act not in ops.GATE_ACTS:
            raise ValueError(f"gated feed-forward: activation {self.act!r} is not known (known: {sorted(ops.GATE_ACTS)})")
        self.group = GROUP if self.inter % GROUP == 0 else self.inter
        self.names = {k: prefix + params.get(k + "_name", f"mlp.{k}") for k in ("gate", "up", "down")}
        self.wgu = self.wdown = None

    def param_specs(self):
        return [ParamSpec(self.names["gate"], (self.inter, self.hidden)), ParamSpec(self.names["up"], (self.inter, self.hidden)),
                ParamSpec(self.names["down"], (self.hidden, self.inter))]

    def load(self, tensors):
        g, u = to_compute(tensors[self.names["gate"]], self.ctx), to_compute(tensors[self.names["up"]], self.ctx)
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        I, H, G = self.inter, self.hidden, self.group
        gu = torch.stack([g.to(dt).reshape(I // G, G, H), u.to(dt).reshape(I // G, G, H)], 1)
        self.wgu = ops.Weight(gu.reshape(2 * I, H).contiguous())
        self.wdown = ops.Weight(to_compute(tensors[self.names["down"]], self.ctx))

    def weight_bytes(self):
        return self.wgu.nbytes + self.wdown.nbytes

    def forward(self, xn, x, batch):
        T = xn.shape[0]
        act = torch.empty(T, self.inter, dtype=self.ctx.dtype, device=xn.device)
        if not ops.linear_gated(xn, self.wgu, act, self.group, self.act):
            gu = torch.empty(T, 2 * self.inter, dtype=torch.float32, device=xn.device)
            ops.linear(xn, self.wgu, gu)
            ops.gated_act(gu, act, self.group, self.act)
        planes.record(batch, "activation", act)
        ops.linear_into_stream(act, self.wdown, x)
        return None


class PolyNormFF(Part):
    """A dense feed-forward without a gate: out = act(xn Wup^T) Wdown^T with the PolyNorm activation
    act(z) = c1 N(z) + c2 N(z^2) + c3 N(z^3) + c0, powers element by element, N(t) = t / sqrt(mean(t^2) + eps) over
    the row's `intermediate_size` values. The four coefficients are a tensor [c1, c2, c3, c0]. The up product stays in
    32-bit until after the activation (the three root mean squares are 32-bit sums), which is rounded once.

    params: hidden_size, intermediate_size, eps, up_name, down_name, act_name. With `out_scale=` (a vector over the
    output columns) the result is multiplied by it before it is added into the residual stream."""

    takes_out_scale = True

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.inter, self.eps = int(params["hidden_size"]), int(params["intermediate_size"]), float(params["eps"])
        self.names = {k: prefix + params.get(k + "_name", f"mlp.{k}") for k in ("up", "down", "act")}
        self.wup = self.wdown = self.coef = None

    def param_specs(self):
        return [ParamSpec(self.names["up"], (self.inter, self.hidden)), ParamSpec(self.names["down"], (self.hidden, self.inter)),
                ParamSpec(self.names["act"], (4,), init="ones")]

    def load(self, tensors):
        self.wup = ops.Weight(to_compute(tensors[self.names["up"]], self.ctx))
        self.wdown = ops.Weight(to_compute(tensors[self.names["down"]], self.ctx))
        self.coef = [float(v) for v in tensors[self.names["act"]].float().cpu().tolist()]

    def weight_bytes(self):
        return self.wup.nbytes + self.wdown.nbytes

    def forward(self, xn, x, batch, out_scale=None):
        T = xn.shape[0]
        z = torch.empty(T, self.inter, dtype=torch.float32, device=xn.device)
        ops.linear(xn, self.wup, z)
        act = torch.empty(T, self.inter, dtype=self.ctx.dtype, device=xn.device)
        ops.polynorm(z, self.coef, self.eps, act)
        planes.record(batch, "activation", act)
        if out_scale is None:
            ops.linear(act, self.wdown, x, accumulate=True)
        else:
            ops.linear_scaled_add(act, self.wdown, x, out_scale)
        return None


class ClampedGLU(Part):
    """A gated dense feed-forward with biases and limits:

        g = min(Wgate h + bg, L);  u = clamp(Wup h + bu, -L, L);  out = Wdown (g sigmoid(alpha g) (u + 1)) + bd

    Gate and up are one product; its 32-bit result takes the biases, the limits and the activation in one kernel, rounded
    once. Any intermediate size (rows interleaved in groups of 16 where the size allows, else gate rows first).

    params: hidden_size, intermediate_size, limit, alpha (default 1.702), gate_name, up_name, down_name; a projection's
    bias is its name + ".b"."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.limit, self.alpha = float(params["limit"]), float(params.get("alpha", 1.702))
        self.group = GROUP if self.inter % GROUP == 0 else self.inter
        self.names = {k: prefix + params.get(k + "_name", f"mlp.{k}") for k in ("gate", "up", "down")}
        self.wgu = self.wdown = self.bgu = self.bdown = None

    def param_specs(self):
        n, I, H = self.names, self.inter, self.hidden
        return [ParamSpec(n["gate"], (I, H)), ParamSpec(n["gate"] + ".b", (I,), init="zeros"),
                ParamSpec(n["up"], (I, H)), ParamSpec(n["up"] + ".b", (I,), init="zeros"),
                ParamSpec(n["down"], (H, I)), ParamSpec(n["down"] + ".b", (H,), init="zeros")]

    def load(self, tensors):
        t = lambda name: to_compute(tensors[name], self.ctx)
        g, u = t(self.names["gate"]), t(self.names["up"])
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        I, H, G = self.inter, self.hidden, self.group
        gu = torch.stack([g.to(dt).reshape(I // G, G, H), u.to(dt).reshape(I // G, G, H)], 1)
        self.wgu = ops.Weight(gu.reshape(2 * I, H).contiguous())
        bg, bu = t(self.names["gate"] + ".b"), t(self.names["up"] + ".b")
        self.bgu = torch.stack([bg.to(dt).reshape(I // G, G), bu.to(dt).reshape(I // G, G)], 1).reshape(2 * I).contiguous()
        self.wdown = ops.Weight(t(self.names["down"]))
        self.bdown = t(self.names["down"] + ".b")

    def weight_bytes(self):
        return self.wgu.nbytes + self.wdown.nbytes + sum(b.numel() * b.element_size() for b in (self.bgu, self.bdown))

    def forward(self, xn, x, batch):
        T = xn.shape[0]
        gu = torch.empty(T, 2 * self.inter, dtype=torch.float32, device=xn.device)
        ops.linear_rows32(xn, self.wgu, gu)
        act = torch.empty(T, self.inter, dtype=self.ctx.dtype, device=xn.device)
        ops.glu_bias(gu, self.bgu, act, self.group, "clamped_sigmoid", self.limit, self.alpha)
        planes.record(batch, "activation", act)
        ops.linear_into_stream(act, self.wdown, x)
        ops.scale_bias_rows(x, 1.0, self.bdown)
        return None


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "polynorm", PolyNormFF)
register_part("feed_forward", "gated", GatedFF)
register_part("feed_forward", "clamped_glu", ClampedGLU)
