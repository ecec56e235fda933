"""RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)), plain weight (not 1 + w), computed in
32-bit from the 32-bit residual stream and rounded once (src/kernels.cuh:108-125 rounds x*r
to fp16 before the product with w, to match a half-precision framework)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from .registry import Part, register_part, to_compute


class RMSNorm(Part):
    """params: name (tensor name relative to the prefix), size, eps, one_plus (default False: the weight multiplies as it is
    stored; True: the tensor is stored around zero and the row is multiplied by 1 + w, a sum made in 32-bit at load and kept
    in 32-bit)."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.name = prefix + params["name"]
        self.one_plus = bool(params.get("one_plus", False))
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.size,), init="zeros" if self.one_plus else "ones")]

    def load(self, tensors):
        if self.one_plus:
            self.weight = (tensors[self.name].to(torch.float32) + 1.0).contiguous()
            return
        self.weight = to_compute(tensors[self.name], self.ctx)

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    takes_pending = True

    def lazy(self, x, feed=None):
        """The norm of x left to its consumer (kernels.ops.LazyNorm) where a consumer could fold it into its product, else
        None. feed: what `feed()` gave and the product that wrote x has filled; the consumer then needs no prologue."""
        if self.weight is None or not ops.lazy_norm_applies(x, self.weight, self.ctx.dtype):
            return None
        ok = feed is not None and feed.filled and feed.weight is self.weight
        return ops.LazyNorm(x, self.weight, self.eps, self.ctx.dtype, feed if ok else None)

    def feed(self, rows):
        """Buffers that the product which writes this norm's input rows may fill on its way (x times this norm's weight in
        bf16, and the pieces of the rows' sums of squares), for steps of a few rows; else None. See kernels.fast.NormFeed."""
        if self.weight is None or self.ctx.dtype != torch.bfloat16:
            return None
        return ops.make_norm_feed(self.weight, self.eps, rows)

    def forward(self, x, rows=None, out=None, pending=None):
        """pending: a sum that has yet to be added into x (it is added before the norm)."""
        M = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty(M, self.size, dtype=self.ctx.dtype, device=x.device)
        return ops.rmsnorm(x, self.weight, self.eps, out, rows, pending)


class LayerNorm(Part):
    """Layer norm with a weight and, where `bias_name` is given, a bias: y = w * (x - mean(x)) / sqrt(mean((x - mean(x))^2)
    + eps) + b, computed in 32-bit from the 32-bit residual stream and rounded once. params: name (tensor name relative
    to the prefix), size, eps, bias_name (absent: no bias). `out` may be a 32-bit tensor (a norm inside the stream)."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.name = prefix + params["name"]
        self.bias_name = prefix + params["bias_name"] if params.get("bias_name") else None
        self.weight = self.bias = None

    def param_specs(self):
        specs = [ParamSpec(self.name, (self.size,), init="ones")]
        if self.bias_name:
            specs.append(ParamSpec(self.bias_name, (self.size,), init="zeros"))
        return specs

    def load(self, tensors):
        self.weight = to_compute(tensors[self.name], self.ctx)
        if self.bias_name:
            self.bias = to_compute(tensors[self.bias_name], self.ctx).to(self.weight.dtype)

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size() * (2 if self.bias is not None else 1)

    def forward(self, x, rows=None, out=None):
        M = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty(M, self.size, dtype=self.ctx.dtype, device=x.device)
        return ops.layernorm(x, self.weight, self.eps, out, rows, self.bias)


class StreamsRMSNorm(Part):
    """RMSNorm of a weighted sum of residual streams: u = sum_s read[s] x_s, y = w * u / sqrt(mean(u^2) + eps), for rows
    x float32 [T, streams * size]; all 32-bit, rounded once. The read weights are a tensor [streams] (`read_name`); without
    one the streams are summed as they are (the norm before the head). params: name, size, eps, streams, read_name."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.size, self.eps, self.streams = int(params["size"]), float(params["eps"]), int(params["streams"])
        self.name = prefix + params["name"]
        self.read_name = prefix + params["read_name"] if params.get("read_name") else None
        self.weight = self.read = None

    def param_specs(self):
        specs = [ParamSpec(self.name, (self.size,), init="ones")]
        if self.read_name:
            specs.append(ParamSpec(self.read_name, (self.streams,), init="ones"))
        return specs

    def load(self, tensors):
        self.weight = to_compute(tensors[self.name], self.ctx)
        if self.read_name:
            self.read = tensors[self.read_name].to(torch.float32).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, rows=None, out=None):
        M = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty(M, self.size, dtype=self.ctx.dtype, device=x.device)
        return ops.streams_norm(x, self.read, self.weight, self.eps, out, self.streams, rows)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
register_part("norm", "streams_rmsnorm", StreamsRMSNorm)
