"""Arrangements of a layer's parts. "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)),
the order of the reference's attn_rows and mlp_rows (src/api.cu:1673, 1712).

A block kind declares its slots (`SLOTS`: slot name -> registry role) and builds the parts the
`LayerSpec` gives under those names; a layer that gives other names, or lacks one, is refused
with a message. Every block has an attribute `mixer`: the part whose `cache_need()` and
`state_need()` the cache manager serves."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .norm import RMSNorm
from .registry import Part, build_part, register_part, to_compute


def build_slots(block: Part, layer, slots, ctx, prefix) -> list:
    """Builds the parts of `layer` (a LayerSpec) for the slots {name: role} of a block kind, sets each as the
    attribute of its slot name on `block`, and returns them in the slots' order."""
    extra = sorted(set(layer.parts) - set(slots))
    if extra:
        raise ValueError(f"layer {layer.prefix!r}: block {layer.block!r} has no part {extra}; its parts are {sorted(slots)}")
    built = []
    for name, role in slots.items():
        part = build_part(role, layer.part(name), ctx, prefix)
        setattr(block, name, part)
        built.append(part)
    return built


class PreNormBlock(Part):
    """params: layer (the LayerSpec)."""

    SLOTS = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.parts = build_slots(self, params["layer"], self.SLOTS, ctx, prefix)

    def param_specs(self):
        return [s for p in self.parts for s in p.param_specs()]

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts)

    takes_pending = True
    takes_next_norm = True      # forward() accepts next_norm=: the norm that reads x after this layer (the next layer's first)

    @staticmethod
    def _normed(norm, x, pending, consumer, feed=None):
        if pending is None:
            # a few rows: a consumer that says so gets the norm unevaluated and folds it into its first product
            if getattr(consumer, "takes_lazy_norm", False) and hasattr(norm, "lazy"):
                lazy = norm.lazy(x, feed) if feed is not None else norm.lazy(x)
                if lazy is not None:
                    return lazy
            return norm.forward(x)
        if norm.takes_pending:
            return norm.forward(x, pending=pending)
        pending.finish()
        return norm.forward(x)

    @staticmethod
    def _feed_of(norm, producer, rows):
        """Buffers for `norm` that `producer` (the part whose last product writes the norm's input) may fill, or None."""
        if norm is None or not getattr(producer, "takes_norm_feed", False) or not hasattr(norm, "feed"):
            return None
        return norm.feed(rows)

    def forward(self, x, batch, cache, state, pending=None, next_norm=None):
        """pending: what the layer before left: a sum it has yet to add into x (kernels.ops.Pending), or the first
        norm of this layer prepared by its last product (kernels.fast.NormFeed). Returns what this layer leaves in
        the same way (None when x is complete and nothing is prepared)."""
        if planes.dumping(batch):
            return self._forward_dumped(x, batch, cache, state, pending)
        feed_in = None
        if pending is not None and not isinstance(pending, ops.Pending):
            feed_in, pending = pending, None
        rows = x.shape[0]
        xn = self._normed(self.mixer_norm, x, pending, self.mixer, feed_in)
        feed = self._feed_of(self.feed_forward_norm, self.mixer, rows)
        left = (self.mixer.forward(xn, x, batch, cache, state, norm_feed=feed) if feed is not None
                else self.mixer.forward(xn, x, batch, cache, state))
        pending = left if isinstance(left, ops.Pending) else None
        xn = self._normed(self.feed_forward_norm, x, pending, self.feed_forward, feed)
        feed = self._feed_of(next_norm, self.feed_forward, rows)
        left = (self.feed_forward.forward(xn, x, batch, norm_feed=feed) if feed is not None
                else self.feed_forward.forward(xn, x, batch))
        if isinstance(left, ops.Pending):
            return left
        return feed if feed is not None and feed.filled else None

    def _forward_dumped(self, x, batch, cache, state, pending):
        """The same layer with every sum finished and every norm evaluated where a plane is recorded (parts/planes.py)."""
        if isinstance(pending, ops.Pending):
            pending.finish()
        xn = self.mixer_norm.forward(x)
        planes.record(batch, "mixer_norm", xn)
        left = self.mixer.forward(xn, x, batch, cache, state)
        if isinstance(left, ops.Pending):
            left.finish()
        planes.record(batch, "after_mixer", x)
        xn = self.feed_forward_norm.forward(x)
        planes.record(batch, "feed_forward_norm", xn)
        left = self.feed_forward.forward(xn, x, batch)
        if isinstance(left, ops.Pending):
            left.finish()
        planes.record(batch, "after_feed_forward", x)
        return None


class ScaledPreNormBlock(Part):
    """Pre-norm with layer scale: x += s1 * mixer(norm(x)); x += s2 * feed_forward(norm(x)), s1 and s2 vectors over the
    width that multiply each sublayer's result before the sum. The feed-forward (with its norm and scale) is optional:
    a layer that gives no `feed_forward` part has the first sublayer only.

    params: layer (the LayerSpec), hidden_size, mixer_scale_name, feed_forward_scale_name (tensor names relative to the
    prefix). A part that sets `takes_out_scale` multiplies by the vector in its own last product (`out_scale=`); any
    other part writes into a zeroed buffer, which is then scaled and added here."""

    SLOTS = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    OPTIONAL = ("feed_forward_norm", "feed_forward")

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        layer = params["layer"]
        has_ff = "feed_forward" in layer.parts
        slots = {n: r for n, r in self.SLOTS.items() if has_ff or n not in self.OPTIONAL}
        self.parts = build_slots(self, layer, slots, ctx, prefix)
        if not has_ff:
            self.feed_forward = self.feed_forward_norm = None
        self.hidden = int(params.get("hidden_size", getattr(self.mixer_norm, "size", 0)))
        self.scale_names = [prefix + params.get("mixer_scale_name", "ls1")]
        if has_ff:
            self.scale_names.append(prefix + params.get("feed_forward_scale_name", "ls2"))
        self.scales = [None, None]

    def param_specs(self):
        return [s for p in self.parts for s in p.param_specs()] + [ParamSpec(n, (self.hidden,), init="ones") for n in self.scale_names]

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)
        for i, n in enumerate(self.scale_names):
            self.scales[i] = to_compute(tensors[n], self.ctx)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts) + sum(s.numel() * s.element_size() for s in self.scales if s is not None)

    def _sublayer(self, part, scale, xn, x, *rest):
        if getattr(part, "takes_out_scale", False):
            left = part.forward(xn, x, *rest, out_scale=scale)
            if isinstance(left, ops.Pending):
                left.finish()
            return
        y = torch.zeros_like(x)
        left = part.forward(xn, y, *rest)
        if isinstance(left, ops.Pending):
            left.finish()
        ops.scale_add(x, y, scale)

    def forward(self, x, batch, cache, state):
        xn = self.mixer_norm.forward(x)
        planes.record(batch, "mixer_norm", xn)
        self._sublayer(self.mixer, self.scales[0], xn, x, batch, cache, state)
        planes.record(batch, "after_mixer", x)
        if self.feed_forward is not None:
            xn = self.feed_forward_norm.forward(x)
            planes.record(batch, "feed_forward_norm", xn)
            self._sublayer(self.feed_forward, self.scales[1], xn, x, batch)
        planes.record(batch, "after_feed_forward", x)
        return None


class ParallelBlock(Part):
    """One norm, two readers: h = norm(x); x += mixer(h) + feed_forward(h). Both sublayers read the same normalised rows
    and add into the 32-bit residual stream; the feed-forward is optional (a layer that gives none has the mixer only).
    params: layer (the LayerSpec) with the parts `norm`, `mixer` and, optionally, `feed_forward`."""

    SLOTS = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        layer = params["layer"]
        has_ff = "feed_forward" in layer.parts
        self.parts = build_slots(self, layer, {n: r for n, r in self.SLOTS.items() if has_ff or n != "feed_forward"}, ctx, prefix)
        if not has_ff:
            self.feed_forward = None

    def param_specs(self):
        return [s for p in self.parts for s in p.param_specs()]

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts)

    def forward(self, x, batch, cache, state):
        h = self.norm.forward(x)
        planes.record(batch, "mixer_norm", h)
        left = self.mixer.forward(h, x, batch, cache, state)
        if isinstance(left, ops.Pending):
            left.finish()
        planes.record(batch, "after_mixer", x)
        if self.feed_forward is not None:
            left = self.feed_forward.forward(h, x, batch)
            if isinstance(left, ops.Pending):
                left.finish()
        planes.record(batch, "after_feed_forward", x)
        return None


class PreparedNorm:
    """The rows of `norm` over the residual rows as a layer left them: the layer's last write-back computed them on its
    way, so the layer that owns `norm` need not read the residual rows again."""

    def __init__(self, norm, rows):
        self.norm, self.rows = norm, rows


class HyperConnectionBlock(Part):
    """Pre-norm sublayers over several residual streams with learned mixing (hyper-connections). A token's residual row
    holds S streams x_1 .. x_S (all equal to the embedding at the start). For each sublayer (the mixer, then the
    feed-forward where the layer has one), with read weights a [S], write weights b [S], a mixing matrix M [S, S]
    (indexed [from, to]) and the model's residual multiplier m:

        u = sum_s a[s] x_s;  y = sublayer(norm(u));  x_t <- sum_s M[s, t] x_s + m * b[t] * y   for all t at once

    The read is part of the sublayer's norm (kind "streams_rmsnorm" with a `read_name`); the write-back of a sublayer and
    the read and norm of the next one are one pass over the row (also across layers: `next_norm`). With S = 1 and no
    learned weights this is the plain pre-norm residual x <- x + m * sublayer(norm(x)).

    params: layer (the LayerSpec), hidden_size, streams, residual_mult (default 1), learned (default True: the layer has
    the tensors below), mixer_write_name / mixer_mix_name / feed_forward_write_name / feed_forward_mix_name (defaults
    "hc1.out", "hc1.mix", "hc2.out", "hc2.mix", relative to the prefix)."""

    SLOTS = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    OPTIONAL = ("feed_forward_norm", "feed_forward")
    takes_pending = True
    takes_next_norm = True

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        layer = params["layer"]
        self.has_ff = "feed_forward" in layer.parts
        slots = {n: r for n, r in self.SLOTS.items() if self.has_ff or n not in self.OPTIONAL}
        self.parts = build_slots(self, layer, slots, ctx, prefix)
        if not self.has_ff:
            self.feed_forward = self.feed_forward_norm = None
        self.hidden, self.streams = int(params["hidden_size"]), int(params.get("streams", 1))
        self.mult, self.learned = float(params.get("residual_mult", 1.0)), bool(params.get("learned", True))
        subs = ["mixer"] + (["feed_forward"] if self.has_ff else [])
        dflt = dict(mixer_write="hc1.out", mixer_mix="hc1.mix", feed_forward_write="hc2.out", feed_forward_mix="hc2.mix")
        self.names = {k: prefix + params.get(k + "_name", d) for k, d in dflt.items() if k.rsplit("_", 1)[0] in subs}
        self.coef = {}

    def param_specs(self):
        specs = [s for p in self.parts for s in p.param_specs()]
        if self.learned:
            S = self.streams
            specs += [ParamSpec(n, (S,) if k.endswith("write") else (S, S), init="ones") for k, n in self.names.items()]
        return specs

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)
        if self.learned:
            self.coef = {k: tensors[n].to(torch.float32).contiguous() for k, n in self.names.items()}

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts)

    def _write(self, x, y, sub, next_norm):
        """The write-back of sublayer `sub`; with a `next_norm` of the streams kind also its rows (else None)."""
        b, M = self.coef.get(sub + "_write"), self.coef.get(sub + "_mix")
        fuse = (next_norm is not None and getattr(next_norm, "streams", None) == self.streams
                and getattr(next_norm, "size", None) == self.hidden and hasattr(next_norm, "read")
                and getattr(next_norm, "weight", None) is not None)
        if not fuse:
            ops.streams_update(x, y, b, M, self.mult, self.streams)
            return None
        out = torch.empty(y.shape[0], self.hidden, dtype=self.ctx.dtype, device=y.device)
        return ops.streams_update(x, y, b, M, self.mult, self.streams, next_norm.read, next_norm.weight, next_norm.eps, out)

    def forward(self, x, batch, cache, state, pending=None, next_norm=None):
        dumping = planes.dumping(batch)
        if isinstance(pending, ops.Pending):
            pending.finish()
        if isinstance(pending, PreparedNorm) and pending.norm is self.mixer_norm and not dumping:
            xn = pending.rows
        else:
            xn = self.mixer_norm.forward(x)
        planes.record(batch, "mixer_norm", xn)
        y = torch.zeros(xn.shape[0], self.hidden, dtype=torch.float32, device=xn.device)
        left = self.mixer.forward(xn, y, batch, cache, state)
        if isinstance(left, ops.Pending):
            left.finish()
        if dumping:
            next_norm = None
        if self.has_ff:
            xn = self._write(x, y, "mixer", None if dumping else self.feed_forward_norm)
            planes.record(batch, "after_mixer", x)
            if xn is None:
                xn = self.feed_forward_norm.forward(x)
            planes.record(batch, "feed_forward_norm", xn)
            y = torch.zeros(xn.shape[0], self.hidden, dtype=torch.float32, device=xn.device)
            left = self.feed_forward.forward(xn, y, batch)
            if isinstance(left, ops.Pending):
                left.finish()
            rows = self._write(x, y, "feed_forward", next_norm)
        else:
            rows = self._write(x, y, "mixer", next_norm)
            planes.record(batch, "after_mixer", x)
        planes.record(batch, "after_feed_forward", x)
        return PreparedNorm(next_norm, rows) if rows is not None else None


class RoundedRows:
    """What a post-norm layer leaves for the next one: the residual rows `x` as it wrote them, rounded to the compute
    element type on the way (`rows`), so that the next layer's products need no pass over x of their own."""

    def __init__(self, x, rows):
        self.x, self.rows = x, rows


class PostNormBlock(Part):
    """The norm AFTER the sum: x <- norm1(alpha * x + mixer(x)), then x <- norm2(alpha * x + feed_forward(x)). The sublayers
    read the residual rows themselves (rounded to the compute element type for their products; the 32-bit engine reads x as
    it is), not a normed copy, and alpha multiplies the residual, not the sublayer. The feed-forward with its norm is
    optional (a layer that gives no `feed_forward` part has the first half only).

    The scaled sum, the norm and the rounded copy for the next reader are one pass over the row (ops.residual_norm); a
    mixer that offers `forward_pair` (two side-by-side results that are normed and joined) has its join in the same pass.
    A norm part of another kind than the RMS norm is run as it is, on the summed rows.

    params: layer (the LayerSpec), hidden_size, alpha (default 1)."""

    SLOTS = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}
    OPTIONAL = ("feed_forward", "feed_forward_norm")
    takes_pending = True

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        layer = params["layer"]
        self.has_ff = "feed_forward" in layer.parts
        slots = {n: r for n, r in self.SLOTS.items() if self.has_ff or n not in self.OPTIONAL}
        self.parts = build_slots(self, layer, slots, ctx, prefix)
        if not self.has_ff:
            self.feed_forward = self.feed_forward_norm = None
        self.hidden, self.alpha = int(params["hidden_size"]), float(params.get("alpha", 1.0))

    def param_specs(self):
        return [s for p in self.parts for s in p.param_specs()]

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts)

    def _rows(self, x, carry):
        """The rows the sublayers' products read: x itself in the 32-bit engine, else its rounded copy."""
        if self.ctx.dtype == torch.float32:
            return x
        if isinstance(carry, RoundedRows) and carry.x is x:
            return carry.rows
        return ops.convert(x, self.ctx.dtype)

    def _close(self, x, norm, y=None, pair=None):
        """x <- norm(alpha * x + y + pair); returns the rounded copy of the new x (None in the 32-bit engine)."""
        rounded = None if self.ctx.dtype == torch.float32 else torch.empty(x.shape, dtype=self.ctx.dtype, device=x.device)
        w = getattr(norm, "weight", None)
        if isinstance(norm, RMSNorm) and w is not None and w.dtype == torch.float32:
            ops.residual_norm(x, y, pair, self.alpha, w, norm.eps, rounded)
            return rounded
        ops.residual_norm(x, y, pair, self.alpha)
        x.copy_(norm.forward(x, out=torch.empty_like(x)))
        return None if rounded is None else ops.convert(x, self.ctx.dtype)

    def forward(self, x, batch, cache, state, pending=None):
        if isinstance(pending, ops.Pending):
            pending.finish()
        h = self._rows(x, pending)
        if hasattr(self.mixer, "forward_pair"):
            h = self._close(x, self.mixer_norm, pair=self.mixer.forward_pair(h, batch, cache, state))
        else:
            y = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            left = self.mixer.forward(h, y, batch, cache, state)
            if isinstance(left, ops.Pending):
                left.finish()
            h = self._close(x, self.mixer_norm, y=y)
        planes.record(batch, "after_mixer", x)
        if self.has_ff:
            y = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            left = self.feed_forward.forward(x if h is None else h, y, batch)
            if isinstance(left, ops.Pending):
                left.finish()
            h = self._close(x, self.feed_forward_norm, y=y)
        planes.record(batch, "after_feed_forward", x)
        return None if h is None or planes.dumping(batch) else RoundedRows(x, h)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "post_norm", PostNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "pre_norm_scaled", ScaledPreNormBlock)
register_part("block", "hyper_connections", HyperConnectionBlock)
