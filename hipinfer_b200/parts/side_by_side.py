"""Two sequence mixers side by side: both read the same rows, each result is divided by its root mean square over the
model's width (eps inside the root) and multiplied by a weight of its own, and the mixer's result is `mix` times their sum:

    out = mix * (left(h) / rms(left(h)) * w_left + right(h) / rms(right(h)) * w_right)

The two mixers are any registered kinds (their PartSpecs are parameters). At most one of them may keep a paged cache; the
per-request state of both lives in the request's state slot under the names "left.<name>" and "right.<name>". A block that
joins sums itself (parts/block.py, "post_norm") asks for the two raw results with `forward_pair` and does the norms and
the join in its own pass over the row; `forward` is the same for any other block.

params: hidden_size, left, right (PartSpecs of kind mixer), eps, mix (default 0.5), left_norm_name, right_norm_name
(defaults "mix.left.out", "mix.right.out", relative to the prefix).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from .registry import Mixer, build_part, register_part, to_compute


class SideBySideMixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.eps, self.mix = int(params["hidden_size"]), float(params["eps"]), float(params.get("mix", 0.5))
        self.left = build_part("mixer", params["left"], ctx, prefix)
        self.right = build_part("mixer", params["right"], ctx, prefix)
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ValueError("side-by-side mixers: at most one of the two may keep a paged cache")
        self.norm_names = (prefix + params.get("left_norm_name", "mix.left.out"),
                           prefix + params.get("right_norm_name", "mix.right.out"))
        self.w_left = self.w_right = None

    def param_specs(self):
        return (self.left.param_specs() + self.right.param_specs()
                + [ParamSpec(n, (self.hidden,), init="ones") for n in self.norm_names])

    def load(self, tensors):
        self.left.load(tensors)
        self.right.load(tensors)
        self.w_left, self.w_right = (to_compute(tensors[n], self.ctx) for n in self.norm_names)
        if self.w_left.dtype != self.w_right.dtype:
            self.w_left, self.w_right = self.w_left.to(torch.float32), self.w_right.to(torch.float32)

    def weight_bytes(self):
        return (self.left.weight_bytes() + self.right.weight_bytes()
                + sum(w.numel() * w.element_size() for w in (self.w_left, self.w_right)))

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self):
        need = {f"left.{k}": v for k, v in self.left.state_need().items()}
        need.update({f"right.{k}": v for k, v in self.right.state_need().items()})
        return need

    def forward_pair(self, xn, batch, cache, state) -> "ops.NormedPair":
        """The two raw results and how they are to be joined, for a caller that joins them on its own way over the row."""
        state = state or {}
        out = []
        for side, part in (("left.", self.left), ("right.", self.right)):
            y = torch.zeros(xn.shape[0], self.hidden, dtype=torch.float32, device=xn.device)
            own = {k[len(side):]: v for k, v in state.items() if k.startswith(side)}
            left = part.forward(xn, y, batch, cache if part.cache_need() is not None else None, own)
            if isinstance(left, ops.Pending):
                left.finish()
            out.append(y)
        return ops.NormedPair(out[0], out[1], self.w_left, self.w_right, self.mix, self.eps)

    def forward(self, xn, x, batch, cache, state):
        ops.residual_norm(x, pair=self.forward_pair(xn, batch, cache, state))
        return None


register_part("mixer", "side_by_side", SideBySideMixer)
