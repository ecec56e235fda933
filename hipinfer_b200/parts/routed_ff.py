"""A routed feed-forward (mixture of experts): E small gated feed-forward layers without biases, of which every token
runs `top`.

    s = sigmoid(Wr h)                             router scores, 32-bit sums
    the `top` largest s choose the experts (ties: the lower index); the weights are the chosen scores, not renormalised
    out = sum over the chosen e of Wdown_e (silu(Wgate_e v) * (Wup_e v)),  v = s_e h     the score multiplies the INPUT

Without biases Wgate_e (s h) = s (Wgate_e h): the products run on h and the score enters the activation in 32-bit.

A second form is chosen by parameters: `router_bias` adds a bias to the router's logits; `score` "softmax_chosen" lets the
`top` largest LOGITS choose and takes as weights the softmax over the chosen logits alone; `weight_at` "output" multiplies
the expert's RESULT by the weight (brought in at the activation too: the down product is linear).
Steps of single rows (decoding) run on the device alone (csrc/moe.cu), so they replay from a CUDA graph: a few rows one
by one, more of them sorted by expert so that an expert's weights are read once for all of its rows. A step with prompt
portions sorts its (row, choice) pairs by expert and gives each expert's block of rows to the ordinary products (the
tensor-core kernels in bfloat16), for which the host reads the experts' row counts once a layer.

params: hidden_size, experts, top, expert_size, score (default "sigmoid"), weight_at (default "input"), router_bias
(default False), router_name (default "mlp.router"), router_bias_name (default "mlp.router.b"), expert_prefix (default
"mlp.e": expert i's tensors are <expert_prefix><i>.gate / .up / .down).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Part, register_part, to_compute

SORTED_MIN_PAIRS = 64     # fewer (row, choice) pairs than this never go to the ordinary products
GROUPED_MIN_PAIRS = 20    # fewer than this run row by row; from here on an expert's rows share one pass over its weights


class RoutedFF(Part):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.hidden, self.experts, self.top = int(params["hidden_size"]), int(params["experts"]), int(params["top"])
        self.inter = int(params["expert_size"])
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"routed feed-forward: top {self.top} of {self.experts} experts")
        self.score, self.weight_at = params.get("score", "sigmoid"), params.get("weight_at", "input")
        if self.score not in ops.MOE_SCORES or self.weight_at not in ("input", "output"):
            raise ValueError(f"routed feed-forward: score {self.score!r} (known: {sorted(ops.MOE_SCORES)}), weight_at "
                             f"{self.weight_at!r} (known: 'input', 'output')")
        self.at_output = self.weight_at == "output"
        self.router_name = prefix + params.get("router_name", "mlp.router")
        self.router_bias_name = prefix + params.get("router_bias_name", "mlp.router.b") if params.get("router_bias") else None
        self.router_bias = None
        self.expert_prefix = prefix + params.get("expert_prefix", "mlp.e")
        self.router = self.wgu = self.wdown = None

    def _expert(self, i, key):
        return f"{self.expert_prefix}{i}.{key}"

    def param_specs(self):
        specs = [ParamSpec(self.router_name, (self.experts, self.hidden))]
        if self.router_bias_name:
            specs.append(ParamSpec(self.router_bias_name, (self.experts,), init="zeros"))
        for i in range(self.experts):
            specs += [ParamSpec(self._expert(i, "gate"), (self.inter, self.hidden)),
                      ParamSpec(self._expert(i, "up"), (self.inter, self.hidden)),
                      ParamSpec(self._expert(i, "down"), (self.hidden, self.inter))]
        return specs

    def load(self, tensors):
        t = lambda name: to_compute(tensors[name], self.ctx)
        self.router = t(self.router_name)
        if self.router_bias_name:
            self.router_bias = t(self.router_bias_name).to(self.router.dtype).contiguous()
        mats = [t(self._expert(i, k)) for i in range(self.experts) for k in ("gate", "up", "down")]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        E, F, W = self.experts, self.inter, self.hidden
        self.wgu = torch.stack([torch.cat([mats[3 * i].to(dt), mats[3 * i + 1].to(dt)], 0) for i in range(E)], 0).contiguous()
        self.wdown = torch.stack([mats[3 * i + 2].to(dt) for i in range(E)], 0).contiguous()      # [E, W, F]
        assert self.wgu.shape == (E, 2 * F, W) and self.wdown.shape == (E, W, F)
        self.w_gu_e = [ops.Weight(self.wgu[i]) for i in range(E)]
        self.w_down_e = [ops.Weight(self.wdown[i]) for i in range(E)]

    def weight_bytes(self):
        """What a single row reads: the router and `top` experts."""
        per = (self.wgu.numel() + self.wdown.numel()) * self.wgu.element_size() // self.experts
        return self.router.numel() * self.router.element_size() + self.top * per

    def forward(self, xn, x, batch):
        T, top, F = xn.shape[0], self.top, self.inter
        expert, score = ops.moe_route(xn, self.router, top, self.router_bias, self.score)
        if T * top < GROUPED_MIN_PAIRS:
            ops.moe_rows(xn, self.wgu, self.wdown, expert, score, x, self.at_output)
            return None
        offsets, pos, src = ops.moe_sort(expert, self.experts)
        if getattr(batch, "max_q_len", 1) <= 1 or T * top < SORTED_MIN_PAIRS:
            gu = torch.empty(T * top, 2 * F, dtype=torch.float32, device=xn.device)
            ops.moe_grouped(xn, src, top, self.wgu, offsets, gu)
            act = torch.empty(T * top, F, dtype=self.ctx.dtype, device=xn.device)
            ops.moe_act(gu, src, score, act, self.at_output)
            planes.record(batch, "activation", act)
            ys = torch.empty(T * top, self.hidden, dtype=torch.float32, device=xn.device)
            ops.moe_grouped(act, None, 1, self.wdown, offsets, ys)
            ops.moe_combine(ys, pos, x, top)
            return None
        xs = ops.moe_gather(xn, src, top)
        bounds = offsets.tolist()                      # the one read by the host: how many rows each expert has
        gu = torch.empty(T * top, 2 * F, dtype=torch.float32, device=xn.device)
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.linear(xs[lo:hi], self.w_gu_e[e], gu[lo:hi])
        act = torch.empty(T * top, F, dtype=self.ctx.dtype, device=xn.device)
        ops.moe_act(gu, src, score, act, self.at_output)
        planes.record(batch, "activation", act)
        ys = torch.empty(T * top, self.hidden, dtype=torch.float32, device=xn.device)
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.linear(act[lo:hi], self.w_down_e[e], ys[lo:hi])
        ops.moe_combine(ys, pos, x, top)
        return None


register_part("feed_forward", "routed", RoutedFF)
