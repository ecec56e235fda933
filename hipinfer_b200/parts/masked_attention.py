"""Grouped-query attention over the paged cache with its mask, softmax and gate chosen by parameters.

    q, k, v = Wq h, Wk h, Wv h                         (heads x dim, kv_heads x dim, kv_heads x vdim; no biases)
    with row_norm: q <- q / rms(q) * wq, k <- k / rms(k) * wk, each over its WHOLE row (all heads at once, before they are
                   split into heads and before the rotation; eps inside the root; a weight per column)
    q, k rotated on their first `rot_dims` dimensions   (pairing "half": (i, i + rot_dims / 2); "interleaved": (2i, 2i + 1))
    q, k divided by their root mean square over dim     (with unit_norm; eps inside the root, no weight)
    score = q . k * scale over the keys the mask shows:
        "causal"   every j <= i
        "window"   j <= i and (i - j < window or j < keep_first)
        "chunk"    j <= i and floor(i / chunk) == floor(j / chunk), chunks counted from position 0 of the sequence
    softmax; with `sink` a learned number per head joins the denominator as exp(sink) (no key, no value, not scaled)
    head h's result times sigmoid(Wg h): one number per head (gate "head") or per element (gate "element")
    out = Wo concat(heads)

Query head h reads kv head h // (heads / kv_heads). The cache keeps keys after rotation and norm, and values. A mixer
with `reads_cache` has no key/value projections: it attends, with its own queries, mask and the rest, over the cache of
the layer the model's run order names. What the cache retains is given apart from the mask (`cache_chunks`: the chunk
sizes of every layer that reads it; empty: everything), because the layers that share a cache may look back differently
far. Rotation angles, the unit norm, scores, softmax and the gate are 32-bit; q, k, v are rounded once.

params: hidden_size, heads, kv_heads, dim, vdim, scale, eps, rot_dims, rot_base, rot_scaling (ops.rope_frequencies),
pairing, unit_norm, row_norm, mask, window, keep_first, chunk, sink, gate, reads_cache, cache_chunks, cache_keep_all (a
window's cache keeps everything: a reader looks back further), and the tensor names q, k, v, g, o, sink, q_norm, k_norm
(`<key>_name`).
"""
from __future__ import annotations

import torch

from ..cache import register_retention
from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import CacheNeed, Mixer, register_part, to_compute

_DEFAULT_NAMES = dict(q="mix.q", k="mix.k", v="mix.v", g="mix.g", o="mix.o", sink="mix.sink", q_norm="mix.q.norm",
                      k_norm="mix.k.norm")


def _chunks_dead(spec, q):
    """Retention of a cache whose readers all look back to the start of their own chunk: dead is what lies before the
    earliest of those starts. The sizes are in `extra` under "chunks"."""
    sizes = dict(spec.extra).get("chunks", ())
    if not sizes:
        return ()
    return ((0, min((q // int(c)) * int(c) for c in sizes)),)


register_retention("chunks", _chunks_dead)


class MaskedAttentionMixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads, self.dim, self.vdim = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 0.0))
        self.rot_dims, self.rot_base = int(p.get("rot_dims") or 0), float(p.get("rot_base") or 10000.0)
        self.pairing = p.get("pairing", "half")
        if self.rot_dims % 2 or self.rot_dims > self.dim or self.pairing not in ops.PAIRINGS:
            raise ValueError(f"attention: {self.rot_dims} rotated dimensions ({self.pairing!r}) of a head of {self.dim}")
        self.unit_norm, self.row_norm = bool(p.get("unit_norm", False)), bool(p.get("row_norm", False))
        self.mask = p.get("mask") or "causal"
        if self.mask not in ops.MASKS:
            raise ValueError(f"attention: mask {self.mask!r} is not known (known: {sorted(ops.MASKS)})")
        self.window, self.keep_first, self.chunk = int(p.get("window") or 0), int(p.get("keep_first") or 0), int(p.get("chunk") or 0)
        if (self.mask == "window" and self.window <= 0) or (self.mask == "chunk" and self.chunk <= 0):
            raise ValueError(f"attention: mask {self.mask!r} needs its size")
        self.has_sink = bool(p.get("sink", False))
        self.gate = p.get("gate") or "none"
        if self.gate not in ("none", "head", "element"):
            raise ValueError(f"attention: gate {self.gate!r} is not known (known: 'none', 'head', 'element')")
        self.reads_cache = bool(p.get("reads_cache", False))
        own = (self.chunk,) if self.mask == "chunk" else ()
        self.cache_chunks = tuple(int(c) for c in p["cache_chunks"]) if "cache_chunks" in p else own
        if self.mask != "chunk" and self.cache_chunks:
            raise ValueError("attention: the cache retains less than the mask sees")
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items()}
        self.w_in = self.wo = self.sink = self.table = self.row_norm_w = None
        if not ctx.is_meta:
            self.table = ops.shared_rope_table(self.rot_dims, self.rot_base, ctx.max_model_len, ctx.device, p.get("rot_scaling"))

    @property
    def n_q(self):
        return self.heads * self.dim

    @property
    def n_kv(self):
        return 0 if self.reads_cache else self.kv_heads * (self.dim + self.vdim)

    @property
    def n_gate(self):
        return {"none": 0, "head": self.heads, "element": self.heads * self.vdim}[self.gate]

    def param_specs(self):
        n, W = self.names, self.hidden
        specs = [ParamSpec(n["q"], (self.n_q, W))]
        if not self.reads_cache:
            specs += [ParamSpec(n["k"], (self.kv_heads * self.dim, W)), ParamSpec(n["v"], (self.kv_heads * self.vdim, W))]
        if self.row_norm:
            specs.append(ParamSpec(n["q_norm"], (self.n_q,), init="ones"))
            if not self.reads_cache:
                specs.append(ParamSpec(n["k_norm"], (self.kv_heads * self.dim,), init="ones"))
        if self.has_sink:
            specs.append(ParamSpec(n["sink"], (self.heads,), init="zeros"))
        if self.n_gate:
            specs.append(ParamSpec(n["g"], (self.n_gate, W)))
        specs.append(ParamSpec(n["o"], (W, self.heads * self.vdim)))
        return specs

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items() if n in tensors}
        mats = [t["q"]] + ([] if self.reads_cache else [t["k"], t["v"]]) + ([t["g"]] if self.n_gate else [])
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = ops.Weight(torch.cat([m.to(dt) for m in mats], 0).contiguous())     # rows [q | k | v | g] or [q | g]
        self.wo = ops.Weight(t["o"])
        self.sink = t["sink"].to(torch.float32).contiguous() if self.has_sink else None
        if self.row_norm:
            wq = t["q_norm"].to(torch.float32).contiguous()
            self.row_norm_w = (wq, wq if self.reads_cache else t["k_norm"].to(torch.float32).contiguous())

    def weight_bytes(self):
        return self.w_in.nbytes + self.wo.nbytes

    def cache_need(self):
        planes_ = (("k", self.kv_heads, self.dim), ("v", self.kv_heads, self.vdim))
        if self.cache_chunks:
            return CacheNeed("chunks", self.kv_heads, self.dim, 0, planes_, (("chunks", tuple(sorted(set(self.cache_chunks)))),))
        if self.mask == "window" and not self.params.get("cache_keep_all", False):
            return CacheNeed("window_keep_first", self.kv_heads, self.dim, self.window, planes_, (("keep_first", self.keep_first),))
        return CacheNeed("full", self.kv_heads, self.dim, 0, planes_)

    def forward(self, xn, x, batch, cache, state):
        T = xn.shape[0]
        proj = torch.empty(T, self.n_q + self.n_kv + self.n_gate, dtype=torch.float32, device=xn.device)
        ops.linear_rows32(xn, self.w_in, proj)
        q = torch.empty(T, self.n_q, dtype=self.ctx.dtype, device=xn.device)
        write = cache.write and not self.reads_cache
        ops.rope_norm_store(proj, (0, self.n_q, self.n_q + self.kv_heads * self.dim), batch.positions,
                            batch.slot_maps[cache.group] if write else None, self.table, self.rot_dims, self.pairing,
                            self.unit_norm, self.eps, q, cache.k, cache.v, self.heads, self.kv_heads, self.dim, self.vdim,
                            self.ctx.page_size, row_norm=self.row_norm_w, row_norm_eps=self.eps)
        att = torch.empty(T, self.heads * self.vdim, dtype=self.ctx.dtype, device=xn.device)
        ops.attention_masked(q, cache.k, cache.v, batch, cache.group, att, self.heads, self.kv_heads, self.dim, self.vdim,
                             self.ctx.page_size, self.scale, self.mask, self.window, self.keep_first, self.chunk, self.sink,
                             gate=proj if self.n_gate else None, gate_offset=self.n_q + self.n_kv,
                             gate_per_head=self.gate == "head")
        planes.record(batch, "q", q)
        planes.record(batch, "attention", att)
        ops.linear_into_stream(att, self.wo, x)
        return None


register_part("mixer", "masked_attention", MaskedAttentionMixer)
