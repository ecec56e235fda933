"""Latent attention: queries, keys and values go through low-rank latents, and the cache keeps one latent and one rotated
key part per token instead of keys and values of every head.

    cq = Wdq h / rms(Wdq h) * wq                         the query latent (q_rank wide; eps inside the root)
    q_h = Wuq_h cq = [plain (dim) | rotated (rot_dim)]    per head
    [c_raw | kr_raw] = Wdkv h;  c = c_raw / rms(c_raw) * wc (kv_rank wide);  kr = rotated(kr_raw) (rot_dim, one for all heads)
    k_h = Wuk_h c,  v_h = Wuv_h c                         (dim and vdim wide)
    score = (q_plain . k_h + q_rot . kr) * scale, causal softmax, heads concatenated, times sigmoid(Wg h), then Wo

The rotation pairs dimensions (2i, 2i + 1) of the rotated parts, i < rot_dims / 2, by the angle p * base^(-2i / rot_dims).
Only c and kr are cached: one plane of kv_rank + rot_dim columns and one "head" per token. Attention runs in the
latent's space: the query's plain part is taken there once per row (Wuk_h^T q_plain, kv_rank wide), a row's pass over
the cache reads [c | kr] rows as keys and their first kv_rank columns as values, and Wuv_h is applied to the summed
latent (csrc/latent.cu). Root mean squares, angles, scores, softmax and the gate are 32-bit; the query that enters
attention and the gated heads are rounded once each, the summed latent stays 32-bit.

A request that brings many rows (a prompt portion; bfloat16) takes the other way round, the one with fewer operations
per (row, key) pair: its latents, context and portion, are gathered from the pages and turned into the keys
[Wuk_h c | kr] and values Wuv_h c of every head by ONE tensor-core product (the weight matrix has kr's columns as an
identity block), and its rows attend over them with queries [plain | rotated] on the tensor-core kernel of
csrc/attention_masked_flash.cu, the gate in its epilogue. Both ways compute the same sums; they differ in rounding.

Several things are optional. Without a query latent (`q_rank` None) the queries are one product, q = Wq h, laid out head
by head as [plain | rotated]. Without `gate` the heads go to Wo as they are; with gate "head" the gate is one number per
head (Wg has `heads` rows) instead of one per element. With `window` a row at position i sees the keys j with
0 <= i - j < window; the cache is then of the kind "window" (pages that no later query sees go back to the pool while the
request runs), and a portion's keys and values are made from the first kept page on. With `sink` a learned number per
head joins the softmax's denominator as exp(sink_h): no key, no value, not scaled. `pairing` "half" rotates the pairs
(i, i + rot_dims / 2) instead of (2i, 2i + 1), and `rot_scaling` rescales the frequencies (ops.rope_frequencies; a
magnitude that it gives multiplies cos and sin of queries and keys alike).

params: hidden_size, heads, dim, rot_dim, vdim, q_rank (None: no query latent), kv_rank, scale, eps, rot_dims (default
rot_dim), rot_base, rot_scaling (default None), pairing (default "interleaved"), gate (True or "element", "head", False),
window (default None), sink (default False), and the tensor names dq, dq_norm, uq (or q), dkv, dkv_norm, uk, uv, g, o, sink
(`<key>_name`).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import CacheNeed, Mixer, register_part, to_compute

_DEFAULT_NAMES = dict(dq="mix.dq", dq_norm="mix.dq.norm", uq="mix.uq", q="mix.q", dkv="mix.dkv", dkv_norm="mix.dkv.norm",
                      uk="mix.uk", uv="mix.uv", g="mix.g", o="mix.o", sink="mix.sink")


class LatentAttentionMixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.rot_dim, self.vdim = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]) if p.get("q_rank") else 0, int(p["kv_rank"])
        gate = p.get("gate", True)
        if gate not in (True, False, None, "element", "head"):
            raise ValueError(f"latent attention: gate {gate!r} is not known (known: True or 'element', 'head', False)")
        self.gated, self.gate_per_head = bool(gate), gate == "head"
        self.window, self.has_sink = int(p["window"]) if p.get("window") else 0, bool(p.get("sink", False))
        self.pairing = p.get("pairing", "interleaved")
        if self.pairing not in ops.PAIRINGS:
            raise ValueError(f"latent attention: pairing {self.pairing!r} is not known (known: {sorted(ops.PAIRINGS)})")
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.rot_dims, self.rot_base = int(p.get("rot_dims", self.rot_dim)), float(p.get("rot_base", 10000.0))
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError(f"latent attention: {self.rot_dims} rotated dimensions of a rotated part of {self.rot_dim}")
        unused = ((("q",) if self.q_rank else ("dq", "dq_norm", "uq")) + (() if self.gated else ("g",))
                  + (() if self.has_sink else ("sink",)))
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items() if k not in unused}
        self.w_in = self.w_uq = self.wo = self.wuk_t = self.wuv_t = self.table = self.sink = None
        if not ctx.is_meta:
            self.table = ops.shared_rope_table(self.rot_dims, self.rot_base, ctx.max_model_len, ctx.device, p.get("rot_scaling"))

    def param_specs(self):
        n, W, H = self.names, self.hidden, self.heads
        if self.q_rank:
            specs = [ParamSpec(n["dq"], (self.q_rank, W)), ParamSpec(n["dq_norm"], (self.q_rank,), init="ones"),
                     ParamSpec(n["uq"], (H * (self.dim + self.rot_dim), self.q_rank))]
        else:
            specs = [ParamSpec(n["q"], (H * (self.dim + self.rot_dim), W))]
        specs += [ParamSpec(n["dkv"], (self.kv_rank + self.rot_dim, W)), ParamSpec(n["dkv_norm"], (self.kv_rank,), init="ones"),
                  ParamSpec(n["uk"], (H * self.dim, self.kv_rank)), ParamSpec(n["uv"], (H * self.vdim, self.kv_rank))]
        if self.gated:
            specs.append(ParamSpec(n["g"], (H if self.gate_per_head else H * self.vdim, W)))
        if self.has_sink:
            specs.append(ParamSpec(n["sink"], (H,), init="zeros"))
        return specs + [ParamSpec(n["o"], (W, H * self.vdim))]

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items()}
        mats = [t["dq"] if self.q_rank else t["q"], t["dkv"]] + ([t["g"]] if self.gated else [])
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = ops.Weight(torch.cat([m.to(dt) for m in mats], 0).contiguous())      # rows [dq or q | dkv | g]
        self.w_uq, self.wo = ops.Weight(t["uq"]) if self.q_rank else None, ops.Weight(t["o"])
        H = self.heads
        self.wuk_t = t["uk"].reshape(H, self.dim, self.kv_rank).contiguous()                      # [h][d][r]
        self.wuv_t = t["uv"].reshape(H, self.vdim, self.kv_rank).transpose(1, 2).contiguous()     # [h][r][e]
        self.wc_norm = t["dkv_norm"]
        self.sink = t["sink"].to(torch.float32).contiguous() if self.has_sink else None
        self.wq_norm = t["dq_norm"].to(self.wc_norm.dtype) if self.q_rank else None
        # for portions: [keys of every head | values of every head] = [c | kr] @ w_kv^T in one product
        self.w_kv = None
        D, Dr, E, R = self.dim, self.rot_dim, self.vdim, self.kv_rank
        if (self.ctx.dtype == torch.bfloat16 and t["uk"].dtype == torch.bfloat16 and t["uv"].dtype == torch.bfloat16
                and ops.masked_flash_supported(D + Dr, E) and (R + Dr) % 8 == 0):
            wk = torch.zeros(H, D + Dr, R + Dr, dtype=torch.bfloat16, device=t["uk"].device)
            wk[:, :D, :R] = t["uk"].reshape(H, D, R)
            wk[:, D:, R:] = torch.eye(Dr, dtype=torch.bfloat16, device=wk.device)
            wv = torch.zeros(H * E, R + Dr, dtype=torch.bfloat16, device=wk.device)
            wv[:, :R] = t["uv"]
            self.w_kv = ops.Weight(torch.cat([wk.reshape(H * (D + Dr), R + Dr), wv], 0).contiguous())

    def weight_bytes(self):
        return (self.w_in.nbytes + (self.w_uq.nbytes if self.w_uq is not None else 0) + self.wo.nbytes
                + sum(w.numel() * w.element_size() for w in (self.wuk_t, self.wuv_t)))

    def cache_need(self):
        width = self.kv_rank + self.rot_dim
        if self.window:
            return CacheNeed("window", 1, width, self.window, (("ckr", 1, width),))
        return CacheNeed("full", 1, width, 0, (("ckr", 1, width),))

    def forward(self, xn, x, batch, cache, state):
        T, H, dev = xn.shape[0], self.heads, xn.device
        Rq, R, Dr, D, E = self.q_rank, self.kv_rank, self.rot_dim, self.dim, self.vdim
        Q0 = Rq if Rq else H * (D + Dr)          # the first columns of the product: the raw query latent, or the queries
        n_gate = 0 if not self.gated else H if self.gate_per_head else H * E
        proj = torch.empty(T, Q0 + R + Dr + n_gate, dtype=torch.float32, device=dev)
        ops.linear_rows32(xn, self.w_in, proj)
        ckr = cache.planes["ckr"]
        cq = torch.empty(T, Rq, dtype=self.ctx.dtype, device=dev)
        ops.latent_prepare(proj, (0, Q0, Q0 + R), self.wq_norm, self.wc_norm, batch.positions,
                           batch.slot_maps[cache.group] if cache.write else None, self.table, self.rot_dims, self.eps, cq, ckr,
                           Rq, R, Dr, self.ctx.page_size, self.pairing)
        if Rq:
            q = torch.empty(T, H * (D + Dr), dtype=torch.float32, device=dev)
            ops.linear_rows32(cq, self.w_uq, q)
        else:
            q = proj[:, :Q0]
        gate = dict(gate=proj, gate_offset=Q0 + R + Dr, gate_per_head=self.gate_per_head) if self.gated else {}
        mask = dict(mask="window", window=self.window) if self.window else dict(mask="causal")
        att = torch.empty(T, H * E, dtype=self.ctx.dtype, device=dev)
        # requests that bring many rows: keys and values of what they can see from one product, tensor-core attention
        many = [r for r in range(batch.n_requests) if batch.h_q_len[r] >= ops.MASKED_FLASH_MIN_ROWS] \
            if self.w_kv is not None and ops.fast_kernels_on() else []
        if many:
            qb = torch.empty(T, H * (D + Dr), dtype=self.ctx.dtype, device=dev)
            ops.rope_norm_store(q, (0, 0, 0), batch.positions, None, self.table, self.rot_dims, self.pairing, False, 0.0, qb,
                                None, None, H, 1, D + Dr, E, self.ctx.page_size, rot_off=D)
            ps = self.ctx.page_size
            for r in many:
                ctx_len = batch.h_ctx_len[r]
                # with a window: from the page of the first key that the portion's first row sees
                first = (max(0, ctx_len - self.window + 1) // ps) * ps if self.window else 0
                n = ctx_len + batch.h_q_len[r] - first
                rows = torch.empty(n, R + Dr, dtype=self.ctx.dtype, device=dev)
                ops.gather_rows(ckr, batch.block_tables[cache.group][r][first // ps:], rows, n, ps)
                kv = torch.empty(n, H * (D + Dr + E), dtype=self.ctx.dtype, device=dev)
                ops.linear(rows, self.w_kv, kv)
                ops.attention_flash_tokens(qb, kv[:, :H * (D + Dr)], kv[:, H * (D + Dr):], batch, r, att, H, H, D + Dr, E,
                                           self.scale, window=self.window, first_pos=first, sink=self.sink, **gate)
            planes.record(batch, "q", qb)
            if len(many) == batch.n_requests:
                planes.record(batch, "attention", att)
                ops.linear_into_stream(att, self.wo, x)
                return None
        limit = ops.MASKED_FLASH_MIN_ROWS if many else 0
        qa = torch.empty(T, H * (R + Dr), dtype=self.ctx.dtype, device=dev)        # per head [Wuk^T q_plain | rotated part]
        ops.heads_linear(q, D + Dr, self.wuk_t, qa, R + Dr, tail=Dr, rot=self.rot_dims, positions=batch.positions,
                         table=self.table, batch=batch, row_limit=limit, pairing=self.pairing)
        lat = torch.empty(T, H * R, dtype=torch.float32, device=dev)               # per head the softmax-weighted sum of c
        ops.attention_masked(qa, ckr, ckr, batch, cache.group, lat, H, 1, R + Dr, R, self.ctx.page_size, self.scale,
                             row_limit=limit, sink=self.sink, **mask)
        ops.heads_linear(lat, R, self.wuv_t, att, E, batch=batch, row_limit=limit, **gate)
        if not many:
            planes.record(batch, "q", qa)
        planes.record(batch, "attention", att)
        ops.linear_into_stream(att, self.wo, x)
        return None


register_part("mixer", "latent_attention", LatentAttentionMixer)
