"""Token embedding (a row gather without scaling, src/kernels.cuh:1877-1881) into the 32-bit
residual stream, and the output head (logits = xn W^T, W the embedding table when tied,
src/api.cu:1367, 1795-1812) producing 32-bit logits."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from .registry import Part, build_part, register_part, to_compute


class TokenEmbedding(Part):
    """params: name, vocab_size, hidden_size."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.name, self.vocab, self.hidden = params["name"], int(params["vocab_size"]), int(params["hidden_size"])
        self.table = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.table = to_compute(tensors[self.name], self.ctx)

    def forward(self, tokens):
        x = torch.empty(tokens.numel(), self.hidden, dtype=torch.float32, device=tokens.device)
        return ops.embedding(self.table, tokens, x)


class ScaledPositionEmbedding(Part):
    """x = table[token] * scale + position_table[position]: a scaled token embedding and a learned vector per absolute
    position (not scaled). params: name, vocab_size, hidden_size, scale (default 1), position_name (absent: no position
    vectors), max_position. The decoder hands it the step's positions (`takes_positions`)."""

    takes_positions = True

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.name, self.vocab, self.hidden = params["name"], int(params["vocab_size"]), int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        self.position_name = params.get("position_name")
        self.max_position = int(params.get("max_position", 0))
        self.table = self.position_table = None

    def param_specs(self):
        specs = [ParamSpec(self.name, (self.vocab, self.hidden))]
        if self.position_name:
            specs.append(ParamSpec(self.position_name, (self.max_position, self.hidden)))
        return specs

    def load(self, tensors):
        self.table = to_compute(tensors[self.name], self.ctx)
        if self.position_name:
            self.position_table = to_compute(tensors[self.position_name], self.ctx).to(self.table.dtype)

    def forward(self, tokens, positions):
        x = torch.empty(tokens.numel(), self.hidden, dtype=torch.float32, device=tokens.device)
        return ops.embedding_scaled(self.table, tokens, x, self.scale, self.position_table, positions)


class NormedTokenEmbedding(Part):
    """x = norm(table[token]): a token embedding whose rows go through a norm of the model's kind before they enter the
    32-bit residual stream (the norm's result stays 32-bit). params: name, vocab_size, hidden_size, norm (the PartSpec
    of a norm over hidden_size)."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.name, self.vocab, self.hidden = params["name"], int(params["vocab_size"]), int(params["hidden_size"])
        self.norm = build_part("norm", params["norm"], ctx, prefix)
        self.table = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.hidden))] + self.norm.param_specs()

    def load(self, tensors):
        self.table = to_compute(tensors[self.name], self.ctx)
        self.norm.load(tensors)

    def forward(self, tokens):
        raw = torch.empty(tokens.numel(), self.hidden, dtype=torch.float32, device=tokens.device)
        ops.embedding(self.table, tokens, raw)
        return self.norm.forward(raw, out=torch.empty_like(raw))


class StreamsTokenEmbedding(Part):
    """A token embedding into `streams` residual streams: every token's row of the 32-bit stream tensor holds `streams`
    copies of its embedding, [T, streams * hidden_size]. params: name, vocab_size, hidden_size, streams."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.name, self.vocab, self.hidden = params["name"], int(params["vocab_size"]), int(params["hidden_size"])
        self.streams = int(params["streams"])
        self.table = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.table = to_compute(tensors[self.name], self.ctx)

    def forward(self, tokens):
        x = torch.empty(tokens.numel(), self.hidden, dtype=torch.float32, device=tokens.device)
        ops.embedding(self.table, tokens, x)
        if self.streams == 1:
            return x
        return ops.streams_expand(x, torch.empty(tokens.numel(), self.streams * self.hidden, dtype=torch.float32,
                                                 device=tokens.device), self.streams)


class LMHead(Part):
    """params: name (its own tensor) or tied_to (the embedding's tensor name), vocab_size, hidden_size, scale (multiplies
    the 32-bit logits; default 1)."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.tied = params.get("tied_to")
        self.name = self.tied or params["name"]
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        self.weight = None

    def param_specs(self):
        return [] if self.tied else [ParamSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.weight = ops.Weight(to_compute(tensors[self.name], self.ctx))

    def weight_bytes(self):
        return self.weight.nbytes

    def forward(self, xn):
        logits = torch.empty(xn.shape[0], self.vocab, dtype=torch.float32, device=xn.device)
        if xn.shape[0]:
            ops.linear(xn, self.weight, logits)
            if self.scale != 1.0:
                ops.scale_bias_rows(logits, self.scale)
        return logits


register_part("embedding", "token", TokenEmbedding)
register_part("embedding", "token_position", ScaledPositionEmbedding)
register_part("embedding", "token_normed", NormedTokenEmbedding)
register_part("embedding", "token_streams", StreamsTokenEmbedding)
register_part("head", "linear", LMHead)
