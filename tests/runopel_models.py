"""Small Runopel configurations of the tests' own, with weights drawn so that faults show: matrices of unit gain, decays
from nearly none to strong, step sizes that move, stream weights away from the identity, norm weights away from 1, biases
away from 0, router rows large enough that the scores spread."""
from __future__ import annotations

import json
import math
import os

import torch

import plain_runopel as plain


def ssm(heads, vdim, state, groups=1, norm_groups=1, conv=4, mlp=None):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv),
                mlp=mlp)


def latent(heads, dim, rot_dim, vdim, kv_rank, window=None, mlp=None, base=10000.0, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale or 1.0 / math.sqrt(dim + rot_dim),
             rot=dict(base=base, dims=rot_dim))
    if window is not None:
        m["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def dense(ff, limit=2.0):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def model(vocab, width, layers, streams=None, mult=1.0, logit_scale=1.0, eps=1e-5, max_positions=None):
    d = dict(architecture="Runopel", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, logit_scale=logit_scale,
             layers=layers)
    if streams is not None:
        d["streams"] = streams
    if max_positions:
        d["max_positions"] = max_positions
    return d


# A: recurrent first; three streams; a window of 24 (a page and a half); two of five experts; a layer without a feed-forward
A = model(160, 64, [ssm(4, 16, 8, groups=2, norm_groups=2, mlp=dense(96)), latent(3, 16, 8, 24, 40, window=24, mlp=moe(32, 5, 2)),
                    ssm(2, 24, 16, conv=2), latent(2, 8, 16, 8, 32, window=24, mlp=dense(48, limit=0.7))],
          streams=3, mult=0.7, logit_scale=0.25, max_positions=700)
# B: latent first with a window of ONE token (a row sees itself only); ONE stream with learned weights; every head its own
#    group; one expert of one; a convolution of one tap (no carried inputs) and one of seven; a layer without a mask
B = model(97, 48, [latent(3, 8, 8, 8, 24, window=1, mlp=moe(40, 1, 1)), ssm(3, 16, 12, groups=3, norm_groups=3, conv=1, mlp=dense(56)),
                   latent(1, 24, 12, 40, 16, mlp=moe(24, 3, 3)), ssm(1, 48, 40, conv=7)],
          streams=1, mult=1.0, logit_scale=1.0, eps=1e-6, max_positions=600)
# C: wider, no streams at all (the plain residual); windows that cross pages and key tiles (70, 200); heads of 64 x 128
#    and 32 x 64; sixteen experts of which four
C = model(211, 128, [ssm(2, 64, 128, mlp=moe(64, 16, 4)), latent(8, 48, 16, 32, 96, window=70, mlp=dense(208, limit=7.0)),
                     ssm(8, 32, 64, groups=2, norm_groups=4, conv=3), latent(4, 64, 32, 48, 96, window=200, mlp=moe(96, 4, 2))],
          mult=0.5, logit_scale=2.0, max_positions=900)
# D: sizes no vectorised kernel takes: a width that is no multiple of 4, heads of 10 and 6 and 7, a latent of 20, four streams
D = model(90, 50, [latent(2, 10, 6, 6, 20, window=5, mlp=dense(30)), ssm(3, 6, 7, conv=5, mlp=moe(22, 3, 2)), ssm(2, 10, 5, groups=2, norm_groups=5)],
          streams=4, mult=1.3, logit_scale=0.8, max_positions=300)

MODELS = {"a": A, "b": B, "c": C, "d": D}


def draw_weights(config: dict, seed: int, dtype=torch.bfloat16, decisive_routers=None):
    """{name: tensor} for `config` from the product's own list of tensors, rounded to `dtype` (so that the engine and the
    plain implementation start from the same numbers).

    decisive_routers (default: when dtype is bfloat16): with random routers two scores nearly tie at a few positions of
    every sequence, rounded inputs then choose another expert than exact ones, and a recurrent layer carries the
    difference to every later position. So the first E channels of the width (E the largest number of experts) carry a
    code that only the embedding writes: per token a permutation of E evenly spaced levels; no mixer or feed-forward
    writes into these channels (those rows of their last matrices are zero), the norm before a routed layer leaves them
    as they are, and router row e reads channel e alone. The experts' order then depends on the token only, with gaps of
    several percent between neighbours, and the scores still differ from expert to expert and from token to token."""
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.parts.spec import spec_param_specs

    c = config_from_dict(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    if decisive_routers is None:
        decisive_routers = dtype == torch.bfloat16
    code = max([L["mlp"]["router"]["experts"] for L in config["layers"] if (L.get("mlp") or {}).get("kind") == "moe"], default=0)
    code = code if decisive_routers else 0
    for s in spec_param_specs(get_architecture(c.architecture).build_spec(c)):
        n, shape = s.name, tuple(s.shape)
        rnd = torch.randn(shape, generator=g)
        leaf = n.split(".", 1)[1] if n.startswith("l") and "." in n else n
        if n == "embed":
            t = rnd * 0.7
        elif leaf in ("hc1.in", "hc2.in"):
            t = 1.0 / shape[0] + 0.3 * rnd
        elif leaf in ("hc1.out", "hc2.out"):
            t = 1.0 + 0.4 * rnd
        elif leaf in ("hc1.mix", "hc2.mix"):
            t = torch.eye(shape[0]) + 0.25 * rnd
        elif leaf == "mix.A_log":
            t = torch.rand(shape, generator=g) * 5.0 - 4.0          # decays from exp(-0.02 dt) to exp(-2.7 dt)
        elif leaf == "mix.dt_bias":
            t = rnd
        elif leaf == "mix.D":
            t = 1.0 + 0.5 * rnd
        elif leaf == "mix.conv":
            t = 0.6 * rnd
        elif leaf == "mlp.router":
            t = rnd * (3.0 / math.sqrt(shape[1]))
        elif leaf.startswith("mlp.e") and leaf.endswith(".down"):
            t = rnd * (1.0 / math.sqrt(shape[1]))
        elif len(shape) == 2:
            t = rnd * (1.2 / math.sqrt(shape[1]))
        elif leaf.endswith(".b"):
            t = 0.5 * rnd
        else:                                                       # norm weights
            t = 1.0 + 0.2 * rnd
        if code:
            if n == "embed":
                for tok in range(shape[0]):
                    t[tok, :code] = (torch.randperm(code, generator=g) + 0.5) * (2.0 / code)
            elif leaf == "mlp.router":
                t = torch.zeros(shape)
                t[:, :shape[0]] = 2.5 * torch.eye(shape[0])
            elif leaf == "norm2":
                t[:code] = 1.0
            elif leaf in ("mix.o", "mlp.down", "mlp.down.b") or (leaf.startswith("mlp.e") and leaf.endswith(".down")):
                t[:code] = 0.0
        out[n] = t.to(dtype)
    return out


def make_folder(folder, which, seed=1, dtype=torch.bfloat16):
    from hipinfer_b200.weights.safetensors_io import save_safetensors

    cfg = MODELS[which] if isinstance(which, str) else which
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    w = draw_weights(cfg, seed, dtype)
    save_safetensors(w, os.path.join(folder, "model.safetensors"), {"format": "pt"})
    return str(folder), cfg, w


class PlainRunopel:
    """The plain implementation with the interface the engine tests use: logits of every position of a sequence; a call
    continues the sequence of the calls before it (by running the whole sequence again), `reset` starts a new one."""

    def __init__(self, cfg, weights):
        self.cfg, self.w, self.tokens = cfg, weights, []

    def reset(self):
        self.tokens = []

    def forward(self, tokens):
        n = len(self.tokens)
        self.tokens = self.tokens + list(tokens)
        return plain.forward(self.cfg, self.w, self.tokens)[n:].float()


def sensitivity(cfg, weights, tokens, ref=None):
    """Per position, how far the plain logits move (largest difference over the vocabulary, over the largest logit) when
    every sublayer's input and result are rounded to bfloat16: large where a norm divides by nearly nothing or sums cancel."""
    ref = plain.forward(cfg, weights, tokens) if ref is None else ref.double()
    got = plain.forward(cfg, weights, tokens, round_to=torch.bfloat16)
    return ((got - ref).abs().amax(-1) / ref.abs().max()).float()
