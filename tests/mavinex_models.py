"""Small Mavinex configurations of the tests' own, with weights drawn so that faults show: matrices of unit gain, decays
from nearly none to strong, step sizes that move, norm weights away from their neutral value, sinks that matter, router
biases that move the choice."""
from __future__ import annotations

import json
import math
import os

import torch

import plain_mavinex as plain


def bands(factor, original, low=1.0, high=4.0):
    return dict(factor=factor, low=low, high=high, original=original)


def yarn(factor, original, fast=32.0, slow=1.0):
    return dict(factor=factor, original=original, fast=fast, slow=slow)


def attention(heads, kv_heads, dim, vdim, window=None, rot_dims=None, base=10000.0, scaling=None, scale=None):
    rot = dict(base=base, dims=dim if rot_dims is None else rot_dims)
    if scaling:
        rot["scaling"] = scaling
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or 1.0 / math.sqrt(dim), rot=rot)
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def scan(inner, state, dt_rank, conv=4):
    return dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv)


def parallel(left, right, mlp=None, weights_of=None):
    d = dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def latent(heads, dim, rot_dim, vdim, kv_rank, window=None, mlp=None, base=10000.0, scaling=None, scale=None, weights_of=None):
    rot = dict(base=base, dims=rot_dim)
    if scaling:
        rot["scaling"] = scaling
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale or 1.0 / math.sqrt(dim + rot_dim), rot=rot)
    if window is not None:
        m["mask"] = dict(size=window)
    d = dict(type="latent_attention", mixer=m, mlp=mlp)
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def model(vocab, width, layers, alpha=1.0, embed_scale=1.0, eps=1e-5, max_positions=None):
    d = dict(architecture="Mavinex", vocab=vocab, width=width, norm=dict(eps=eps), postln_alpha=alpha,
             embedding=dict(scale=embed_scale), layers=layers)
    if max_positions:
        d["max_positions"] = max_positions
    return d


def repeat(layer, weights_of):
    d = json.loads(json.dumps(layer))
    d["weights_of"] = weights_of
    return d


# A: a side-by-side layer first, run three times in all (layers 1 and 3 use layer 0's tensors); groups of two heads, values
#    wider than keys, a window of 24 (a page and a half), rotation over part of the head, both scalings; two of five experts
_A0 = parallel(attention(4, 2, 16, 24, window=24, rot_dims=8, scaling=bands(4.0, 64)), scan(48, 8, 5), mlp=moe(32, 5, 2))
A = model(160, 64, [_A0, repeat(_A0, 0), latent(3, 16, 8, 24, 40, window=40, scaling=yarn(4.0, 32), mlp=moe(24, 3, 3)), repeat(_A0, 0)],
          alpha=2.0, embed_scale=8.0, max_positions=700)
# B: latent first, with a window of ONE token (a row sees itself and the sink only) and then without any mask; a latent layer
#    run twice; every head its own kv head; one expert of one; a convolution of one tap (no carried inputs) and one of seven
_B1 = latent(1, 24, 12, 40, 16, mlp=moe(24, 4, 1))
B = model(97, 48, [latent(3, 8, 8, 8, 24, window=1, mlp=moe(40, 1, 1)), _B1,
                   parallel(attention(3, 3, 8, 8, window=1), scan(24, 12, 3, conv=1)), repeat(_B1, 1),
                   parallel(attention(2, 1, 24, 8, base=100.0), scan(80, 3, 1, conv=7), mlp=moe(16, 2, 2))],
          alpha=1.0, embed_scale=1.0, eps=1e-6, max_positions=600)
# C: wider; windows that cross pages and key tiles (70, 200); heads of 64 with values of 128 and 32; 128 and 40 states a
#    channel; sixteen experts of which four
C = model(211, 128, [parallel(attention(4, 1, 64, 128, window=70, scaling=bands(8.0, 128)), scan(256, 128, 8, conv=3), mlp=moe(64, 16, 4)),
                     latent(8, 48, 16, 32, 96, window=200, scaling=yarn(16.0, 64, fast=8.0, slow=2.0), mlp=moe(96, 4, 2)),
                     parallel(attention(8, 4, 32, 32, window=200, rot_dims=16), scan(64, 40, 16, conv=2)),
                     latent(4, 64, 32, 48, 96, window=70, base=500000.0)],
          alpha=0.5, embed_scale=11.0, max_positions=900)
# D: sizes no vectorised kernel takes: a width that is no multiple of 4, heads of 10 and 6 and 7, a latent of 20, 5 and 7 states
D = model(90, 50, [latent(2, 10, 6, 6, 20, window=5, mlp=moe(30, 3, 2)),
                   parallel(attention(3, 1, 10, 6, window=37, rot_dims=6), scan(18, 7, 2, conv=5), mlp=moe(22, 3, 1)),
                   parallel(attention(2, 2, 6, 14, window=5), scan(30, 5, 7, conv=2))],
          alpha=1.7, embed_scale=3.0, max_positions=300)

MODELS = {"a": A, "b": B, "c": C, "d": D}


def draw_weights(config: dict, seed: int, dtype=torch.bfloat16, decisive_routers=None):
    """{name: tensor} for `config` from the product's own list of tensors, rounded to `dtype` (so that the engine and the
    plain implementation start from the same numbers).

    decisive_routers (default: on): with random routers two logits nearly tie at a few positions of every sequence, inputs
    that differ by rounding alone (bfloat16 against exact ones; in 32-bit a sum taken in another order) then choose
    another expert, and a recurrent layer carries the difference to every later position. So the first E channels of the
    width (E the largest number of experts) carry a code that only the embedding writes: per token a permutation of E
    evenly spaced levels; no mixer or expert writes
    into these channels (those rows of their last matrices are zero, and the weights that follow the side-by-side norms
    are zero there), every norm multiplies them by one number (a row's scale keeps their order), and router row e reads
    channel e alone, without a bias. The experts' order then depends on the token only, with gaps of several percent
    between neighbours, and the weights still differ from expert to expert and from token to token. (Random routers with
    their biases are compared in tests/test_gpu_mavinex_parts.py, row by row, with the nearly tied rows left out.)"""
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.parts.spec import spec_param_specs

    c = config_from_dict(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    if decisive_routers is None:
        decisive_routers = True
    code = max([L["mlp"]["router"]["experts"] for L in config["layers"] if L.get("mlp")], default=0)
    code = code if decisive_routers else 0
    for s in spec_param_specs(get_architecture(c.architecture).build_spec(c)):
        n, shape = s.name, tuple(s.shape)
        rnd = torch.randn(shape, generator=g)
        leaf = n.split(".", 1)[1] if n.startswith("l") and "." in n else n
        if n == "embed":
            t = rnd * 0.7
        elif leaf.endswith("A_log"):
            t = torch.rand(shape, generator=g) * 5.0 - 4.0          # decays from exp(-0.02 dt) to exp(-2.7 dt)
        elif leaf.endswith("dt.b") or leaf.endswith("conv.b"):
            t = 0.7 * rnd
        elif leaf.endswith(".D"):
            t = 1.0 + 0.5 * rnd
        elif leaf.endswith(".conv"):
            t = 0.6 * rnd
        elif leaf.endswith(".dt"):
            t = rnd * (1.5 / math.sqrt(shape[1]))
        elif leaf == "mix.sink":
            t = 1.5 * rnd
        elif leaf == "mlp.router":
            t = rnd * (3.0 / math.sqrt(shape[1]))
        elif leaf == "mlp.router.b":
            t = 0.5 * rnd
        elif leaf.startswith("mlp.e") and leaf.endswith(".down"):
            t = rnd * (1.0 / math.sqrt(shape[1]))
        elif len(shape) == 2:
            t = rnd * (1.2 / math.sqrt(shape[1]))
        elif leaf in ("norm1", "norm2") or n == "final.norm":       # stored around zero: the row is multiplied by 1 + w
            t = 0.2 * rnd
        else:                                                       # plain norm weights
            t = 1.0 + 0.2 * rnd
        if code:
            if n == "embed":
                for tok in range(shape[0]):
                    t[tok, :code] = (torch.randperm(code, generator=g) + 0.5) * (2.0 / code)
            elif leaf == "mlp.router":
                t = torch.zeros(shape)
                t[:, :shape[0]] = 2.5 * torch.eye(shape[0])
            elif leaf == "mlp.router.b":
                t = torch.zeros(shape)
            elif leaf in ("norm1", "norm2"):
                t[:code] = 0.0
            elif leaf in ("mix.o", "mix.left.out", "mix.right.out") or (leaf.startswith("mlp.e") and leaf.endswith(".down")):
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


class PlainMavinex:
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
