"""`RunopelConfig`: the config.json of the Runopel decoder, typed and checked.

A Runopel model is a list of pre-norm layers, each a sequence mixer followed, where the layer has one, by a feed-forward;
the residual is one stream or several (hyper-connections):

    architecture    "Runopel"
    vocab, width
    norm.eps                        of every norm of the model
    residual_mult                   multiplies every sublayer's result before it joins the residual (absent: 1)
    streams                         number of residual streams (absent: one plain residual, no stream weights)
    logit_scale                     multiplies the logits (absent: 1); the head is the embedding table
    max_positions                   optional: the longest sequence (absent: DEFAULT_MAX_POSITIONS)
    layers[i].type                  "mamba2" or "latent_attention"
    layers[i].mixer                 mamba2: heads, vdim, state, groups, norm_groups, conv (taps)
                                    latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims},
                                    mask {size} (a sliding window of that many positions; absent: every earlier token)
    layers[i].mlp                   null, {kind: "dense", ff, limit} or {kind: "moe", expert {ff}, router {experts, top}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take
from .vegodra import DEFAULT_MAX_POSITIONS, RotaryConfig, _rot, _sub


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    def to_dict(self):
        return dict(heads=self.heads, vdim=self.vdim, state=self.state, groups=self.groups, norm_groups=self.norm_groups,
                    conv=self.conv)


@dataclass(frozen=True)
class WindowLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    window: Optional[int] = None      # mask.size; None: no mask beyond the causal one

    def to_dict(self):
        d = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, kv_rank=self.kv_rank, scale=self.scale,
                 rot=self.rot.to_dict())
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        return d


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int
    limit: float

    def to_dict(self):
        return dict(kind="dense", ff=self.ff, limit=self.limit)


@dataclass(frozen=True)
class RoutedFFConfig:
    ff: int
    experts: int
    top: int

    def to_dict(self):
        return dict(kind="moe", expert=dict(ff=self.ff), router=dict(experts=self.experts, top=self.top))


@dataclass(frozen=True)
class RunopelLayerConfig:
    type: str                         # "mamba2" | "latent_attention"
    mixer: Any
    mlp: Any = None                   # DenseFFConfig, RoutedFFConfig or None

    def to_dict(self):
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=None if self.mlp is None else self.mlp.to_dict())


@dataclass(frozen=True)
class RunopelConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RunopelLayerConfig, ...]
    residual_mult: float = 1.0
    streams: Optional[int] = None
    logit_scale: float = 1.0
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RunopelConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = take(L, "type", str)
            m = _sub(L, "mixer", where)
            pos = lambda key: take(m, key, int, positive=True)
            if kind == "mamba2":
                mixer = Mamba2Config(pos("heads"), pos("vdim"), pos("state"), pos("groups"), pos("norm_groups"), pos("conv"))
                if mixer.heads % mixer.groups:
                    raise ConfigError(f"config.json: {where}mixer: {mixer.heads} heads are not a multiple of {mixer.groups} groups")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json: {where}mixer: {mixer.heads} x {mixer.vdim} channels do not fall into "
                                      f"{mixer.norm_groups} equal norm_groups")
            elif kind == "latent_attention":
                rot_dim = pos("rot_dim")
                mask = m.get("mask")
                if mask is not None and not isinstance(mask, dict):
                    raise ConfigError(f"config.json: {where}mixer.mask must be an object or null")
                window = take(mask, "size", int, None, positive=True) if mask else None
                mixer = WindowLatentConfig(pos("heads"), pos("dim"), rot_dim, pos("vdim"), pos("kv_rank"),
                                           take(m, "scale", float, positive=True), _rot(m, where, rot_dim, "rot_dim"), window)
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (known: 'mamba2', 'latent_attention')")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}mlp must be an object or null")
                k = take(mlp, "kind", str)
                if k == "dense":
                    ff = DenseFFConfig(take(mlp, "ff", int, positive=True), take(mlp, "limit", float, positive=True))
                elif k == "moe":
                    r = _sub(mlp, "router", where + "mlp.")
                    ff = RoutedFFConfig(take(_sub(mlp, "expert", where + "mlp."), "ff", int, positive=True),
                                        take(r, "experts", int, positive=True), take(r, "top", int, positive=True))
                    if ff.top > ff.experts:
                        raise ConfigError(f"config.json: {where}mlp.router: top = {ff.top} of {ff.experts} experts")
                else:
                    raise ConfigError(f"config.json: {where}mlp.kind {k!r} is not known (known: 'dense', 'moe')")
            layers.append(RunopelLayerConfig(kind, mixer, ff))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos)
        return cls(architecture=d["architectures"][0] if "architectures" in d else d["architecture"],
                   vocab=take(d, "vocab", int, positive=True), width=take(d, "width", int, positive=True),
                   norm_eps=take(_sub(d, "norm", ""), "eps", float, positive=True), layers=tuple(layers),
                   residual_mult=take(d, "residual_mult", float, 1.0), streams=take(d, "streams", int, None, positive=True),
                   logit_scale=take(d, "logit_scale", float, 1.0),
                   max_positions=take(d, "max_positions", int, DEFAULT_MAX_POSITIONS, positive=True), eos_token_ids=eos_ids)

    def to_dict(self) -> Dict[str, Any]:
        d = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 residual_mult=self.residual_mult, logit_scale=self.logit_scale, layers=[L.to_dict() for L in self.layers])
        if self.streams is not None:
            d["streams"] = self.streams
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
