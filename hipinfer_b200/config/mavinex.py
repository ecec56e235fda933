"""`MavinexConfig`: the config.json of the Mavinex decoder, typed and checked.

A Mavinex model is a list of layers with the norm AFTER the sum, x <- norm(alpha * x + sublayer(x)), each a sequence mixer
followed, where the layer has one, by a mixture of experts:

    architecture    "Mavinex"
    vocab, width
    norm.eps                        of every norm of the model
    postln_alpha                    multiplies the residual before a sublayer's result is added (absent: 1)
    embedding.scale                 multiplies the token embedding (absent: 1)
    max_positions                   optional: the longest sequence (absent: DEFAULT_MAX_POSITIONS)
    layers[i].type                  "parallel" (attention and a selective state-space mixer side by side) or
                                    "latent_attention"
    layers[i].weights_of            optional: the index of the layer whose tensors this layer runs with (its own cache and
                                    state); such a layer has no tensors of its own
    layers[i].mixer                 parallel: left {heads, kv_heads, dim, vdim, scale, rot, mask {size}},
                                              right {inner, state, dt_rank, conv}
                                    latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot, mask {size}
                                    rot = {base, dims, scaling}; scaling (optional) is {factor, low, high, original} for
                                    the left attention (frequencies rescaled by wavelength bands) and {factor, original,
                                    fast, slow} for latent attention (YaRN); mask absent: every earlier token is seen
    layers[i].mlp                   null, or {kind: "moe", expert {ff}, router {experts, top}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take
from .runopel import RoutedFFConfig
from .vegodra import DEFAULT_MAX_POSITIONS, _sub


@dataclass(frozen=True)
class ScaledRotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]] = None     # the scaling's keys and numbers, sorted by key

    def scaling_dict(self) -> Optional[Dict[str, float]]:
        return dict(self.scaling) if self.scaling else None

    def to_dict(self):
        d = dict(base=self.base, dims=self.dims)
        if self.scaling:
            d["scaling"] = dict(self.scaling)
        return d


def _scaled_rot(m, where, limit, limit_name, keys) -> ScaledRotaryConfig:
    r = _sub(m, "rot", where)
    base, dims = take(r, "base", float, positive=True), take(r, "dims", int)
    if dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}mixer.rot.dims = {dims} must be even and at most {limit_name} = {limit}")
    sc = r.get("scaling")
    scaling = None
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}mixer.rot.scaling must be an object or null")
        scaling = tuple(sorted((k, take(sc, k, float, positive=True)) for k in keys))
    return ScaledRotaryConfig(base, dims, scaling)


def _window(m, where) -> Optional[int]:
    mask = m.get("mask")
    if mask is not None and not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}mixer.mask must be an object or null")
    return take(mask, "size", int, None, positive=True) if mask else None


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: ScaledRotaryConfig
    window: Optional[int] = None

    def to_dict(self):
        d = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale, rot=self.rot.to_dict())
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        return d


@dataclass(frozen=True)
class SelectiveScanConfig:
    inner: int
    state: int
    dt_rank: int
    conv: int

    def to_dict(self):
        return dict(inner=self.inner, state=self.state, dt_rank=self.dt_rank, conv=self.conv)


@dataclass(frozen=True)
class SideBySideConfig:
    left: WindowAttentionConfig
    right: SelectiveScanConfig

    def to_dict(self):
        return dict(left=self.left.to_dict(), right=self.right.to_dict())


@dataclass(frozen=True)
class SinkLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: ScaledRotaryConfig
    window: Optional[int] = None

    def to_dict(self):
        d = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, kv_rank=self.kv_rank, scale=self.scale,
                 rot=self.rot.to_dict())
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        return d


@dataclass(frozen=True)
class MavinexLayerConfig:
    type: str                         # "parallel" | "latent_attention"
    mixer: Any
    mlp: Optional[RoutedFFConfig] = None
    weights_of: Optional[int] = None

    def to_dict(self):
        d = dict(type=self.type, mixer=self.mixer.to_dict(), mlp=None if self.mlp is None else self.mlp.to_dict())
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


@dataclass(frozen=True)
class MavinexConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[MavinexLayerConfig, ...]
    postln_alpha: float = 1.0
    embedding_scale: float = 1.0
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs with (i itself for a layer with tensors of its own)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of goes round in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MavinexConfig":
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
            if kind == "parallel":
                a, b = _sub(m, "left", where + "mixer."), _sub(m, "right", where + "mixer.")
                pa, pb = (lambda key: take(a, key, int, positive=True)), (lambda key: take(b, key, int, positive=True))
                dim = pa("dim")
                left = WindowAttentionConfig(pa("heads"), pa("kv_heads"), dim, pa("vdim"), take(a, "scale", float, positive=True),
                                             _scaled_rot(a, where + "mixer.left.", dim, "dim", ("factor", "low", "high", "original")),
                                             _window(a, where + "mixer.left."))
                if left.heads % left.kv_heads:
                    raise ConfigError(f"config.json: {where}mixer.left: {left.heads} heads are not a multiple of {left.kv_heads} kv_heads")
                mixer = SideBySideConfig(left, SelectiveScanConfig(pb("inner"), pb("state"), pb("dt_rank"), pb("conv")))
            elif kind == "latent_attention":
                pos = lambda key: take(m, key, int, positive=True)
                rot_dim = pos("rot_dim")
                mixer = SinkLatentConfig(pos("heads"), pos("dim"), rot_dim, pos("vdim"), pos("kv_rank"),
                                         take(m, "scale", float, positive=True),
                                         _scaled_rot(m, where, rot_dim, "rot_dim", ("factor", "original", "fast", "slow")),
                                         _window(m, where))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (known: 'parallel', 'latent_attention')")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}mlp must be an object or null")
                k = take(mlp, "kind", str, "moe")
                if k != "moe":
                    raise ConfigError(f"config.json: {where}mlp.kind {k!r} is not known (known: 'moe')")
                r = _sub(mlp, "router", where + "mlp.")
                ff = RoutedFFConfig(take(_sub(mlp, "expert", where + "mlp."), "ff", int, positive=True),
                                    take(r, "experts", int, positive=True), take(r, "top", int, positive=True))
                if ff.top > ff.experts:
                    raise ConfigError(f"config.json: {where}mlp.router: top = {ff.top} of {ff.experts} experts")
            wo = take(L, "weights_of", int, None)
            if wo is not None and not 0 <= wo < len(raw):
                raise ConfigError(f"config.json: {where}weights_of = {wo} names no layer (there are {len(raw)})")
            layers.append(MavinexLayerConfig(kind, mixer, ff, wo))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos)
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: key 'embedding' must be an object")
        cfg = cls(architecture=d["architectures"][0] if "architectures" in d else d["architecture"],
                  vocab=take(d, "vocab", int, positive=True), width=take(d, "width", int, positive=True),
                  norm_eps=take(_sub(d, "norm", ""), "eps", float, positive=True), layers=tuple(layers),
                  postln_alpha=take(d, "postln_alpha", float, 1.0), embedding_scale=take(emb, "scale", float, 1.0),
                  max_positions=take(d, "max_positions", int, DEFAULT_MAX_POSITIONS, positive=True), eos_token_ids=eos_ids)
        for i, L in enumerate(cfg.layers):
            j = cfg.weights_layer(i)
            if cfg.layers[j].type != L.type or (cfg.layers[j].mlp is None) != (L.mlp is None):
                raise ConfigError(f"config.json: layers[{i}] runs with the tensors of layers[{j}], a layer of another kind")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 postln_alpha=self.postln_alpha, embedding=dict(scale=self.embedding_scale),
                 layers=[L.to_dict() for L in self.layers])
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
