"""Typed configuration of the Koduzen decoder, read from config.json's own keys.

A Koduzen model is a list of pre-norm layers (plain RMS norms) over ``streams`` residual rows per token
(hyper-connections: every sublayer reads a weighted sum of the rows and writes back into all of them while they mix;
without the key there is one row and a plain residual sum).  A layer has one of three mixers,

* ``retention``: linear attention with one fixed decay per head, q and k rotated (rotate-half) on their first entries;
* ``attention``: grouped-query softmax attention over a sliding window, q and k RMS-normed over the whole projection
  and then rotated, optionally with YaRN-scaled frequencies;
* ``attention_2``: windowed attention without rotation: a query temperature that grows with the position, a bias per
  head that grows with the distance, a learned sink in the softmax; a layer with ``kv_from`` projects no keys and
  values and reads another layer's,

and a feed-forward that is dense (a clipped gated unit), a mixture of such experts (softmax router with a correction
on the choice, a limit to the best groups, experts that hand their input on, a shared expert) or missing.  The
embedding table is also the output head.  Every size and constant that can differ between two models is a key of the file.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .base import ConfigError, read_key, require


@dataclasses.dataclass(frozen=True)
class YarnSpec:
    factor: float
    original: float
    fast: float
    slow: float


@dataclasses.dataclass(frozen=True)
class RotSpec:
    base: float
    dims: int
    scaling: YarnSpec | None = None


@dataclasses.dataclass(frozen=True)
class RetentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: RotSpec | None


@dataclasses.dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int | None
    scale: float
    rot: RotSpec | None


@dataclasses.dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: float


@dataclasses.dataclass(frozen=True)
class BiasedAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int | None
    scale: float
    q_temp: QueryTemperature | None
    kv_from: int | None


@dataclasses.dataclass(frozen=True)
class GluSpec:
    ff: int
    limit: float


@dataclasses.dataclass(frozen=True)
class MoeSpec:
    experts: int  # experts with weights
    identity: int  # router outputs after them whose expert hands its input on
    top: int
    groups: int
    keep: int
    scale: float
    expert: GluSpec
    shared: GluSpec | None


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: "RetentionSpec | AttentionSpec | BiasedAttentionSpec"
    mlp: "GluSpec | MoeSpec | None"


def _rot(m: Mapping[str, Any], dim: int, where: str, scaling_allowed: bool) -> RotSpec | None:
    rot = read_key(m, "rot", dict, None)
    if rot is None:
        return None
    base, dims = read_key(rot, "base", float), read_key(rot, "dims", int)
    require(base > 0, f"{where}.rot.base must be positive")
    require(dims % 2 == 0 and 0 <= dims <= dim, f"{where}: rot.dims = {dims} must be even and at most dim = {dim}")
    sc = read_key(rot, "scaling", dict, None)
    scaling = None
    if sc is not None:
        require(scaling_allowed, f"{where}.rot.scaling: this mixer's rotation has no frequency scaling")
        scaling = YarnSpec(read_key(sc, "factor", float), float(read_key(sc, "original", float)), read_key(sc, "fast", float),
                           read_key(sc, "slow", float))
        require(min(scaling.factor, scaling.original, scaling.fast, scaling.slow) > 0 and base != 1.0,
                f"{where}.rot.scaling: factor, original, fast and slow must be positive (and the base not 1)")
    return RotSpec(base, dims, scaling)


def _window(m: Mapping[str, Any], where: str) -> int | None:
    mask = read_key(m, "mask", dict, None)
    if mask is None:
        return None
    size = read_key(mask, "size", int)
    require(size > 0, f"{where}: mask.size must be positive")
    return size


def _glu(d: Mapping[str, Any], where: str) -> GluSpec:
    g = GluSpec(read_key(d, "ff", int), read_key(d, "limit", float))
    require(g.ff > 0 and g.limit > 0, f"{where}: ff and limit must be positive")
    return g


@dataclasses.dataclass(frozen=True)
class KoduzenConfig:
    vocab: int
    width: int
    layers: tuple[LayerSpec, ...]
    norm_eps: float
    streams: int | None  # None: one residual row and a plain residual sum

    # the names the rest of the framework asks a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def readers_of(self, j: int) -> list[int]:
        """The layers that read layer j's keys and values."""
        return [i for i, L in enumerate(self.layers) if getattr(L.mixer, "kv_from", None) == j]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "KoduzenConfig":
        raw_layers = read_key(d, "layers", list)
        require(len(raw_layers) > 0, "'layers' is empty")
        layers: list[LayerSpec] = []
        for i, L in enumerate(raw_layers):
            require(isinstance(L, dict), f"layers[{i}] must be an object")
            kind = read_key(L, "type", str)
            m = read_key(L, "mixer", dict)
            where = f"layers[{i}].mixer"
            heads, dim, vdim = read_key(m, "heads", int), read_key(m, "dim", int), read_key(m, "vdim", int)
            require(heads > 0 and dim > 0 and vdim > 0, f"{where}: sizes must be positive")
            if kind == "retention":
                decay = tuple(float(x) for x in read_key(m, "decay", list))
                require(len(decay) == heads and all(0 < x <= 1 for x in decay), f"{where}: 'decay' needs {heads} numbers in (0, 1]")
                mixer: Any = RetentionSpec(heads, dim, vdim, decay, _rot(m, dim, where, False))
            elif kind in ("attention", "attention_2"):
                kv_heads = read_key(m, "kv_heads", int)
                require(kv_heads > 0 and heads % kv_heads == 0, f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
                scale = read_key(m, "scale", float)
                if kind == "attention":
                    mixer = AttentionSpec(heads, kv_heads, dim, vdim, _window(m, where), scale, _rot(m, dim, where, True))
                else:
                    qt = read_key(m, "q_temp", dict, None)
                    temp = None
                    if qt is not None:
                        temp = QueryTemperature(read_key(qt, "coef", float), float(read_key(qt, "every", float)))
                        require(temp.every > 0, f"{where}.q_temp.every must be positive")
                    src = read_key(m, "kv_from", int, None)
                    if src is not None:
                        require(0 <= src < i, f"{where}: kv_from = {src} must name an earlier layer")
                        other = layers[src].mixer
                        require(isinstance(other, BiasedAttentionSpec) and other.kv_from is None,
                                f"{where}: kv_from = {src} must name an attention_2 layer with projections of its own")
                        require((other.kv_heads, other.dim, other.vdim) == (kv_heads, dim, vdim),
                                f"{where}: layer {src} keeps {other.kv_heads} heads of {other.dim}/{other.vdim}, not {kv_heads} of {dim}/{vdim}")
                    mixer = BiasedAttentionSpec(heads, kv_heads, dim, vdim, _window(m, where), scale, temp, src)
            else:
                raise ConfigError(f"config.json: layers[{i}].type = {kind!r} is no mixer of this architecture "
                                  "(retention, attention, attention_2)")
            mlp: Any = None
            if L.get("mlp") is not None:
                ml = read_key(L, "mlp", dict)
                mk = read_key(ml, "kind", str)
                at = f"layers[{i}].mlp"
                if mk == "dense":
                    mlp = _glu(ml, at)
                elif mk == "moe":
                    r = read_key(ml, "router", dict)
                    g = read_key(r, "groups", dict, None)
                    groups, keep = (1, 1) if g is None else (read_key(g, "count", int), read_key(g, "keep", int))
                    sh = read_key(ml, "shared", dict, None)
                    mlp = MoeSpec(read_key(r, "experts", int), read_key(r, "identity", int, 0), read_key(r, "top", int), groups, keep,
                                  read_key(r, "scale", float, 1.0), _glu(read_key(ml, "expert", dict), at + ".expert"),
                                  None if sh is None else _glu(sh, at + ".shared"))
                    total = mlp.experts + mlp.identity
                    require(mlp.experts > 0 and mlp.identity >= 0 and 1 <= mlp.top <= total,
                            f"{at}.router: top-{mlp.top} of {mlp.experts} experts + {mlp.identity} identity experts")
                    require(groups >= 1 and total % groups == 0 and 1 <= keep <= groups,
                            f"{at}.router.groups: {groups} groups (keep {keep}) of {total} router outputs")
                else:
                    raise ConfigError(f"config.json: {at}.kind = {mk!r}; this architecture has 'dense' and 'moe'")
            layers.append(LayerSpec(kind, mixer, mlp))
        streams = read_key(d, "streams", int, None)
        cfg = KoduzenConfig(vocab=read_key(d, "vocab", int), width=read_key(d, "width", int), layers=tuple(layers),
                            norm_eps=read_key(read_key(d, "norm", dict), "eps", float), streams=streams)
        require(cfg.vocab > 0 and cfg.width > 0, "vocab and width must be positive")
        require(cfg.norm_eps > 0, "norm.eps must be positive")
        require(streams is None or streams >= 1, "streams must be at least 1")
        return cfg
