"""Typed configuration of the Vofusun decoder, read from config.json's own keys.

A Vofusun model is a list of pre-norm layers (plain RMS norms), each with one of three mixers and a dense SwiGLU
feed-forward or none:

* ``attention``: grouped-query softmax attention over a sliding window, without positions in its scores, with a sink
  (one more term of score zero in the softmax's denominator);
* ``delta``: the gated delta rule behind short convolutions on q, k and v;
* ``attention_2``: attention whose values are its keys as projected, with a rotation of neighbouring pairs on part of
  the head (frequencies rescaled by wavelength), an RMS norm of q and k after the rotation, queries that see their own
  chunk of positions, the sink, and a sigmoid gate on every output channel.

A stretch of layers may run several times with the same weights (``loop``); before every pass but the first the
embedding's output is added to the stream.  The embedding is scaled and is also the output head (unscaled).  Every size
and constant that can differ between two models is a key of the file.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .base import ConfigError, read_key, require


@dataclasses.dataclass(frozen=True)
class WindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int
    scale: float


@dataclasses.dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclasses.dataclass(frozen=True)
class RotScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclasses.dataclass(frozen=True)
class ChunkAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int  # the keys are the values: equal to dim
    chunk: int
    scale: float
    rot_base: float
    rot_dims: int  # 0: no rotation
    rot_scaling: RotScaling | None


@dataclasses.dataclass(frozen=True)
class MlpSpec:
    kind: str  # "dense"
    ff: int


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: "WindowAttentionSpec | DeltaSpec | ChunkAttentionSpec"
    mlp: MlpSpec | None


@dataclasses.dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class VofusunConfig:
    vocab: int
    width: int
    layers: tuple[LayerSpec, ...]
    loop: LoopSpec | None
    norm_eps: float
    embedding_scale: float

    # the names the rest of the framework asks a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def layer_order(self) -> list[tuple[int, bool]]:
        """(layer index, whether this run opens a pass of the loop after the first) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        lo, hi = self.loop.start, self.loop.stop
        order = [(i, False) for i in range(lo)]
        for t in range(self.loop.times):
            order += [(i, t > 0 and i == lo) for i in range(lo, hi)]
        return order + [(i, False) for i in range(hi, n)]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "VofusunConfig":
        raw_layers = read_key(d, "layers", list)
        require(len(raw_layers) > 0, "'layers' is empty")
        layers = []
        for i, L in enumerate(raw_layers):
            require(isinstance(L, dict), f"layers[{i}] must be an object")
            kind = read_key(L, "type", str)
            m = read_key(L, "mixer", dict)
            where = f"layers[{i}].mixer"
            heads, kv_heads, dim = read_key(m, "heads", int), read_key(m, "kv_heads", int), read_key(m, "dim", int)
            require(heads > 0 and kv_heads > 0 and dim > 0, f"{where}: sizes must be positive")
            require(heads % kv_heads == 0, f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
            if kind == "attention":
                mixer: Any = WindowAttentionSpec(heads, kv_heads, dim, read_key(m, "vdim", int),
                                                 read_key(read_key(m, "mask", dict), "size", int), read_key(m, "scale", float))
                require(mixer.vdim > 0 and mixer.window > 0, f"{where}: vdim and mask.size must be positive")
            elif kind == "delta":
                mixer = DeltaSpec(heads, kv_heads, dim, read_key(m, "vdim", int), read_key(m, "conv", int))
                require(mixer.vdim > 0 and mixer.conv > 0, f"{where}: vdim and conv must be positive")
            elif kind == "attention_2":
                rot = read_key(m, "rot", dict, None)
                base, dims, scaling = 1.0, 0, None
                if rot is not None:
                    base, dims = read_key(rot, "base", float), read_key(rot, "dims", int)
                    sc = read_key(rot, "scaling", dict, None)
                    if sc is not None:
                        scaling = RotScaling(read_key(sc, "factor", float), read_key(sc, "low", float), read_key(sc, "high", float),
                                             float(read_key(sc, "original", float)))
                        require(scaling.factor > 0 and scaling.original > 0 and scaling.low > 0 and scaling.high > 0,
                                f"{where}.rot.scaling: factor, low, high and original must be positive")
                    require(base > 0, f"{where}.rot.base must be positive")
                vdim = read_key(m, "vdim", int, dim)
                require(vdim == dim, f"{where}: the values are the keys, so vdim = {vdim} must equal dim = {dim}")
                mixer = ChunkAttentionSpec(heads, kv_heads, dim, vdim, read_key(read_key(m, "mask", dict), "size", int),
                                           read_key(m, "scale", float), base, dims, scaling)
                require(mixer.chunk > 0, f"{where}: mask.size must be positive")
                require(dims % 2 == 0 and 0 <= dims <= dim, f"{where}: rot.dims = {dims} must be even and at most dim = {dim}")
            else:
                raise ConfigError(f"config.json: layers[{i}].type = {kind!r} is no mixer of this architecture "
                                  "(attention, delta, attention_2)")
            mlp = None
            if L.get("mlp") is not None:
                ml = read_key(L, "mlp", dict)
                mk = read_key(ml, "kind", str)
                if mk != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind = {mk!r}; this architecture has 'dense'")
                mlp = MlpSpec("dense", read_key(ml, "ff", int))
                require(mlp.ff > 0, f"layers[{i}].mlp: ff must be positive")
            layers.append(LayerSpec(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = read_key(d, "loop", dict)
            loop = LoopSpec(read_key(lp, "start", int), read_key(lp, "stop", int), read_key(lp, "times", int))
            require(0 <= loop.start < loop.stop <= len(layers), f"loop: layers {loop.start}..{loop.stop - 1} of {len(layers)}")
            require(loop.times >= 1, "loop.times must be at least 1")
        cfg = VofusunConfig(
            vocab=read_key(d, "vocab", int), width=read_key(d, "width", int), layers=tuple(layers), loop=loop,
            norm_eps=read_key(read_key(d, "norm", dict), "eps", float),
            embedding_scale=read_key(read_key(d, "embedding", dict), "scale", float))
        require(cfg.vocab > 0 and cfg.width > 0, "vocab and width must be positive")
        require(cfg.norm_eps > 0, "norm.eps must be positive")
        return cfg
