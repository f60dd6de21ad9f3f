"""Vofusun: its tensors by name and how its layers are put together from parts.

Tensor names: ``embed`` (also the output head, unscaled), ``final.norm`` and per layer ``l<i>.``: ``norm1``, ``norm2``
(if the layer has a feed-forward), ``mix.*`` and ``mlp.{gate,up,down}``.  Linear weights are [out, in].

* ``attention`` mixer: ``mix.{q,k,v,o}``.
* ``delta`` mixer: ``mix.{q,k,v}`` with ``mix.{q,k,v}.conv`` ([channels, taps]), ``mix.b`` (step size), ``mix.a``,
  ``mix.A_log``, ``mix.dt_bias`` (decay), ``mix.g`` (output gate), ``mix.norm``, ``mix.o``.
* ``attention_2`` mixer: ``mix.{q,k,g,o}`` (the keys as projected are the values).

Layer rules (config: :class:`..config.vofusun.VofusunConfig`): x += mixer(norm1(x)); x += ff(norm2(x)), plain RMS norms,
ff = W_down (silu(W_gate h) * W_up h).  A stretch of layers may run several times with the same weights; every pass has
caches and states of its own, and every pass but the first opens with x += (the embedding's output).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.registry import Architecture, register_architecture
from ..config.vofusun import ChunkAttentionSpec, DeltaSpec, VofusunConfig, WindowAttentionSpec
from ..parts import DecoderModel, GatedPagedAttention, Runtime, make_part, rotary_frequencies, wavelength_scaled_frequencies
from ..weights.loader import TensorSpec


def tensor_specs(cfg: VofusunConfig) -> dict[str, TensorSpec]:
    D, V = cfg.width, cfg.vocab
    specs: list[TensorSpec] = [TensorSpec("embed", (V, D))]
    for i, L in enumerate(cfg.layers):
        p, m, q = f"l{i}.", L.mixer, f"l{i}.mix."
        specs.append(TensorSpec(p + "norm1", (D,), "norm"))
        if isinstance(m, WindowAttentionSpec):
            specs += [TensorSpec(q + "q", (m.heads * m.dim, D)), TensorSpec(q + "k", (m.kv_heads * m.dim, D)),
                      TensorSpec(q + "v", (m.kv_heads * m.vdim, D)), TensorSpec(q + "o", (D, m.heads * m.vdim))]
        elif isinstance(m, DeltaSpec):
            hk, hv = m.kv_heads * m.dim, m.heads * m.vdim
            specs += [TensorSpec(q + "q", (hk, D)), TensorSpec(q + "q.conv", (hk, m.conv), "bias"),
                      TensorSpec(q + "k", (hk, D)), TensorSpec(q + "k.conv", (hk, m.conv), "bias"),
                      TensorSpec(q + "v", (hv, D)), TensorSpec(q + "v.conv", (hv, m.conv), "bias"),
                      TensorSpec(q + "b", (m.heads, D)), TensorSpec(q + "A_log", (m.heads,), "bias"),
                      TensorSpec(q + "norm", (m.vdim,), "norm"), TensorSpec(q + "a", (m.heads, D)),
                      TensorSpec(q + "dt_bias", (m.heads,), "bias"), TensorSpec(q + "g", (hv, D)), TensorSpec(q + "o", (D, hv))]
        else:
            assert isinstance(m, ChunkAttentionSpec)
            specs += [TensorSpec(q + "q", (m.heads * m.dim, D)), TensorSpec(q + "k", (m.kv_heads * m.dim, D)),
                      TensorSpec(q + "g", (m.heads * m.dim, D)), TensorSpec(q + "o", (D, m.heads * m.dim))]
        if L.mlp is not None:
            specs += [TensorSpec(p + "norm2", (D,), "norm"), TensorSpec(p + "mlp.gate", (L.mlp.ff, D)),
                      TensorSpec(p + "mlp.up", (L.mlp.ff, D)), TensorSpec(p + "mlp.down", (D, L.mlp.ff))]
    specs.append(TensorSpec("final.norm", (D,), "norm"))
    return {s.name: s for s in specs}


def build(cfg: VofusunConfig, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> DecoderModel:
    """Puts the decoder together.  ``tensors`` (by spec name) is consumed as the weights are stacked into the layouts
    the kernels read."""
    t = dict(tensors) if not isinstance(tensors, dict) else tensors
    dev, eps = runtime.device, cfg.norm_eps

    def take(name: str) -> torch.Tensor:
        return t.pop(name).to(dev)

    def norm(name: str):
        return make_part("norm", "rms", weight=take(name), eps=eps)

    blocks = []
    for i, L in enumerate(cfg.layers):
        p, m, q = f"l{i}.", L.mixer, f"l{i}.mix."
        if isinstance(m, WindowAttentionSpec):
            mixer = make_part(
                "mixer", "gated_paged_attention",
                w_in=torch.cat([take(q + "q"), take(q + "k"), take(q + "v")], dim=0).contiguous(), w_o=take(q + "o").contiguous(),
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
                window=m.window, gate="none", sink=torch.zeros(m.heads, device=dev),
                padded_dim=GatedPagedAttention.padded_size(m.dim, m.vdim, runtime.dtype))
        elif isinstance(m, DeltaSpec):
            mixer = make_part(
                "mixer", "gated_delta_rule",
                w_in=torch.cat([take(q + s) for s in ("q", "k", "v", "g", "b", "a")], dim=0).contiguous(),
                conv_weight=torch.cat([take(q + s + ".conv") for s in ("q", "k", "v")], dim=0),
                rate_log=take(q + "A_log"), a_bias=take(q + "dt_bias"), norm_weight=take(q + "norm"),
                w_o=take(q + "o").contiguous(), heads=m.heads, key_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, eps=eps,
                activation="silu", unit_eps=1e-6, q_scale=float(m.dim) ** -0.5)
        else:
            inv_freq = None
            if m.rot_dims:
                sc = m.rot_scaling
                inv_freq = (rotary_frequencies(m.rot_base, m.rot_dims) if sc is None else
                            wavelength_scaled_frequencies(m.rot_base, m.rot_dims, sc.factor, sc.low, sc.high, sc.original)).to(dev)
            mixer = make_part(
                "mixer", "gated_paged_attention",
                w_in=torch.cat([take(q + "q"), take(q + "k"), take(q + "g")], dim=0).contiguous(), w_o=take(q + "o").contiguous(),
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.dim, scale=m.scale, eps=eps,
                inv_freq=inv_freq, rot_dims=m.rot_dims, pairing="pairs", norm="after", chunk=m.chunk, values_are_keys=True,
                gate="channel", sink=torch.zeros(m.heads, device=dev),
                padded_dim=GatedPagedAttention.padded_size(m.dim, m.dim, runtime.dtype))
        if L.mlp is None:
            blocks.append(make_part("block", "pre_norm", norm1=norm(p + "norm1"), mixer=mixer, norm2=None, feed_forward=None))
            continue
        ff = make_part("feed_forward", "dense_swiglu",
                       w_gate_up=torch.cat([take(p + "mlp.gate"), take(p + "mlp.up")], dim=0).contiguous(),
                       w_down=take(p + "mlp.down").contiguous())
        blocks.append(make_part("block", "pre_norm", norm1=norm(p + "norm1"), mixer=mixer, norm2=norm(p + "norm2"), feed_forward=ff))
    # the order of execution: every pass of the loop but the first opens with the embedding's output added once more
    reentry = len(blocks)
    if any(opens for _, opens in cfg.layer_order()):
        blocks.append(make_part("block", "embedding_reentry"))
    order: list[tuple[int]] = []
    for i, opens in cfg.layer_order():
        if opens:
            order.append((reentry,))
        order.append((i,))
    embedding = take("embed").contiguous()
    final_norm = norm("final.norm")
    return DecoderModel(runtime, embedding, blocks, final_norm, embedding, schedule=DecoderModel.schedule_of(order, blocks),
                        config=cfg, embedding_scale=cfg.embedding_scale)


VOFUSUN = Architecture(name="Vofusun", parse_config=VofusunConfig.from_dict, tensor_specs=tensor_specs, build=build)
register_architecture(VOFUSUN)
