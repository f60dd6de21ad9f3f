"""Koduzen: its tensors by name and how its layers are put together from parts.

Tensor names: ``embed`` (also the output head), ``final.norm`` and per layer ``l<i>.``: ``norm1``, ``norm2`` (if the
layer has a feed-forward), ``mix.*``, ``mlp.*`` and, in a model with residual streams, ``hc1.{in,out,mix}`` and
``hc2.{in,out,mix}`` (read weights [S], write weights [S], mix matrix [S, S] indexed [from, to]).  Linear weights are [out, in].

* ``retention`` mixer: ``mix.{q,k,v,g,o}``.
* ``attention`` mixer: ``mix.{q,k,v,o}``, ``mix.q.norm`` [heads * dim], ``mix.k.norm`` [kv_heads * dim].
* ``attention_2`` mixer: ``mix.{q,k,v,o}``, ``mix.sink`` [heads]; with ``kv_from`` no ``mix.k`` and ``mix.v``.
* dense feed-forward: ``mlp.{gate,up,down}``; mixture: ``mlp.router`` [experts + identity, width], ``mlp.correction``,
  ``mlp.e<j>.{gate,up,down}``, ``mlp.shared.{gate,up,down}``.

Layer rules (config: :class:`..config.koduzen.KoduzenConfig`): with S residual rows x_1 .. x_S per token (all equal to
the embedding's output at the start), sublayer q of a layer reads u = sum_s in_q[s] x_s, makes y = sublayer(norm_q(u))
and leaves x_t <- sum_s mix_q[s, t] x_s + out_q[t] y; the final norm sees the sum of the rows.  Without streams:
x += mixer(norm1(x)); x += ff(norm2(x)).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.koduzen import AttentionSpec, BiasedAttentionSpec, GluSpec, KoduzenConfig, MoeSpec, RetentionSpec
from ..config.registry import Architecture, register_architecture
from ..kernels import api as K
from ..parts import DecoderModel, GatedPagedAttention, LayerRun, Runtime, make_part, rotary_frequencies, yarn_frequencies
from ..weights.loader import TensorSpec

GLU_ALPHA, GLU_SHIFT = 1.702, 1.0  # the gated unit of this design: g sigmoid(1.702 g) (u + 1)
SLOPE_RANGE = 8.0  # head h of H takes the distance bias 2^(-SLOPE_RANGE (h + 1) / H) per position


def distance_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-SLOPE_RANGE * (h + 1) / heads) for h in range(heads)], dtype=torch.float64).to(torch.float32)


def tensor_specs(cfg: KoduzenConfig) -> dict[str, TensorSpec]:
    D, V, S = cfg.width, cfg.vocab, cfg.streams
    specs: list[TensorSpec] = [TensorSpec("embed", (V, D))]

    def glu(prefix: str, g: GluSpec):
        return [TensorSpec(prefix + "gate", (g.ff, D)), TensorSpec(prefix + "up", (g.ff, D)), TensorSpec(prefix + "down", (D, g.ff))]

    for i, L in enumerate(cfg.layers):
        p, m, q = f"l{i}.", L.mixer, f"l{i}.mix."
        specs.append(TensorSpec(p + "norm1", (D,), "norm"))
        if isinstance(m, RetentionSpec):
            specs += [TensorSpec(q + "q", (m.heads * m.dim, D)), TensorSpec(q + "k", (m.heads * m.dim, D)),
                      TensorSpec(q + "v", (m.heads * m.vdim, D)), TensorSpec(q + "g", (m.heads * m.vdim, D)),
                      TensorSpec(q + "o", (D, m.heads * m.vdim))]
        elif isinstance(m, AttentionSpec):
            specs += [TensorSpec(q + "q", (m.heads * m.dim, D)), TensorSpec(q + "k", (m.kv_heads * m.dim, D)),
                      TensorSpec(q + "v", (m.kv_heads * m.vdim, D)), TensorSpec(q + "q.norm", (m.heads * m.dim,), "norm"),
                      TensorSpec(q + "k.norm", (m.kv_heads * m.dim,), "norm"), TensorSpec(q + "o", (D, m.heads * m.vdim))]
        else:
            assert isinstance(m, BiasedAttentionSpec)
            specs.append(TensorSpec(q + "q", (m.heads * m.dim, D)))
            if m.kv_from is None:
                specs += [TensorSpec(q + "k", (m.kv_heads * m.dim, D)), TensorSpec(q + "v", (m.kv_heads * m.vdim, D))]
            specs += [TensorSpec(q + "sink", (m.heads,), "bias"), TensorSpec(q + "o", (D, m.heads * m.vdim))]
        if L.mlp is not None:
            specs.append(TensorSpec(p + "norm2", (D,), "norm"))
            if isinstance(L.mlp, GluSpec):
                specs += glu(p + "mlp.", L.mlp)
            else:
                total = L.mlp.experts + L.mlp.identity
                for e in range(L.mlp.experts):
                    specs += glu(f"{p}mlp.e{e}.", L.mlp.expert)
                specs += [TensorSpec(p + "mlp.router", (total, D)), TensorSpec(p + "mlp.correction", (total,), "bias")]
                if L.mlp.shared is not None:
                    specs += glu(p + "mlp.shared.", L.mlp.shared)
        if S is not None:
            for hc in ("hc1.",) + (("hc2.",) if L.mlp is not None else ()):
                specs += [TensorSpec(p + hc + "in", (S,), "norm"), TensorSpec(p + hc + "out", (S,), "norm"),
                          TensorSpec(p + hc + "mix", (S, S), "identity")]
    specs.append(TensorSpec("final.norm", (D,), "norm"))
    return {s.name: s for s in specs}


def build(cfg: KoduzenConfig, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> DecoderModel:
    """Puts the decoder together.  ``tensors`` (by spec name) is consumed as the weights are stacked into the layouts
    the kernels read."""
    t = dict(tensors) if not isinstance(tensors, dict) else tensors
    dev, eps, S = runtime.device, cfg.norm_eps, cfg.streams

    def take(name: str) -> torch.Tensor:
        return t.pop(name).to(dev)

    def norm(name: str, read: torch.Tensor | None = None):
        if S is None:
            return make_part("norm", "rms", weight=take(name), eps=eps)
        return make_part("norm", "stream_rms", weight=take(name), eps=eps, streams=S, read=read)

    def glu_unit(prefix: str, g: GluSpec):
        return make_part("feed_forward", "dense_swiglu",
                         w_gate_up=torch.cat([take(prefix + "gate"), take(prefix + "up")], dim=0).contiguous(),
                         w_down=take(prefix + "down").contiguous(), glu=K.glu_form(GLU_ALPHA, g.limit, GLU_SHIFT))

    def rotation(rot):
        """(frequencies, rotated entries, amplitude) of a mixer's rotation."""
        if rot is None or rot.dims == 0:
            return None, 0, 1.0
        if rot.scaling is None:
            return rotary_frequencies(rot.base, rot.dims).to(dev), rot.dims, 1.0
        sc = rot.scaling
        f, amplitude = yarn_frequencies(rot.base, rot.dims, sc.factor, sc.original, sc.fast, sc.slow)
        return f.to(dev), rot.dims, amplitude

    blocks = []
    for i, L in enumerate(cfg.layers):
        p, m, q = f"l{i}.", L.mixer, f"l{i}.mix."
        if isinstance(m, RetentionSpec):
            inv_freq, rot_dims, _ = rotation(m.rot)
            mixer = make_part(
                "mixer", "retention", w_in=torch.cat([take(q + s) for s in ("q", "k", "v", "g")], dim=0).contiguous(),
                w_o=take(q + "o").contiguous(), decay=torch.tensor(m.decay, dtype=torch.float32, device=dev), heads=m.heads, dim=m.dim,
                vdim=m.vdim, eps=eps, k_scale=float(m.dim) ** -0.5, inv_freq=inv_freq, rot_dims=rot_dims)
        elif isinstance(m, AttentionSpec):
            inv_freq, rot_dims, amplitude = rotation(m.rot)
            mixer = make_part(
                "mixer", "gated_paged_attention",
                w_in=torch.cat([take(q + "q"), take(q + "k"), take(q + "v")], dim=0).contiguous(), w_o=take(q + "o").contiguous(),
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
                q_norm_weight=take(q + "q.norm"), k_norm_weight=take(q + "k.norm"), norm="whole", inv_freq=inv_freq,
                rot_dims=rot_dims, rot_amplitude=amplitude, window=m.window, gate="none",
                padded_dim=GatedPagedAttention.padded_size(m.dim, m.vdim, runtime.dtype))
        else:
            own = m.kv_from is None
            w_in = torch.cat([take(q + "q"), take(q + "k"), take(q + "v")], dim=0) if own else take(q + "q")
            # the pages of a layer that others read live as long as the longest window among them (0: for good)
            windows = [cfg.layers[j].mixer.window for j in cfg.readers_of(i)] if own else []
            keep = None if not windows else (0 if None in windows else max(windows))
            mixer = make_part(
                "mixer", "gated_paged_attention", w_in=w_in.contiguous(), w_o=take(q + "o").contiguous(),
                n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
                window=m.window, gate="none", sink=take(q + "sink"), slopes=distance_slopes(m.heads).to(dev),
                query_temperature=None if m.q_temp is None else (m.q_temp.coef, m.q_temp.every), projects_kv=own, keep_window=keep,
                padded_dim=GatedPagedAttention.padded_size(m.dim, m.vdim, runtime.dtype))
        ff = None
        if isinstance(L.mlp, GluSpec):
            ff = glu_unit(p + "mlp.", L.mlp)
        elif isinstance(L.mlp, MoeSpec):
            r = L.mlp
            gate_up = torch.stack([torch.cat([take(f"{p}mlp.e{e}.gate"), take(f"{p}mlp.e{e}.up")], dim=0) for e in range(r.experts)])
            down = torch.stack([take(f"{p}mlp.e{e}.down") for e in range(r.experts)])
            ff = make_part("feed_forward", "group_limited_glu_experts", w_router=take(p + "mlp.router"),
                           correction=take(p + "mlp.correction"), we_gate_up=gate_up.contiguous(), we_down=down.contiguous(),
                           top_k=r.top, identity=r.identity, groups=r.groups, keep=r.keep, route_scale=r.scale,
                           glu=K.glu_form(GLU_ALPHA, r.expert.limit, GLU_SHIFT),
                           shared=None if r.shared is None else glu_unit(p + "mlp.shared.", r.shared))
        if S is None:
            blocks.append(make_part("block", "pre_norm", norm1=norm(p + "norm1"), mixer=mixer,
                                    norm2=None if ff is None else norm(p + "norm2"), feed_forward=ff))
        else:
            blocks.append(make_part(
                "block", "hyper_connection", norm1=norm(p + "norm1", take(p + "hc1.in")), mixer=mixer, mix1=take(p + "hc1.mix"),
                write1=take(p + "hc1.out"), norm2=None if ff is None else norm(p + "norm2", take(p + "hc2.in")), feed_forward=ff,
                mix2=None if ff is None else take(p + "hc2.mix"), write2=None if ff is None else take(p + "hc2.out")))
    # the schedule: a layer with kv_from reads the cache that the named layer fills
    schedule, cache_of, c, s = [], {}, 0, 0
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if isinstance(m, RetentionSpec):
            schedule.append(LayerRun(i, None, True, s))
            s += 1
        elif getattr(m, "kv_from", None) is not None:
            schedule.append(LayerRun(i, cache_of[m.kv_from], False, None))
        else:
            cache_of[i] = c
            schedule.append(LayerRun(i, c, True, None))
            c += 1
    embedding = take("embed").contiguous()
    final_norm = norm("final.norm")
    return DecoderModel(runtime, embedding, blocks, final_norm, embedding, schedule=schedule, config=cfg, residual_streams=S)


KODUZEN = Architecture(name="Koduzen", parse_config=KoduzenConfig.from_dict, tensor_specs=tensor_specs, build=build)
register_architecture(KODUZEN)
