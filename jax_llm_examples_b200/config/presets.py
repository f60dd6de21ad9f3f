"""Named configurations as data: the tiny test models and the benchmark layer sizes.

The reference keeps its two model sizes as constants in llama4/llama4_jax/configs.py:19-93.
Here a preset is a config.json dictionary, so it goes through the same reader as a file.
"""

from __future__ import annotations

from typing import Any


def _text(**kw: Any) -> dict[str, Any]:
    return {"architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text", **kw}


def _llama3(factor: float, low: float, high: float, orig: int) -> dict[str, Any]:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": low, "high_freq_factor": high,
            "original_max_position_embeddings": orig}


def _every_nth_nope(layers: int, n: int) -> list[int]:
    return [int((i + 1) % n != 0) for i in range(layers)]


PRESETS: dict[str, dict[str, Any]] = {
    # Tiny A: MoE on every layer, top-1 of 4, qk-norm on, no rope scaling, last layer NoPE.
    "tiny_a": _text(
        num_hidden_layers=4, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        interleave_moe_layer_step=1, num_local_experts=4, num_experts_per_tok=1, intermediate_size=128,
        intermediate_size_mlp=128, vocab_size=256, rope_theta=10000.0, rope_scaling=None, use_qk_norm=True,
        attention_chunk_size=32, no_rope_layers=[1, 1, 1, 0], attn_temperature_tuning=True, floor_scale=16.0,
        attn_scale=0.1, rms_norm_eps=1e-5, tie_word_embeddings=False),
    # Tiny B: MoE on odd layers, top-2 of 8, dense SwiGLU on even layers, llama3 rope scaling, no qk-norm.
    "tiny_b": _text(
        num_hidden_layers=8, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=24,
        interleave_moe_layer_step=2, num_local_experts=8, num_experts_per_tok=2, intermediate_size=64,
        intermediate_size_mlp=192, vocab_size=384, rope_theta=500000.0, rope_scaling=_llama3(8.0, 1.0, 4.0, 64),
        use_qk_norm=False, attention_chunk_size=48, no_rope_layers=_every_nth_nope(8, 4),
        attn_temperature_tuning=True, floor_scale=24.0, attn_scale=0.1, rms_norm_eps=1e-6,
        tie_word_embeddings=False),
    # Scout layer sizes, 16 layers (the benchmark configuration).
    "scout16": _text(
        num_hidden_layers=16, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
        interleave_moe_layer_step=1, num_local_experts=16, num_experts_per_tok=1, intermediate_size=8192,
        intermediate_size_mlp=16384, vocab_size=202048, rope_theta=500000.0,
        rope_scaling=_llama3(16.0, 1.0, 1.0, 8192), use_qk_norm=True, attention_chunk_size=8192,
        no_rope_layers=_every_nth_nope(16, 4), attn_temperature_tuning=True, floor_scale=8192.0, attn_scale=0.1,
        rms_norm_eps=1e-5, tie_word_embeddings=False),
    # Maverick layer sizes, 4 layers: dense layers 0 and 2, 128 experts on layers 1 and 3.
    "maverick4": _text(
        num_hidden_layers=4, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
        interleave_moe_layer_step=2, num_local_experts=128, num_experts_per_tok=1, intermediate_size=8192,
        intermediate_size_mlp=16384, vocab_size=202048, rope_theta=500000.0, rope_scaling=None,
        use_qk_norm=False, attention_chunk_size=8192, no_rope_layers=[1, 1, 1, 0], attn_temperature_tuning=True,
        floor_scale=8192.0, attn_scale=0.1, rms_norm_eps=1e-5, tie_word_embeddings=False),
}


def tebivik_sized(width: int, layers: int, heads: int, ff: int, vocab: int = 32768) -> dict[str, Any]:
    """A Tebivik configuration at the layer sizes of a real model: latent attention (head size 128 + 64 rotated, latent
    512, query latent 3/8 of the width) and HGRN2 (state 128 x 128 per head) in turn, a feed-forward in every layer,
    the first half of the layers run twice."""
    att = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 3 * width // 8, "kv_rank": 512,
                     "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}},
           "mlp": {"kind": "dense", "ff": ff}}
    rec = {"type": "hgrn2", "mixer": {"heads": heads, "dim": 128, "vdim": 128}, "mlp": {"kind": "dense", "ff": ff}}
    return {"architecture": "Tebivik", "vocab": vocab, "width": width, "residual_mult": 0.7, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6, "groups": 4}, "canon": {"taps": 4}, "loop": {"start": 0, "stop": layers // 2, "times": 2},
            "layers": [att if i % 2 == 0 else rec for i in range(layers)]}


def dense_llama_sized(width: int, layers: int, heads: int, ff: int, vocab: int = 32768) -> dict[str, Any]:
    """The closest model the framework had before: a dense Llama-4-style decoder of the same width, depth, head count
    and head size (4 query heads per KV head, SwiGLU of two thirds the other's feed-forward width, so that the
    feed-forward weights weigh the same), every layer rotary and unchunked."""
    return _text(num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads, num_key_value_heads=max(heads // 4, 1),
                 head_dim=128, interleave_moe_layer_step=0, moe_layers=[], num_local_experts=1, num_experts_per_tok=1,
                 intermediate_size=ff * 2 // 3 // 64 * 64, intermediate_size_mlp=ff * 2 // 3 // 64 * 64, vocab_size=vocab,
                 rope_theta=10000.0, rope_scaling=None, use_qk_norm=False, attention_chunk_size=1 << 20,
                 no_rope_layers=[1] * layers, attn_temperature_tuning=False, floor_scale=8192.0, attn_scale=0.1,
                 rms_norm_eps=1e-6, tie_word_embeddings=True)


# Tebivik: a tiny one (every size a multiple of 8, so bfloat16 products run on the tensor cores) and real layer sizes.
PRESETS["tebivik_tiny"] = {
    "architecture": "Tebivik", "vocab": 256, "width": 64, "residual_mult": 0.5, "embedding": {"scale": 2.0},
    "norm": {"eps": 1e-6, "groups": 2}, "canon": {"taps": 3}, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "hgrn2", "mixer": {"heads": 2, "dim": 16, "vdim": 24}, "mlp": {"kind": "dense", "ff": 96}},
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 4, "dim": 16, "rot_dim": 8, "vdim": 16, "q_rank": 24, "kv_rank": 32, "scale": 0.2,
                   "rot": {"base": 10000.0, "dims": 8}}},
        {"type": "hgrn2", "mixer": {"heads": 4, "dim": 8, "vdim": 16}, "mlp": None},
    ],
}
def makisun_sized(width: int, layers: int, heads: int, ff: int, vocab: int = 32768, experts: int = 0) -> dict[str, Any]:
    """A Makisun configuration at the layer sizes of a real model: layers of windowed attention (head size 128, four
    query heads per key head, a window of 1024, half the head rotated) beside gated linear attention (half as many heads,
    state 128 x 128), and time-mix layers (state 128 x 128 per head) in turn; a dense feed-forward in every layer, or
    with ``experts`` > 0 a mixture (top 2, each expert and the shared one a quarter of ``ff``) in every second layer."""
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": experts, "top": 2}, "shared": {"ff": ff // 4}}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": 128, "vdim": 128, "mask": {"size": 1024},
                              "rot": {"base": 10000.0, "dims": 64}, "scale": 128 ** -0.5},
                     "right": {"heads": max(heads // 2, 1), "dim": 128, "vdim": 128, "tau": 16.0, "decay_rank": 64},
                     "left_scale": 1.0, "right_scale": 1.0}}
    rec = {"type": "wkv", "mixer": {"heads": heads, "dim": 128, "decay_rank": 64}}
    return {"architecture": "Makisun", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [dict(par if i % 2 == 0 else rec, mlp=routed if experts and i % 2 else dense) for i in range(layers)]}


PRESETS["makisun_tiny"] = {
    "architecture": "Makisun", "vocab": 256, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "wkv", "mixer": {"heads": 2, "dim": 16, "decay_rank": 8},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 16}}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "mask": {"size": 24}, "rot": {"base": 10000.0, "dims": 8},
                            "scale": 0.25},
                   "right": {"heads": 2, "dim": 8, "vdim": 16, "tau": 4.0, "decay_rank": 8}, "left_scale": 0.75, "right_scale": 1.25}},
        {"type": "wkv", "mixer": {"heads": 4, "dim": 8, "decay_rank": 8}, "mlp": None},
    ],
}
def vofusun_sized(width: int, layers: int, heads: int, ff: int, vocab: int = 32768) -> dict[str, Any]:
    """A Vofusun configuration at the layer sizes of a real model: windowed attention with a sink (head size 128, four
    query heads per key head, a window of 1024, no rotation), the gated delta rule (state 128 x 128 per head, two heads
    per key head, convolutions over 4 tokens) and chunked, gated attention whose keys are its values (chunks of 2048,
    the whole head rotated in pairs with wavelength-scaled frequencies) in turn; a dense feed-forward in every layer."""
    kv = max(heads // 4, 1)
    kinds = [
        {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 128 ** -0.5}},
        {"type": "delta", "mixer": {"heads": heads, "kv_heads": max(heads // 2, 1), "dim": 128, "vdim": 128, "conv": 4}},
        {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "mask": {"size": 2048}, "scale": 1.0 / 128,
                                          "rot": {"base": 500000.0, "dims": 128,
                                                  "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}},
    ]
    return {"architecture": "Vofusun", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [dict(kinds[i % 3], mlp={"kind": "dense", "ff": ff}) for i in range(layers)]}


# Vofusun, tiny: a looped stretch (layers 1 and 2, twice), a layer without a feed-forward, part of the head rotated.
PRESETS["vofusun_tiny"] = {
    "architecture": "Vofusun", "vocab": 256, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "mask": {"size": 24}, "scale": 0.25}},
        {"type": "delta", "mlp": None, "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 3}},
        {"type": "attention_2", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "mask": {"size": 40}, "scale": 0.2,
                   "rot": {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 64}}}},
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
def koduzen_sized(width: int, layers: int, heads: int, ff: int, vocab: int = 32768, experts: int = 0, streams: int = 2) -> dict[str, Any]:
    """A Koduzen configuration at the layer sizes of a real model, ``streams`` residual rows per token: biased attention
    (head size 128, four query heads per key head, a window of 1024, a query temperature), a second such layer that reads
    the first one's keys and values, retention (state 128 x 128 per head, half of each head rotated) and attention normed
    over the whole projection with YaRN-scaled rotation in turn; a dense gated unit in every layer, or with ``experts``
    > 0 a mixture (top 2 of the experts plus two that hand their input on, in groups of which half are kept; each expert
    and the shared one a quarter of ``ff``) in every second layer."""
    kv = max(heads // 4, 1)
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    groups = 2 if (experts + 2) % 2 == 0 else 1
    routed = {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0}, "shared": {"ff": ff // 4, "limit": 7.0},
              "router": {"experts": experts, "identity": 2, "top": 2, "scale": 1.0, "groups": {"count": groups, "keep": max(groups // 2, 1)}}}
    biased = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 128 ** -0.5,
              "q_temp": {"coef": 0.1, "every": 1024}}
    kinds = [
        lambda i: {"type": "attention_2", "mixer": dict(biased)},
        lambda i: {"type": "attention_2", "mixer": dict(biased, kv_from=i - 1)},
        lambda i: {"type": "retention", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "rot": {"base": 10000.0, "dims": 64},
                                                  "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(heads - 1, 1)) for h in range(heads)]}},
        lambda i: {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 128 ** -0.5,
                                                  "rot": {"base": 250000.0, "dims": 128,
                                                          "scaling": {"factor": 4.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}},
    ]
    cfg = {"architecture": "Koduzen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
           "layers": [dict(kinds[i % 4](i), mlp=routed if experts and i % 2 else dense) for i in range(layers)]}
    if streams:
        cfg["streams"] = streams
    return cfg


# Koduzen, tiny: three streams, a layer that reads its neighbour's keys, identity experts in groups, a layer without a feed-forward.
PRESETS["koduzen_tiny"] = {
    "architecture": "Koduzen", "vocab": 256, "width": 64, "norm": {"eps": 1e-6}, "streams": 3,
    "layers": [
        {"type": "attention_2", "mlp": {"kind": "dense", "ff": 96, "limit": 2.0},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "mask": {"size": 24}, "scale": 0.25, "q_temp": {"coef": 0.2, "every": 8}}},
        {"type": "attention_2", "mlp": {"kind": "moe", "expert": {"ff": 32, "limit": 1.0}, "shared": {"ff": 16, "limit": 1.0},
                                        "router": {"experts": 4, "identity": 2, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "mask": {"size": 40}, "scale": 0.2, "kv_from": 0}},
        {"type": "retention", "mlp": None, "mixer": {"heads": 2, "dim": 8, "vdim": 16, "decay": [0.97, 0.995], "rot": {"base": 10000.0, "dims": 4}}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 64, "limit": 1.0},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "mask": {"size": 33}, "scale": 0.2,
                   "rot": {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}}},
    ],
}
PRESETS["koduzen_2k"] = koduzen_sized(2048, 8, 16, 8192)
PRESETS["koduzen_4k"] = koduzen_sized(4096, 8, 32, 14336)
PRESETS["vofusun_2k"] = vofusun_sized(2048, 8, 16, 8192)
PRESETS["vofusun_4k"] = vofusun_sized(4096, 8, 32, 14336)
PRESETS["makisun_2k"] = makisun_sized(2048, 8, 16, 8192)
PRESETS["makisun_4k"] = makisun_sized(4096, 8, 32, 14336)
PRESETS["tebivik_2k"] = tebivik_sized(2048, 8, 16, 8192)
PRESETS["tebivik_4k"] = tebivik_sized(4096, 8, 32, 14336)
PRESETS["scout8_long"] = {**PRESETS["scout16"], "num_hidden_layers": 8, "no_rope_layers": _every_nth_nope(8, 4)}


def preset(name: str, **overrides: Any) -> dict[str, Any]:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {', '.join(sorted(PRESETS))}")
    d = dict(PRESETS[name])
    d.update(overrides)
    if "num_hidden_layers" in overrides and "no_rope_layers" not in overrides and "no_rope_layers" in PRESETS[name]:
        n = overrides["num_hidden_layers"]
        base = PRESETS[name]["no_rope_layers"]
        d["no_rope_layers"] = [base[i % len(base)] for i in range(n)]
    return d
