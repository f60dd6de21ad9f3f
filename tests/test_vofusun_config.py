"""Vofusun without a GPU: the configuration reader, the tensor list, random model folders, the order of layer runs, and
the plain implementation against other ways of writing the same mathematics."""

import json
import math

import pytest
import torch

from tests import vofusun_helpers as VH
from tests.plain import vofusun_plain as plain


def test_config_is_read_from_the_files_own_keys():
    from jax_llm_examples_b200.config.registry import resolve
    from jax_llm_examples_b200.config.vofusun import ChunkAttentionSpec, DeltaSpec, VofusunConfig, WindowAttentionSpec

    cj = VH.config("small")
    arch = resolve(cj)
    assert arch.name == "Vofusun"
    cfg = arch.parse_config(cj)
    assert isinstance(cfg, VofusunConfig) and (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.embedding_scale) == (61, 36, 1e-5, 2.5)
    assert [type(L.mixer) for L in cfg.layers] == [WindowAttentionSpec, DeltaSpec, ChunkAttentionSpec, DeltaSpec]
    a, d, c = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[2].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.scale) == (6, 2, 10, 6, 7, 0.4)
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 5, 9, 3)
    assert (c.heads, c.kv_heads, c.dim, c.vdim, c.chunk, c.scale, c.rot_base, c.rot_dims) == (3, 1, 12, 12, 11, 0.3, 40.0, 8)
    assert (c.rot_scaling.factor, c.rot_scaling.low, c.rot_scaling.high, c.rot_scaling.original) == (4.0, 1.0, 3.0, 30.0)
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 30
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 3, 3)
    # no rotation and no scaling are configurations too
    p = VofusunConfig.from_dict(VH.config("padded"))
    assert p.layers[1].mixer.rot_dims == 0 and p.layers[1].mixer.rot_scaling is None
    w = VofusunConfig.from_dict(VH.config("wide"))
    assert w.loop is None and w.layers[0].mixer.rot_dims == 64 and w.layers[0].mixer.rot_scaling is None


def test_the_order_of_layer_runs():
    from jax_llm_examples_b200.config.vofusun import VofusunConfig

    order = VofusunConfig.from_dict(VH.config("small")).layer_order()
    assert order == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert order == plain.layer_order(VH.config("small"))
    assert VofusunConfig.from_dict(VH.config("wide")).layer_order() == [(0, False), (1, False), (2, False)]
    whole = VofusunConfig.from_dict(VH.config("padded")).layer_order()
    assert whole == [(0, False), (1, False), (2, False), (3, False), (0, True), (1, False), (2, False), (3, False)]
    assert VofusunConfig.from_dict(VH.config("recurrent")).layer_order() == [(0, False), (1, False), (1, True)]
    once = VH.config("small")
    once["loop"]["times"] = 1
    assert all(not opens for _, opens in VofusunConfig.from_dict(once).layer_order())


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "mamba", "no mixer"),
    (("layers", 0, "mixer", "kv_heads"), 4, "no multiple"),
    (("layers", 1, "mixer", "kv_heads"), 3, "no multiple"),
    (("layers", 2, "mixer", "rot", "dims"), 5, "even"),
    (("layers", 2, "mixer", "rot", "dims"), 14, "at most"),
    (("layers", 2, "mixer", "vdim"), 10, "values are the keys"),
    (("layers", 0, "mlp", "kind"), "moe", "dense"),
    (("norm", "eps"), 0.0, "eps"),
    (("loop", "stop"), 5, "loop"),
    (("loop", "times"), 0, "times"),
    (("layers", 1, "mixer", "conv"), 0, "conv"),
])
def test_config_errors_name_the_key(path, value, word):
    from jax_llm_examples_b200.config.base import ConfigError
    from jax_llm_examples_b200.config.vofusun import VofusunConfig

    cj = VH.config("small")
    d = cj
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        VofusunConfig.from_dict(cj)
    cj = VH.config("small")
    del cj["layers"][0]["mixer"]["mask"]
    with pytest.raises(ConfigError, match="mask"):
        VofusunConfig.from_dict(cj)


def test_tensor_list_and_random_folder(tmp_path):
    """A folder written from a configuration holds exactly the architecture's tensors, in the shapes the sizes give."""
    from jax_llm_examples_b200.config.registry import resolve
    from jax_llm_examples_b200.weights.loader import WeightError, load_tensors

    folder = VH.make_dir(tmp_path / "m", "small", seed=3)
    cj = json.loads((folder / "config.json").read_text())
    arch = resolve(cj)
    specs = arch.tensor_specs(arch.parse_config(cj))
    P = plain.read_safetensors(folder / "model.safetensors")
    assert set(P) == set(specs)
    assert P["l0.mix.q"].shape == (60, 36) and P["l0.mix.v"].shape == (12, 36) and P["l0.mix.o"].shape == (36, 36)
    assert P["l1.mix.q"].shape == (10, 36) and P["l1.mix.q.conv"].shape == (10, 3) and P["l1.mix.v.conv"].shape == (36, 3)
    assert P["l1.mix.b"].shape == (4, 36) and P["l1.mix.A_log"].shape == (4,) and P["l1.mix.norm"].shape == (9,)
    assert P["l2.mix.g"].shape == (36, 36) and "l2.mix.v" not in P and "l1.norm2" not in P and "head" not in P
    wrong = json.loads(json.dumps(cj))
    wrong["layers"][1]["mixer"]["heads"] = 2
    with pytest.raises(WeightError, match="wrong shapes"):
        load_tensors(folder, arch.tensor_specs(arch.parse_config(wrong)), None, torch.float32)


def test_frequencies_follow_the_three_bands():
    from jax_llm_examples_b200.parts import rotary_frequencies, wavelength_scaled_frequencies

    base, dims, factor, low, high, orig = 40.0, 8, 4.0, 1.0, 3.0, 30.0
    f = wavelength_scaled_frequencies(base, dims, factor, low, high, orig).double()
    raw = rotary_frequencies(base, dims).double()
    lam = 2 * math.pi / raw
    assert lam[0] < orig / high and abs(float(f[0] - raw[0])) < 1e-7  # short waves stay
    assert orig / high <= lam[1] <= orig / low and raw[1] / factor < f[1] < raw[1]  # the band between: a blend
    s = (orig / lam[1] - low) / (high - low)
    assert abs(float(f[1] - ((1 - s) * raw[1] / factor + s * raw[1]))) < 1e-7
    assert lam[2] > orig / low and torch.allclose(f[2:], raw[2:] / factor, rtol=1e-6)  # long waves are slowed
    assert torch.allclose(f, plain.scaled_frequencies(base, dims, {"factor": factor, "low": low, "high": high, "original": orig}), rtol=1e-6)
    # equal bounds: no band between, and no division by zero
    g = wavelength_scaled_frequencies(base, dims, factor, 2.0, 2.0, orig)
    assert torch.isfinite(g).all()


def test_plain_delta_rule_equals_its_other_forms():
    """The recurrence of the plain implementation against (a) the same rule with the read-out written through the
    update, o = g S_old^T q + (q . k) u, and (b) for beta = 1 and no decay, the property that gives the rule its name:
    right after a token is written, reading the state with its unit key returns its value."""
    torch.manual_seed(0)
    T, D, eps = 11, 12, 1e-5
    h = torch.randn(T, D, dtype=torch.float64)
    m = {"heads": 4, "kv_heads": 2, "dim": 3, "vdim": 5, "conv": 3}
    P = {"q": torch.randn(6, D), "k": torch.randn(6, D), "v": torch.randn(20, D), "g": torch.randn(20, D), "b": torch.randn(4, D),
         "a": torch.randn(4, D), "A_log": torch.randn(4) * 0.3, "dt_bias": torch.randn(4), "norm": torch.rand(5) + 0.5,
         "o": torch.randn(D, 20), "q.conv": torch.randn(6, 3), "k.conv": torch.randn(6, 3), "v.conv": torch.randn(20, 3)}
    P = {"m." + k: v.double() for k, v in P.items()}
    got = plain.delta_mixer(h, P, "m.", m, eps)
    q = plain.unit_vector(plain.causal_conv_silu(h @ P["m.q"].T, P["m.q.conv"]).view(T, 2, 3)) * 3 ** -0.5
    k = plain.unit_vector(plain.causal_conv_silu(h @ P["m.k"].T, P["m.k.conv"]).view(T, 2, 3))
    v = plain.causal_conv_silu(h @ P["m.v"].T, P["m.v.conv"]).view(T, 4, 5)
    beta = torch.sigmoid(h @ P["m.b"].T)
    g = torch.exp(-torch.exp(P["m.A_log"]) * torch.log1p(torch.exp(h @ P["m.a"].T + P["m.dt_bias"])))
    S = torch.zeros(4, 3, 5, dtype=torch.float64)
    o = torch.zeros(T, 4, 5, dtype=torch.float64)
    for t in range(T):
        for a in range(4):
            kk, qq = k[t, a // 2], q[t, a // 2]
            u = beta[t, a] * (v[t, a] - g[t, a] * (S[a].T @ kk))
            o[t, a] = g[t, a] * (S[a].T @ qq) + (qq @ kk) * u
            S[a] = g[t, a] * S[a] + torch.outer(kk, u)
    o = o / (o.pow(2).mean(-1, keepdim=True) + eps).sqrt() * P["m.norm"]
    gate = h @ P["m.g"].T
    ref = (o.reshape(T, 20) * gate * torch.sigmoid(gate)) @ P["m.o"].T
    assert torch.allclose(got, ref, atol=1e-10)
    # the convolution: zeros before the start, the last tap is the token's own
    x = torch.randn(5, 2, dtype=torch.float64)
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = plain.causal_conv_silu(x, w)
    assert torch.allclose(y[:, 0], plain.silu(x[:, 0])) and torch.allclose(y[2:, 1], plain.silu(x[:-2, 1])) and float(y[:2, 1].abs().max()) == 0.0
    # (b) the delta property
    S = torch.zeros(3, 5, dtype=torch.float64)
    for t in range(T):
        kk = k[t, 0]
        before, n2 = S.T @ kk, float(kk @ kk)  # |k|^2 = 1 but for the 1e-6 under the root (which tells on a tiny key)
        S = S + torch.outer(kk, v[t, 0] - before)
        assert torch.allclose(S.T @ kk, n2 * v[t, 0] + (1 - n2) * before, atol=1e-12)
        assert n2 < 0.999 or torch.allclose(S.T @ kk, v[t, 0], atol=1e-2)


def test_plain_masks_sink_and_rotation():
    """A window of n: a query sees itself and n - 1 tokens before it.  A chunk of n: the positions of its own chunk,
    counted from 0.  The sink takes its share of the weight and gives nothing.  Rotated scores depend on the distance
    only, neighbouring entries turn together, entries beyond the rotated ones pass unchanged."""
    D = 8
    h = torch.eye(8, dtype=torch.float64)
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 8, "mask": {"size": 3}, "scale": 0.0}
    P = {"m.q": torch.zeros(4, D), "m.k": torch.zeros(4, D), "m.v": torch.eye(8), "m.o": torch.eye(8)}
    P = {k: v.double() for k, v in P.items()}
    out = plain.window_attention(h, P, "m.", m, 1e-6)  # scale 0: every score is 0, as the sink's: weights 1 / (1 + keys)
    assert torch.allclose(out[5], torch.tensor([0, 0, 0, 1, 1, 1, 0, 0], dtype=torch.float64) / 4)
    assert torch.allclose(out[1], torch.tensor([1, 1, 0, 0, 0, 0, 0, 0], dtype=torch.float64) / 3)
    assert torch.allclose(out[0], torch.tensor([1, 0, 0, 0, 0, 0, 0, 0], dtype=torch.float64) / 2)
    # chunks of 3: position 5 sees 3, 4, 5; position 6 opens a chunk and sees itself only
    m2 = {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "mask": {"size": 3}, "scale": 0.0}
    P2 = {"m.q": torch.zeros(8, D), "m.k": torch.eye(8), "m.g": torch.zeros(8, D), "m.o": torch.eye(8)}
    P2 = {k: v.double() for k, v in P2.items()}
    out = plain.chunk_attention(h, P2, "m.", m2, 1e-6)  # values = keys as projected = one-hot; the gate is a half
    assert torch.allclose(out[5], 0.5 * torch.tensor([0, 0, 0, 1, 1, 1, 0, 0], dtype=torch.float64) / 4)
    assert torch.allclose(out[6], 0.5 * torch.tensor([0, 0, 0, 0, 0, 0, 1, 0], dtype=torch.float64) / 2)
    assert torch.allclose(out[2], 0.5 * torch.tensor([1, 1, 1, 0, 0, 0, 0, 0], dtype=torch.float64) / 4)
    # the sink: p = exp(s) / (1 + sum exp(s)), also where every score is far below zero
    s = torch.tensor([-50.0, -51.0], dtype=torch.float64)
    assert torch.allclose(plain.softmax_with_sink(s), torch.exp(s) / (1 + torch.exp(s).sum()))
    s = torch.tensor([3.0, 1.0], dtype=torch.float64)
    assert torch.allclose(plain.softmax_with_sink(s), torch.exp(s) / (1 + torch.exp(s).sum()))
    # rotation of neighbouring pairs
    torch.manual_seed(1)
    x = torch.randn(7, 2, 10, dtype=torch.float64)
    pos = torch.arange(7)
    f = plain.scaled_frequencies(100.0, 6, None)
    y = plain.rotate_pairs(x, pos, f)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    z = torch.view_as_complex(x[..., :6].reshape(7, 2, 3, 2).contiguous()) * torch.polar(torch.ones(7, 1, 3, dtype=torch.float64),
                                                                                         pos.double()[:, None, None] * f[None, None, :])
    assert torch.allclose(torch.view_as_real(z).reshape(7, 2, 6), y[..., :6])
    same = x[:1].expand(7, 2, 10).contiguous()
    r = plain.rotate_pairs(same, pos, f)
    sc = torch.einsum("ihd,jhd->hij", r, r)
    assert torch.allclose(sc[:, 2, 0], sc[:, 5, 3]) and torch.allclose(sc[:, 6, 5], sc[:, 1, 0])


def test_plain_loop_adds_the_embedding_before_every_pass_but_the_first(tmp_path):
    """With every mixer and feed-forward silenced (output products zero), the stream is the embedding's output times
    the number of passes begun."""
    folder = VH.make_dir(tmp_path / "m", "small", seed=5)
    cfg, P = VH.plain_model(str(folder))
    P = {k: (torch.zeros_like(v) if k.endswith(".o") or k.endswith(".down") else v) for k, v in P.items()}
    toks = [3, 9, 27]
    _, after = plain.forward(cfg, P, toks)
    x0 = P["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    factor = [1, 1, 1, 2, 2, 3, 3, 3]
    assert after.shape[0] == len(factor)
    for run, f in enumerate(factor):
        assert torch.allclose(after[run], f * x0)
