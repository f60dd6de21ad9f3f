"""Koduzen without a GPU: the configuration reader, the tensor list, random model folders, which cache a layer reads, and
the plain implementation against other ways of writing the same mathematics."""

import json
import math

import pytest
import torch

from tests import koduzen_helpers as KH
from tests.plain import koduzen_plain as plain

F64 = torch.float64


def test_config_is_read_from_the_files_own_keys():
    from jax_llm_examples_b200.config.koduzen import AttentionSpec, BiasedAttentionSpec, GluSpec, KoduzenConfig, MoeSpec, RetentionSpec
    from jax_llm_examples_b200.config.registry import resolve

    cj = KH.config("small")
    arch = resolve(cj)
    assert arch.name == "Koduzen"
    cfg = arch.parse_config(cj)
    assert isinstance(cfg, KoduzenConfig) and (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.streams) == (61, 36, 1e-5, 3)
    assert [type(L.mixer) for L in cfg.layers] == [BiasedAttentionSpec, RetentionSpec, BiasedAttentionSpec, AttentionSpec, RetentionSpec]
    b, r, rd, a = (cfg.layers[i].mixer for i in (0, 1, 2, 3))
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.window, b.scale, b.q_temp.coef, b.q_temp.every, b.kv_from) == (6, 2, 10, 6, 7, 0.4, 0.25, 5.0, None)
    assert (r.heads, r.dim, r.vdim, r.decay, r.rot.base, r.rot.dims, r.rot.scaling) == (4, 5, 9, (0.9, 0.97, 0.99, 1.0), 50.0, 4, None)
    assert (rd.kv_from, rd.window, rd.q_temp) == (0, 19, None) and cfg.readers_of(0) == [2] and cfg.readers_of(2) == []
    assert (a.rot.dims, a.rot.scaling.factor, a.rot.scaling.original, a.rot.scaling.fast, a.rot.scaling.slow) == (8, 4.0, 30.0, 4.0, 1.0)
    d, m, last = cfg.layers[0].mlp, cfg.layers[1].mlp, cfg.layers[4]
    assert isinstance(d, GluSpec) and (d.ff, d.limit) == (30, 0.8) and last.mlp is None and last.mixer.rot is None
    assert isinstance(m, MoeSpec) and (m.experts, m.identity, m.top, m.groups, m.keep, m.scale) == (5, 1, 2, 3, 2, 1.5)
    assert (m.expert.ff, m.expert.limit, m.shared.ff, m.shared.limit) == (14, 0.7, 10, 1.2)
    plainer = cfg.layers[3].mlp
    assert (plainer.identity, plainer.groups, plainer.keep, plainer.scale, plainer.shared) == (0, 1, 1, 1.0, None)
    assert KoduzenConfig.from_dict(KH.config("recurrent")).streams is None and KoduzenConfig.from_dict(KH.config("padded")).streams == 1


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "mamba", "no mixer"),
    (("layers", 0, "mixer", "kv_heads"), 4, "no multiple"),
    (("layers", 3, "mixer", "rot", "dims"), 5, "even"),
    (("layers", 3, "mixer", "rot", "dims"), 14, "at most"),
    (("layers", 1, "mixer", "decay"), [0.5, 0.5], "decay"),
    (("layers", 1, "mixer", "decay"), [0.5, 0.5, 1.5, 0.5], "decay"),
    (("layers", 2, "mixer", "kv_from"), 1, "attention_2"),
    (("layers", 2, "mixer", "kv_from"), 2, "earlier"),
    (("layers", 2, "mixer", "dim"), 12, "layer 0 keeps"),
    (("layers", 0, "mlp", "kind"), "swiglu", "dense"),
    (("layers", 0, "mlp", "limit"), 0.0, "limit"),
    (("layers", 1, "mlp", "router", "top"), 7, "top-7"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "groups"),
    (("norm", "eps"), 0.0, "eps"),
    (("streams",), 0, "streams"),
])
def test_config_errors_name_the_key(path, value, word):
    from jax_llm_examples_b200.config.base import ConfigError
    from jax_llm_examples_b200.config.koduzen import KoduzenConfig

    cj = KH.config("small")
    d = cj
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        KoduzenConfig.from_dict(cj)
    cj = KH.config("small")
    del cj["layers"][0]["mixer"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        KoduzenConfig.from_dict(cj)
    cj = KH.config("recurrent")
    cj["layers"][0]["mixer"]["rot"]["scaling"] = {"factor": 2.0, "original": 8, "fast": 2.0, "slow": 1.0}
    with pytest.raises(ConfigError, match="no frequency scaling"):
        KoduzenConfig.from_dict(cj)


def test_tensor_list_and_random_folder(tmp_path):
    """A folder written from a configuration holds exactly the architecture's tensors, in the shapes the sizes give."""
    from jax_llm_examples_b200.config.registry import resolve
    from jax_llm_examples_b200.weights.loader import WeightError, load_tensors

    folder = KH.make_dir(tmp_path / "m", "small", seed=3)
    cj = json.loads((folder / "config.json").read_text())
    arch = resolve(cj)
    specs = arch.tensor_specs(arch.parse_config(cj))
    P = plain.read_safetensors(folder / "model.safetensors")
    assert set(P) == set(specs)
    assert P["l0.mix.q"].shape == (60, 36) and P["l0.mix.v"].shape == (12, 36) and P["l0.mix.sink"].shape == (6,)
    assert P["l1.mix.q"].shape == (20, 36) and P["l1.mix.g"].shape == (36, 36) and P["l1.mix.o"].shape == (36, 36)
    assert "l2.mix.k" not in P and "l2.mix.v" not in P and P["l2.mix.sink"].shape == (6,)
    assert P["l3.mix.q.norm"].shape == (36,) and P["l3.mix.k.norm"].shape == (12,) and P["l3.mix.v"].shape == (7, 36)
    assert P["l1.mlp.router"].shape == (6, 36) and P["l1.mlp.correction"].shape == (6,) and "l1.mlp.e5.gate" not in P
    assert P["l1.mlp.e4.down"].shape == (36, 14) and P["l1.mlp.shared.up"].shape == (10, 36) and "l3.mlp.shared.up" not in P
    assert P["l0.hc1.in"].shape == (3,) and P["l0.hc2.mix"].shape == (3, 3) and "l4.hc2.in" not in P and "l4.norm2" not in P
    none = plain.read_safetensors(KH.make_dir(tmp_path / "r", "recurrent", seed=3) / "model.safetensors")
    assert not any(".hc" in n for n in none)
    wrong = json.loads(json.dumps(cj))
    wrong["layers"][1]["mixer"]["heads"] = 2
    wrong["layers"][1]["mixer"]["decay"] = [0.5, 0.5]
    with pytest.raises(WeightError, match="wrong shapes"):
        load_tensors(folder, arch.tensor_specs(arch.parse_config(wrong)), None, torch.float32)


def test_which_cache_a_layer_reads_and_how_long_its_pages_live(tmp_path):
    """A layer with kv_from gets the cache index of the layer it names and writes nothing; the named layer keeps its pages
    for the longest window among its readers; retention layers get a state slab and no cache."""
    from jax_llm_examples_b200.cache.manager import Retention
    from jax_llm_examples_b200.config.registry import resolve
    from jax_llm_examples_b200.parts import Runtime
    from jax_llm_examples_b200.weights.random_init import random_tensors

    def built(cj):
        arch = resolve(cj)
        cfg = arch.parse_config(cj)
        return arch.build(cfg, random_tensors(arch.tensor_specs(cfg), 1), Runtime(torch.float32, torch.device("cpu")))

    model = built(KH.config("small"))
    runs = [(r.block, r.cache, r.writes, r.state) for r in model.schedule]
    assert runs == [(0, 0, True, None), (1, None, True, 0), (2, 0, False, None), (3, 1, True, None), (4, None, True, 1)]
    assert model.plan.caches[0].retention == Retention.window(19) and model.plan.caches[1].retention == Retention.window(11)
    assert model.blocks[0].mixer.window == 7 and model.blocks[2].mixer.window == 19 and model.residual_streams == 3
    assert [tuple(s.shape) for s in model.plan.states] == [(4, 5, 9), (2, 7, 6)]
    wide = built(KH.config("wide"))
    assert [(r.cache, r.writes) for r in wide.schedule] == [(0, True), (None, True), (1, True), (1, False)]
    assert wide.plan.caches[1].retention == Retention.window(40)
    # a reader with a SHORTER window leaves the writer's own
    cj = KH.config("small")
    cj["layers"][2]["mixer"]["mask"]["size"] = 3
    assert built(cj).plan.caches[0].retention == Retention.window(7)
    rec = built(KH.config("recurrent"))
    assert rec.plan.caches == () and rec.residual_streams is None and len(rec.plan.states) == 2


def test_yarn_frequencies_keep_fast_waves_and_stretch_slow_ones():
    from jax_llm_examples_b200.parts import rotary_frequencies, yarn_frequencies

    base, dims, factor, original, fast, slow = 10000.0, 32, 8.0, 256, 16.0, 1.0
    f, amp = yarn_frequencies(base, dims, factor, original, fast, slow)
    ref, ramp_amp = plain.yarn_frequencies(base, dims, {"factor": factor, "original": original, "fast": fast, "slow": slow})
    assert torch.allclose(f.double(), ref, rtol=1e-6) and amp == pytest.approx(0.1 * math.log(8.0) + 1.0) and amp == pytest.approx(ramp_amp)
    plain_f = rotary_frequencies(base, dims).double()
    turns = original * plain_f / (2 * math.pi)  # turns that each pair's wave makes over the original length
    kept, stretched = turns > fast * 2.0, turns < slow / 2.0
    assert kept.any() and stretched.any() and (~kept & ~stretched).any()
    assert torch.allclose(f.double()[kept], plain_f[kept], rtol=1e-6) and torch.allclose(f.double()[stretched], plain_f[stretched] / factor, rtol=1e-6)
    between = ~kept & ~stretched
    assert ((f.double()[between] <= plain_f[between] * (1 + 1e-6)) & (f.double()[between] >= plain_f[between] / factor * (1 - 1e-6))).all()
    # lo = hi (no pair between the two limits): the ramp is a step and nothing divides by zero
    f2, _ = yarn_frequencies(100.0, 8, 2.0, 64, 1.0, 1.0)
    assert torch.isfinite(f2).all()


def test_plain_retention_equals_its_sum_over_the_past():
    """o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j, per head."""
    torch.manual_seed(0)
    T, H, d, dv = 13, 3, 4, 5
    q, k, v = torch.randn(T, H, d, dtype=F64), torch.randn(T, H, d, dtype=F64), torch.randn(T, H, dv, dtype=F64)
    decay = [0.9, 1.0, 0.5]
    o = plain.retention_recurrence(q, k, v, decay)
    for a in range(H):
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        w = torch.where(i >= j, torch.tensor(decay[a], dtype=F64) ** (i - j).clamp_min(0), torch.zeros((), dtype=F64))
        assert torch.allclose(o[:, a], ((q[:, a] @ k[:, a].T) * w) @ v[:, a], atol=1e-12)


def test_plain_attention_pieces():
    torch.manual_seed(1)
    T = 9
    m = plain.window_mask(T, 3)
    assert m[5].tolist() == [False, False, False, True, True, True, False, False, False] and m[0].sum() == 1
    # the sink takes its share and carries nothing: with one visible key of score 0 and a sink of ln 3 the key weighs 1/4
    q, k, v = torch.zeros(T, 1, 2, dtype=F64), torch.zeros(T, 1, 2, dtype=F64), torch.ones(T, 1, 2, dtype=F64)
    out = plain.softmax_attention(q, k, v, 1.0, plain.window_mask(T, 1), sink=torch.tensor([math.log(3.0)], dtype=F64))
    assert torch.allclose(out, torch.full((T, 2), 0.25, dtype=F64))
    # the distance bias: two keys with equal scores, one 2 further back, weigh as 1 : exp(-2 slope)
    bias = plain.distance_bias(T, 4)
    assert bias.shape == (4, T, T) and float(bias[1, 6, 2]) == pytest.approx(2.0 ** -4 * 4) and float(bias[3, 6, 6]) == 0.0
    v2 = torch.zeros(T, 1, 2, dtype=F64)
    v2[5, 0, 0], v2[7, 0, 1] = 1.0, 1.0
    out = plain.softmax_attention(torch.zeros(T, 4, 2, dtype=F64), k, v2, 1.0, torch.zeros(T, T, dtype=torch.bool).index_put_(
        (torch.tensor([8, 8]), torch.tensor([5, 7])), torch.tensor(True)) | torch.eye(T, dtype=torch.bool) & (torch.arange(T) < 8)[:, None], bias=bias)
    for a in range(4):
        assert float(out[8, 2 * a] / out[8, 2 * a + 1]) == pytest.approx(math.exp(-2.0 * 2.0 ** (-8.0 * (a + 1) / 4)))
    # the query temperature steps where floor((p + 1) / every) steps
    t = plain.query_temperature(10, 0.5, 4)
    assert t[0] == t[2] == 1.0 and t[3] == t[6] == pytest.approx(1 + 0.5 * math.log(2.0)) and t[7] == pytest.approx(1 + 0.5 * math.log(3.0))
    # rotate-half turns pairs (i, i + dims / 2) and leaves the rest; the amplitude stretches what it turns
    x = torch.randn(T, 2, 6, dtype=F64)
    f = plain.plain_frequencies(100.0, 4)
    y = plain.rotate_half(x, torch.arange(T), f, 4, 1.5)
    assert torch.equal(y[..., 4:], x[..., 4:]) and torch.allclose(y[0, :, :4], 1.5 * x[0, :, :4])
    assert torch.allclose((y[..., 0] ** 2 + y[..., 2] ** 2), 2.25 * (x[..., 0] ** 2 + x[..., 2] ** 2))


def test_plain_router_groups_corrections_and_identity_experts():
    torch.manual_seed(2)
    D, T = 8, 40
    P = {"m.router": torch.randn(6, D, dtype=F64), "m.correction": torch.tensor([0.0, -0.3, 0.2, 0.0, 0.5, -1.0], dtype=F64)}
    for e in range(4):
        P[f"m.e{e}.gate"], P[f"m.e{e}.up"], P[f"m.e{e}.down"] = torch.randn(5, D, dtype=F64), torch.randn(5, D, dtype=F64), torch.randn(D, 5, dtype=F64)
    h = torch.randn(T, D, dtype=F64)
    r = {"experts": 4, "identity": 2, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    chosen, w = plain.route(h, P, "m.", r)
    s = torch.softmax(h @ P["m.router"].T, -1)
    for t in range(T):
        c = (s[t] + P["m.correction"]).tolist()
        groups = sorted(range(3), key=lambda g: -max(c[2 * g], c[2 * g + 1]))[:2]
        allowed = [e for e in range(6) if e // 2 in groups]
        best = sorted(allowed, key=lambda e: -c[e])[:2]
        assert sorted(chosen[t].tolist()) == sorted(best)
        share = s[t, chosen[t]]
        assert torch.allclose(w[t], share / share.sum() * 2.0)
    ml = {"kind": "moe", "router": r, "expert": {"ff": 5, "limit": 0.7}}
    out, used, own = plain.expert_mixture(h, P, "m.", ml)
    assert torch.equal(used, own)
    t = next(t for t in range(T) if (chosen[t] >= 4).any())  # a token that took an identity expert: its own row, weighted
    want = sum(wt * (h[t] if c >= 4 else plain.clipped_glu(h[t:t + 1], P, f"m.e{c}.", 0.7)[0]) for c, wt in zip(chosen[t].tolist(), w[t]))
    assert torch.allclose(out[t], want)
    # the gated unit clips the gate from above only and the linear half on both sides, and adds one to it
    Pg = {"g.gate": torch.eye(3, dtype=F64), "g.up": torch.eye(3, dtype=F64), "g.down": torch.eye(3, dtype=F64)}
    y = plain.clipped_glu(torch.tensor([[5.0, -5.0, 0.5]], dtype=F64), Pg, "g.", 2.0)[0]
    assert float(y[0]) == pytest.approx(2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0)
    assert float(y[1]) == pytest.approx(-5.0 / (1 + math.exp(1.702 * 5.0)) * -1.0)
    assert float(y[2]) == pytest.approx(0.5 / (1 + math.exp(-1.702 * 0.5)) * 1.5)


def test_plain_streams_reduce_to_a_residual_sum():
    """One stream with read, write and mix weights of one is the plain residual block; S equal streams with an identity
    mix, read weights that sum to one and write weights of one stay equal."""
    torch.manual_seed(3)
    T, D = 5, 6
    x = torch.randn(T, D, dtype=F64)
    fn = lambda u: torch.tanh(u) * 2.0  # noqa: E731
    one = {"h.in": torch.ones(1, dtype=F64), "h.out": torch.ones(1, dtype=F64), "h.mix": torch.ones(1, 1, dtype=F64)}
    assert torch.allclose(plain.hyper_sublayer(x[None], one, "h.", fn)[0], x + fn(x))
    three = {"h.in": torch.tensor([0.2, 0.5, 0.3], dtype=F64), "h.out": torch.ones(3, dtype=F64), "h.mix": torch.eye(3, dtype=F64)}
    X = plain.hyper_sublayer(x[None].repeat(3, 1, 1), three, "h.", fn)
    assert torch.allclose(X[0], x + fn(x)) and torch.allclose(X[1], X[0]) and torch.allclose(X[2], X[0])
    # the mix matrix is indexed [from, to]
    swap = {"h.in": torch.tensor([1.0, 0.0], dtype=F64), "h.out": torch.zeros(2, dtype=F64), "h.mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=F64)}
    X = plain.hyper_sublayer(torch.stack([x, 2 * x]), swap, "h.", fn)
    assert torch.allclose(X[1], x) and torch.allclose(X[0], torch.zeros_like(x))
