"""Shared by the Koduzen tests: small configurations of their own, model folders from a seed, the plain implementation's
logits and the comparison of a trace's rows with them."""

from __future__ import annotations

import copy
import functools
import json
from pathlib import Path

import numpy as np
import torch

from tests.plain import koduzen_plain as plain


def retention(heads, dim, vdim, decay, rot=None, mlp=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "retention", "mlp": mlp, "mixer": m}


def attention(heads, kv, dim, vdim, window, scale, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale}
    if rot is not None:
        base, dims, scaling = rot
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            factor, original, fast, slow = scaling
            m["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return {"type": "attention", "mlp": mlp, "mixer": m}


def attention_2(heads, kv, dim, vdim, window, scale, q_temp=None, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mlp": mlp, "mixer": m}


def dense(ff, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, identity=0, groups=None, scale=1.0, limit=1.0, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if identity:
        r["identity"] = identity
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    d = {"kind": "moe", "router": r, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


CONFIGS = {
    # every size small and odd (no size is a multiple of 8: every product runs on the 32-bit FMA kernel in both
    # precisions); three streams; windows shorter than a page; values of another size than keys; three query heads per
    # key head; a layer that reads the keys of layer 0 through a LONGER window than layer 0's own; part of the head
    # rotated, with the frequency scaling's ramp in use; limits other than 1; a router with identity experts and groups
    "small": {
        "architecture": "Koduzen", "vocab": 61, "width": 36, "norm": {"eps": 1e-5}, "streams": 3,
        "layers": [attention_2(6, 2, 10, 6, 7, 0.4, (0.25, 5), None, dense(30, 0.8)),
                   retention(4, 5, 9, (0.9, 0.97, 0.99, 1.0), (50.0, 4), moe(5, 2, 14, 1, (3, 2), 1.5, 0.7, (10, 1.2))),
                   attention_2(6, 2, 10, 6, 19, 0.3, None, 0, dense(20, 2.0)),
                   attention(3, 1, 12, 7, 11, 0.3, (40.0, 8, (4.0, 30, 4.0, 1.0)), moe(4, 1, 9)),
                   retention(2, 7, 6, (0.95, 0.5), None)],
    },
    # sizes in multiples of 8 (bfloat16 products on the tcgen05 streaming kernel with the gated unit in its epilogue,
    # attention on the tensor-core kernels at head sizes 64 and 128); two streams; one key head for four query heads;
    # windows that straddle page borders; the whole head rotated without frequency scaling; a reader with the writer's
    # own window; eight experts in four groups of which two are kept
    "wide": {
        "architecture": "Koduzen", "vocab": 96, "width": 128, "norm": {"eps": 1e-6}, "streams": 2,
        "layers": [attention(4, 1, 64, 64, 24, 0.11, (10000.0, 64, None), dense(256)),
                   retention(2, 32, 64, (0.98, 0.995), (10000.0, 32), moe(6, 2, 64, 2, (4, 2), 2.0, 1.0, (64, 1.0))),
                   attention_2(2, 2, 128, 128, 40, 0.09, (0.3, 16), None, dense(64)),
                   attention_2(2, 2, 128, 128, 40, 0.07, (0.1, 7), 2, moe(4, 2, 32))],
    },
    # keys shorter than values and both padded in the cache (to 64 in bfloat16); ONE stream that still has read, write
    # and mix weights; no rotation at all; a window of one token (a query sees itself, or itself and the sink); top-1
    # routing; the model's last layer has no feed-forward
    "padded": {
        "architecture": "Koduzen", "vocab": 50, "width": 48, "norm": {"eps": 1e-6}, "streams": 1,
        "layers": [attention(3, 3, 24, 40, 1, 0.2, None, dense(40)),
                   attention_2(2, 2, 16, 24, 1, 0.25, None, None, moe(3, 1, 16, 0, None, 1.0, 1.0, (8, 0.5))),
                   retention(3, 16, 8, (1.0, 1.0, 0.9), (10000.0, 16), dense(24)),
                   attention_2(2, 1, 40, 24, 33, 0.15, (0.5, 1))],
    },
    # no "streams" key: one residual row and a plain residual sum; retention only: a model without a page of cache
    "recurrent": {
        "architecture": "Koduzen", "vocab": 40, "width": 32, "norm": {"eps": 1e-6},
        "layers": [retention(2, 16, 16, (0.9, 0.99), (100.0, 8), dense(48)), retention(4, 24, 4, (0.999, 0.8, 1.0, 0.97), None, moe(3, 2, 16, 2))],
    },
}


def random_config(rng) -> dict:
    """A configuration drawn at random: two to six layers of the three mixers in any order, odd and even sizes, one to
    four query heads per key head, windows from one token to more than a prompt, with and without rotation, frequency
    scaling and query temperature, layers that read an earlier layer's keys, every kind of feed-forward, 1 to 4 streams
    or none."""
    width = rng.choice([24, 40, 64, 96, 128])

    def mlp():
        u = rng.random()
        if u < 0.15:
            return None
        if u < 0.5:
            return dense(rng.choice([16, 24, 72, 128]), rng.choice([0.5, 1.0, 3.0]))
        experts, identity = rng.choice([2, 3, 4, 6, 8]), rng.choice([0, 0, 1, 2])
        total = experts + identity
        groups = None
        divisors = [g for g in (2, 3, 4) if total % g == 0]
        if divisors and rng.random() < 0.6:
            g = rng.choice(divisors)
            groups = (g, rng.randint(1, g))
        per_kept = total if groups is None else total // groups[0] * groups[1]
        top = rng.randint(1, min(4, per_kept))
        shared = None if rng.random() < 0.4 else (rng.choice([8, 16, 24]), rng.choice([0.5, 1.0]))
        return moe(experts, top, rng.choice([8, 12, 16, 32]), identity, groups, rng.choice([1.0, 2.0, 0.5]), rng.choice([0.6, 1.0]), shared)

    def rot(dim, scaling_ok):
        if rng.random() < 0.2:
            return None
        dims = rng.choice([d for d in (2, 4, 8, dim // 2, dim) if d <= dim and d % 2 == 0])
        base = rng.choice([100.0, 10000.0, 500000.0])
        if not scaling_ok:
            return (base, dims)
        scaling = None if rng.random() < 0.4 else (rng.choice([2.0, 4.0]), rng.choice([16, 64, 512]), rng.choice([8.0, 16.0]), rng.choice([1.0, 2.0]))
        return (base, dims, scaling)

    layers = []
    n = rng.randint(2, 6)
    for i in range(n):
        kind = rng.choice(["ret", "att", "at2", "at2"])
        if kind == "ret":
            heads, dim = rng.choice([1, 2, 3, 6]), rng.choice([4, 6, 16, 20, 32, 64])
            decay = [rng.choice([1.0, 0.999, 0.99, 0.9, 0.6]) for _ in range(heads)]
            layers.append(retention(heads, dim, rng.choice([4, 7, 16, 36, 64]), decay, rot(dim, False), mlp()))
        elif kind == "att":
            kv = rng.choice([1, 2, 3]); heads = kv * rng.choice([1, 2, 4]); dim = rng.choice([8, 12, 16, 32, 64, 128])
            layers.append(attention(heads, kv, dim, rng.choice([8, 20, 16, 64, 128]), rng.choice([1, 2, 5, 16, 17, 31, 64, 100]),
                                    rng.uniform(0.05, 0.4), rot(dim, True), mlp()))
        else:
            sources = [j for j, L in enumerate(layers) if L["type"] == "attention_2" and "kv_from" not in L["mixer"]]
            temp = None if rng.random() < 0.3 else (rng.uniform(0.05, 0.5), rng.choice([1, 3, 16, 64]))
            window = rng.choice([1, 3, 8, 16, 20, 33, 64, 100])
            if sources and rng.random() < 0.5:
                j = rng.choice(sources)
                src = layers[j]["mixer"]
                layers.append(attention_2(src["heads"], src["kv_heads"], src["dim"], src["vdim"], window, rng.uniform(0.05, 0.3), temp, j, mlp()))
            else:
                kv = rng.choice([1, 2]); heads = kv * rng.choice([1, 2, 4])
                layers.append(attention_2(heads, kv, rng.choice([8, 16, 24, 64, 128]), rng.choice([8, 16, 40, 64, 128]), window,
                                          rng.uniform(0.05, 0.3), temp, None, mlp()))
    cfg = {"architecture": "Koduzen", "vocab": rng.choice([37, 64, 100]), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    streams = rng.choice([None, 1, 2, 2, 3, 4])
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def mid_size_config(rng) -> dict:
    """A configuration drawn at random at sizes between the tiny ones above and a real model's: widths of 192 to 512, head
    sizes 32 to 128 (96 is padded to 128 in bfloat16), up to 32 query heads, windows of 40 to 300 tokens, 6 to 30 experts
    in up to 8 groups with up to 4 identity experts, four to seven layers."""
    width = rng.choice([192, 256, 384, 512])

    def mlp():
        u = rng.random()
        if u < 0.1:
            return None
        if u < 0.4:
            return dense(rng.choice([320, 512, 200]), rng.choice([1.0, 2.0, 7.0]))
        experts, identity = rng.choice([6, 12, 14, 30]), rng.choice([0, 2, 4, 2])
        total = experts + identity
        divisors = [g for g in (2, 4, 8) if total % g == 0]
        groups = None
        if divisors and rng.random() < 0.8:
            g = rng.choice(divisors)
            groups = (g, rng.randint(max(1, g // 2), g))
        per_kept = total if groups is None else total // groups[0] * groups[1]
        shared = None if rng.random() < 0.3 else (rng.choice([96, 64, 128]), rng.choice([1.0, 3.0]))
        return moe(experts, rng.randint(1, min(6, per_kept)), rng.choice([96, 64, 80, 128]), identity, groups, rng.choice([1.0, 2.0, 2.5]),
                   rng.choice([1.0, 4.0]), shared)

    layers = []
    for _ in range(rng.randint(4, 7)):
        kind = rng.choice(["ret", "att", "at2", "at2"])
        if kind == "ret":
            heads, dim = rng.choice([2, 4, 6, 8]), rng.choice([32, 64, 96, 128])
            rot = None if rng.random() < 0.2 else (rng.choice([1e4, 1e6]), rng.choice([d for d in (16, 32, dim) if d <= dim]))
            layers.append(retention(heads, dim, rng.choice([32, 64, 128]), [1 - 2.0 ** -rng.randint(3, 11) for _ in range(heads)], rot, mlp()))
        elif kind == "att":
            kv = rng.choice([1, 2, 4]); heads = kv * rng.choice([1, 2, 4]); dim = rng.choice([32, 64, 96, 128])
            sc = None if rng.random() < 0.3 else (rng.choice([4.0, 16.0]), rng.choice([256, 512, 4096]), rng.choice([16.0, 24.0]), rng.choice([1.0, 2.0]))
            rot = None if rng.random() < 0.15 else (rng.choice([1e4, 5e5]), rng.choice([d for d in (16, 32, 64, dim) if d <= dim]), sc)
            layers.append(attention(heads, kv, dim, rng.choice([32, 64, 128]), rng.choice([40, 72, 100, 128, 200, 300]), rng.uniform(0.05, 0.2), rot, mlp()))
        else:
            sources = [j for j, L in enumerate(layers) if L["type"] == "attention_2" and "kv_from" not in L["mixer"]]
            temp = None if rng.random() < 0.2 else (rng.uniform(0.1, 0.4), rng.choice([32, 50, 128, 100]))
            window = rng.choice([48, 64, 100, 130, 256])
            if sources and rng.random() < 0.5:
                j = rng.choice(sources)
                src = layers[j]["mixer"]
                layers.append(attention_2(src["heads"], src["kv_heads"], src["dim"], src["vdim"], window, rng.uniform(0.05, 0.2), temp, j, mlp()))
            else:
                kv = rng.choice([1, 2, 4]); heads = kv * rng.choice([1, 2, 4, 8])
                layers.append(attention_2(heads, kv, rng.choice([32, 64, 96, 128]), rng.choice([32, 64, 128]), window, rng.uniform(0.05, 0.2), temp, None, mlp()))
    cfg = {"architecture": "Koduzen", "vocab": rng.choice([300, 500, 1000]), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    streams = rng.choice([None, 1, 2, 2, 3, 4])
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def config(name: str, **overrides) -> dict:
    c = copy.deepcopy(CONFIGS[name])
    c.update(overrides)
    return c


def write_model(path, cfg: dict, seed: int):
    from jax_llm_examples_b200 import write_random_model

    return write_random_model(path, cfg, seed, norm_noise=0.1, std=0.15)


def make_dir(path, name: str, seed: int, **overrides):
    return write_model(path, config(name, **overrides), seed)


@functools.lru_cache(maxsize=32)
def plain_model(folder: str):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain.read_safetensors(folder / "model.safetensors")


def routed_layers(folder) -> list[int]:
    cfg, _ = plain_model(str(folder))
    return [i for i, L in enumerate(cfg["layers"]) if L.get("mlp") and L["mlp"]["kind"] == "moe"]


def plain_logits(folder, tokens, forced=None):
    """(logits [T, V], the share of (token, routed layer) pairs whose forced experts are not the set the plain router
    chose itself)."""
    cfg, P = plain_model(str(folder))
    trace = []
    with torch.no_grad():
        logits = plain.forward(cfg, P, list(tokens), forced, trace)
    differ = total = 0
    for _, used, own in trace:
        if used is not None:
            total += used.shape[0]
            differ += int((torch.sort(used, dim=1).values != torch.sort(own, dim=1).values).any(dim=1).sum())
    return logits.numpy(), differ / max(total, 1)


# float32: a few thousand roundings of 6e-8 per logit.  bfloat16: activations are rounded (4e-3) several times per layer,
# and a tiny model's logits are sums of few terms, so single rows scatter: the mean over all rows is held tight and a
# single row is capped where a fault (a lost state, a key off by one, a sink left out) would still stand out by far.
TOL = {"float32": 3e-5, "bfloat16": 1.2e-1}
TOL_MEAN = {"float32": 1e-5, "bfloat16": 3e-2}
# The share of choices that may differ from the plain router's: two scores that tie within the precision go either way
# (under 1 % were seen in bfloat16); a fault in the routing (a group, a correction, a tie rule) changes tens of percent.
OTHER_CHOICES = {"float32": 0.004, "bfloat16": 0.05}


def row_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Difference of two logit rows, each with its mean taken off, relative to the reference row's spread."""
    d = (got - got.mean()) - (ref - ref.mean())
    return float(np.sqrt((d ** 2).mean()) / max(np.sqrt(((ref - ref.mean()) ** 2).mean()), 1e-9))


def compare(folder, requests: dict, got: dict, routing: dict | None, dtype: str, stray: int = 0) -> float:
    """Every logit row a trace produced against the plain implementation's row at that place.  With ``routing`` (the
    engine's expert choices by (request, position)) the plain implementation takes those experts; they must be its own
    choice too but for a small share of near-ties.  Among hundreds of rows `stray` of them may scatter past the cap for
    a single row, up to twice as far; the mean stays as tight."""
    errs, shares = [], []
    routed = routed_layers(folder)
    for rid, toks in requests.items():
        forced = None
        if routing is not None and routed:
            forced = {layer: torch.as_tensor(np.stack([routing[(rid, p)][j] for p in range(len(toks))])) for j, layer in enumerate(routed)}
        ref, share = plain_logits(folder, toks, forced)
        shares.append((share, len(toks)))
        for pos in range(len(toks)):
            if (rid, pos) in got:
                err = row_err(got[(rid, pos)], ref[pos])
                assert err < TOL[dtype] * (2 if stray else 1), f"{dtype}: request {rid} position {pos}: relative error {err:.3e}"
                errs.append(err)
    other = sum(s * n for s, n in shares) / max(sum(n for _, n in shares), 1)
    assert other <= OTHER_CHOICES[dtype], f"{dtype}: {other:.2%} of the expert choices differ from the plain router's"
    assert sum(e >= TOL[dtype] for e in errs) <= stray, f"{dtype}: more than {stray} rows beyond {TOL[dtype]}"
    mean = float(np.mean(errs))
    assert mean < TOL_MEAN[dtype], f"{dtype}: mean relative error {mean:.3e} over {len(errs)} rows"
    return max(errs)


def greedy_checked(folder, prompt, got, dtype: str) -> None:
    """``got`` must be the plain implementation's greedy continuation, except where its two best logits are closer
    than the precision tells apart; after such a step the comparison follows the engine's choice."""
    toks = list(prompt)
    tol = 1e-4 if dtype == "float32" else 8e-2
    for step, g in enumerate(got):
        logits = plain_logits(folder, toks)[0][-1]
        best = int(np.argmax(logits))
        if g != best:
            gap = float(logits[best] - logits[g]) / float(np.abs(logits - logits.mean()).max())
            assert gap < tol, f"{dtype}: step {step}: engine chose {g}, plain {best}, relative logit gap {gap:.2e}"
        toks.append(g)
