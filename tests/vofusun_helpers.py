"""Shared by the Vofusun tests: small configurations of their own, model folders from a seed, the plain implementation's
logits and the comparison of a trace's rows with them."""

from __future__ import annotations

import copy
import functools
import json
from pathlib import Path

import numpy as np
import torch

from tests.plain import vofusun_plain as plain


def attention(heads, kv, dim, vdim, window, scale, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale}}


def delta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def attention_2(heads, kv, dim, chunk, scale, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "mask": {"size": chunk}, "scale": scale}
    if rot is not None:
        base, dims, scaling = rot
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            factor, low, high, original = scaling
            m["rot"]["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return {"type": "attention_2", "mlp": mlp, "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


CONFIGS = {
    # every size small and odd (no size is a multiple of 8: every product runs on the 32-bit FMA kernel in both
    # precisions); a window and a chunk shorter than a page; values of another size than keys; three query heads per key
    # head; two delta heads per key head; a layer without a feed-forward inside the loop; part of the head rotated, with
    # all three bands of the frequency scaling in use; the loop opens at layer 1 and runs three times
    "small": {
        "architecture": "Vofusun", "vocab": 61, "width": 36, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
        "layers": [attention(6, 2, 10, 6, 7, 0.4, dense(30)),
                   delta(4, 2, 5, 9, 3),
                   attention_2(3, 1, 12, 11, 0.3, (40.0, 8, (4.0, 1.0, 3.0, 30)), dense(20)),
                   delta(2, 2, 7, 6, 2, dense(12))],
        "loop": {"start": 1, "stop": 3, "times": 3},
    },
    # sizes in multiples of 8 (bfloat16 products on the tcgen05 streaming kernel, attention on the tensor-core kernels at
    # head sizes 64 and 128); one key head for four query heads; a window and a chunk that straddle page borders; the
    # whole head rotated without frequency scaling; no loop
    "wide": {
        "architecture": "Vofusun", "vocab": 96, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
        "layers": [attention_2(4, 1, 64, 24, 0.11, (10000.0, 64, None), dense(256)),
                   delta(2, 1, 32, 64, 4, dense(128)),
                   attention(2, 2, 128, 128, 40, 0.09, dense(64))],
    },
    # keys shorter than values and both padded in the cache (to 64 in bfloat16); no rotation at all; a window of one
    # token (a query sees itself and the sink only) and a chunk of one; one tap (no convolution state); the loop is the
    # whole model and starts at layer 0; the model's last layer has no feed-forward
    "padded": {
        "architecture": "Vofusun", "vocab": 50, "width": 48, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-6},
        "layers": [attention(3, 3, 24, 40, 1, 0.2, dense(40)),
                   attention_2(2, 2, 16, 1, 0.25, None, dense(16)),
                   delta(3, 3, 16, 8, 1, dense(24)),
                   attention(2, 1, 40, 24, 33, 0.15)],
        "loop": {"start": 0, "stop": 4, "times": 2},
    },
    # recurrences only: a model without a page of cache; a loop of one layer at the end; many taps
    "recurrent": {
        "architecture": "Vofusun", "vocab": 40, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
        "layers": [delta(2, 1, 16, 16, 4, dense(48)), delta(4, 4, 24, 4, 7, dense(16))],
        "loop": {"start": 1, "stop": 2, "times": 2},
    },
}


def random_config(rng) -> dict:
    """A configuration drawn at random: two to six layers of the three mixers in any order, odd and even sizes, one to four
    query heads per key head, windows and chunks from one token to more than a prompt, with and without rotation and
    frequency scaling, layers without a feed-forward, and (mostly) a loop somewhere that runs one to three times."""
    width = rng.choice([24, 40, 64, 96, 128])
    def mlp():
        return None if rng.random() < 0.2 else dense(rng.choice([16, 24, 72, 128]))
    def att():
        kv = rng.choice([1, 2, 3]); heads = kv * rng.choice([1, 2, 4])
        return attention(heads, kv, rng.choice([8, 12, 16, 32, 64, 128]), rng.choice([8, 20, 16, 64, 128]), rng.choice([1, 2, 5, 16, 17, 31, 64, 100]), rng.uniform(0.05, 0.4), mlp())
    def dl():
        kv = rng.choice([1, 2, 3]); heads = kv * rng.choice([1, 2, 3])
        return delta(heads, kv, rng.choice([4, 6, 16, 20, 32, 64]), rng.choice([4, 7, 16, 36, 64]), rng.choice([1, 2, 3, 4, 5]), mlp())
    def at2():
        kv = rng.choice([1, 2]); heads = kv * rng.choice([1, 2, 4]); dim = rng.choice([8, 16, 24, 64, 128])
        rot = None
        if rng.random() < 0.8:
            dims = rng.choice([d for d in (2, 4, 8, dim // 2, dim) if d <= dim and d % 2 == 0])
            scaling = None if rng.random() < 0.4 else (rng.choice([2.0, 8.0]), rng.choice([1.0, 2.0]), rng.choice([3.0, 4.0]), rng.choice([16, 64, 8192]))
            rot = (rng.choice([100.0, 10000.0, 500000.0]), dims, scaling)
        return attention_2(heads, kv, dim, rng.choice([1, 3, 8, 16, 20, 33, 64]), rng.uniform(0.05, 0.3), rot, mlp())
    n = rng.randint(2, 6)
    layers = [rng.choice([att, dl, at2])() for _ in range(n)]
    cfg = {"architecture": "Vofusun", "vocab": rng.choice([37, 64, 100]), "width": width, "embedding": {"scale": rng.uniform(0.5, 4.0)},
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.7:
        a = rng.randint(0, n - 1); b = rng.randint(a + 1, n)
        cfg["loop"] = {"start": a, "stop": b, "times": rng.randint(1, 3)}
    return cfg


def config(name: str, **overrides) -> dict:
    c = copy.deepcopy(CONFIGS[name])
    c.update(overrides)
    return c


def make_dir(path, name: str, seed: int, **overrides):
    from jax_llm_examples_b200 import write_random_model

    return write_random_model(path, config(name, **overrides), seed, norm_noise=0.1, std=0.15)


@functools.lru_cache(maxsize=32)
def plain_model(folder: str):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain.read_safetensors(folder / "model.safetensors")


def plain_logits(folder, tokens):
    cfg, P = plain_model(str(folder))
    with torch.no_grad():
        logits, _ = plain.forward(cfg, P, list(tokens))
    return logits.numpy()


# float32: a few thousand roundings of 6e-8 per logit.  bfloat16: activations are rounded (4e-3) several times per layer,
# and a tiny model's logits are sums of few terms, so single rows scatter: the mean over all rows is held tight and a
# single row is capped where a fault (a lost state, a key off by one, a sink left out) would still stand out by far.
TOL = {"float32": 3e-5, "bfloat16": 1.2e-1}
TOL_MEAN = {"float32": 1e-5, "bfloat16": 3e-2}


def row_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Difference of two logit rows, each with its mean taken off, relative to the reference row's spread."""
    d = (got - got.mean()) - (ref - ref.mean())
    return float(np.sqrt((d ** 2).mean()) / max(np.sqrt(((ref - ref.mean()) ** 2).mean()), 1e-9))


def compare(folder, requests: dict, got: dict, dtype: str, stray: int = 0) -> float:
    """Every logit row a trace produced against the plain implementation's row at that place.  Among hundreds of rows
    `stray` of them may scatter past the cap for a single row, up to twice as far; the mean stays as tight."""
    errs = []
    for rid, toks in requests.items():
        ref = plain_logits(folder, toks)
        for pos in range(len(toks)):
            if (rid, pos) in got:
                err = row_err(got[(rid, pos)], ref[pos])
                assert err < TOL[dtype] * (2 if stray else 1), f"{dtype}: request {rid} position {pos}: relative error {err:.3e}"
                errs.append(err)
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
        logits = plain_logits(folder, toks)[-1]
        best = int(np.argmax(logits))
        if g != best:
            gap = float(logits[best] - logits[g]) / float(np.abs(logits - logits.mean()).max())
            assert gap < tol, f"{dtype}: step {step}: engine chose {g}, plain {best}, relative logit gap {gap:.2e}"
        toks.append(g)
