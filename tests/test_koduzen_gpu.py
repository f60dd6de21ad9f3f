"""Koduzen on the GPU against the plain implementation: each mechanism alone (kernel or part against the plain function of
the same name), inputs made so that a fault shows (a far token, a window's edge, the sink's share, the distance bias, the
step of the query temperature), then whole models through the engine's step function under every kind of cut, batches
against requests alone, pages and slots that are used again, long decoding, and greedy generation through the scheduler.
All configurations are this file's own (``tests/koduzen_helpers.py``)."""

import json
import math
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests import koduzen_helpers as KH
from tests.plain import koduzen_plain as plain
from tests.test_makisun_gpu import _run_in_cuts
from tests.test_tebivik_gpu import _close, _ctx

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 3e-2)]
F64 = torch.float64


# ------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("S, D, splits", [(1, 36, 1), (2, 200, 3), (3, 30, 2), (4, 1024, 1), (8, 2048, 2)])
def test_streams_are_written_read_and_normed_in_one_pass(S, D, splits):
    """x_t <- sum_s mix[s, t] x_s + write[t] y (y = a sum of partials), u = sum_t read[t] x_t, rms norm of u: against the
    plain sublayer step; then the first call of a step (streams unwritten, all equal to a given row), the plain sum for
    the final norm, and gathered rows that leave the streams alone."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(S * D)
    N, eps = 7, 1e-5
    X = torch.randn(N, S, D, device=DEV)
    y = torch.randn(splits, N, D, device=DEV)
    mix, write, read, gamma = (torch.randn(*s, device=DEV) for s in ((S, S), (S,), (S,), (D,)))
    x = X.reshape(N, S * D).clone()
    out32, total = torch.empty(N, D, device=DEV), torch.empty(N, D, device=DEV)
    K.stream_mix_norm(x, S, y=y, y_splits=splits, mix=mix, write=write, read=read, gamma=gamma, eps=eps, out32=out32, sum_out=total)
    Xd, yd = X.double().cpu().permute(1, 0, 2), y.sum(0).double().cpu()
    new = torch.einsum("sr,std->rtd", mix.double().cpu(), Xd) + write.double().cpu()[:, None, None] * yd[None]
    u = torch.einsum("s,std->td", read.double().cpu(), new)
    _close(x.view(N, S, D).permute(1, 0, 2), new, 5e-6, "streams")
    _close(out32, plain.rms_norm(u, gamma.double().cpu(), eps), 1e-5, "normed read")
    _close(total, new.sum(0), 5e-6, "sum of the streams")
    # the first call: the streams are written from the embedding's rows while they are read
    first = torch.randn(N, D, device=DEV)
    x2 = torch.full((N, S * D), float("nan"), device=DEV)
    out = torch.empty(N, D, device=DEV, dtype=torch.bfloat16)
    K.stream_mix_norm(x2, S, first=first, read=read, gamma=gamma, eps=eps, out=out)
    assert torch.equal(x2.view(N, S, D), first[:, None, :].expand(N, S, D))
    _close(out, plain.rms_norm(read.double().cpu().sum() * first.double().cpu(), gamma.double().cpu(), eps), 1e-2, "first read")
    # the final norm: no read weights, rows gathered, nothing written back
    rows = torch.tensor([5, 0, 5], device=DEV, dtype=torch.int32)
    before = x.clone()
    K.stream_mix_norm(x, S, y=y, y_splits=splits, mix=mix, write=write, gamma=gamma, eps=eps, out32=(o := torch.empty(3, D, device=DEV)), row_index=rows)
    assert torch.equal(x, before)
    Xn = x.view(N, S, D).double().cpu().permute(1, 0, 2)
    again = torch.einsum("sr,std->rtd", mix.double().cpu(), Xn) + write.double().cpu()[:, None, None] * yd[None]
    _close(o, plain.rms_norm(again.sum(0)[rows.cpu().long()], gamma.double().cpu(), eps), 1e-5, "gathered rows")


@pytest.mark.parametrize("limit, alpha, shift", [(0.0, 1.0, 0.0), (0.8, 1.702, 1.0), (3.0, 1.702, 1.0)])
def test_gated_unit_on_partial_sums_and_in_the_products_epilogue(limit, alpha, shift):
    from jax_llm_examples_b200.kernels import api as K
    from jax_llm_examples_b200.parts import DenseSwiGLU, Runtime

    torch.manual_seed(int(limit * 10))
    form = K.glu_form(alpha, limit, shift)

    def ref(g, u):
        if limit > 0:
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        return g * torch.sigmoid(alpha * g) * (u + shift)

    gu = torch.randn(3, 9, 2 * 20, device=DEV) * 2
    out = torch.empty(9, 20, device=DEV)
    K.silu_mul(gu, out, splits=3, glu=form)
    s = gu.sum(0).double().cpu()
    _close(out, ref(s[:, :20], s[:, 20:]), 3e-6, "activation kernel")
    # the part: bfloat16 with the activation in the streaming product's epilogue (F % 16 == 0, few rows), with many rows
    # (library product, then the activation kernel), and float32
    D, F = 64, 96
    wg, wu, wd = torch.randn(F, D) * 0.3, torch.randn(F, D) * 0.3, torch.randn(D, F) * 0.3
    for dtype, rows, tol in ((torch.bfloat16, 5, 2e-2), (torch.bfloat16, 300, 3e-2), (torch.float32, 5, 1e-5)):
        c = lambda t: t.to(dtype).to(DEV)  # noqa: E731
        part = DenseSwiGLU(torch.cat([c(wg), c(wu)]), c(wd), glu=form)
        h = c(torch.randn(rows, D))
        got = H.as_rows_sum(part.forward(_ctx(Runtime(dtype, torch.device(DEV)), [rows], [0]), h))
        hd, g64, u64, d64 = h.double().cpu(), c(wg).double().cpu(), c(wu).double().cpu(), c(wd).double().cpu()
        _close(got, ref(hd @ g64.T, hd @ u64.T) @ d64.T, tol, f"dense part {dtype} {rows}")


@pytest.mark.parametrize("E, k, groups, keep, N, D", [(6, 2, 3, 2, 40, 36), (16, 4, 4, 3, 300, 64), (8, 3, 1, 1, 9, 24), (12, 1, 6, 1, 100, 128),
                                                      (64, 8, 8, 4, 70, 32)])
def test_router_softmax_over_all_with_groups_and_corrections(E, k, groups, keep, N, D):
    """Both router kernels (one token per block; eight tokens per block) against the plain router: the softmax over all
    outputs, the correction on the choice only (negative ones too), the best groups, the normalised weights."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(E + k)
    h, w = torch.randn(N, D, device=DEV), torch.randn(E, D, device=DEV) * 0.4
    corr = (torch.randn(E, device=DEV) * 0.2).contiguous()
    P = {"m.router": w.double().cpu(), "m.correction": corr.double().cpu()}
    r = {"top": k, "scale": 1.7}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    chosen, weights = plain.route(h.double().cpu(), P, "m.", r)
    for many in (False, True):
        idx, wt = torch.empty(N, k, device=DEV, dtype=torch.int32), torch.empty(N, k, device=DEV)
        K.router(h, w, idx, wt, many_rows=many, weight_form="softmax_normalized", correction=corr, groups=groups, keep=keep, scale=1.7)
        same = (torch.sort(idx.cpu().long(), 1).values == torch.sort(chosen, 1).values).all(1)
        assert same.float().mean() > 0.98, f"many_rows={many}: {(~same).sum()} of {N} tokens chose other experts"
        order = torch.argsort(idx.cpu().long(), 1)
        ref_order = torch.argsort(chosen, 1)
        got_w, ref_w = torch.gather(wt.cpu().double(), 1, order), torch.gather(weights, 1, ref_order)
        assert float((got_w[same] - ref_w[same]).abs().max()) < 1e-5
        assert torch.allclose(wt.sum(1).cpu(), torch.full((N,), 1.7), atol=1e-5)


def _expert_part(P, ml, dtype):
    from jax_llm_examples_b200.kernels import api as K
    from jax_llm_examples_b200.parts import DenseSwiGLU, GroupLimitedGLUExperts

    c = lambda t: t.to(dtype).to(DEV)  # noqa: E731
    r = ml["router"]
    E = r["experts"]
    gu = torch.stack([torch.cat([P[f"m.e{e}.gate"], P[f"m.e{e}.up"]]) for e in range(E)])
    down = torch.stack([P[f"m.e{e}.down"] for e in range(E)])
    shared = None
    if ml.get("shared"):
        shared = DenseSwiGLU(c(torch.cat([P["m.shared.gate"], P["m.shared.up"]])), c(P["m.shared.down"]), glu=K.glu_form(1.702, ml["shared"]["limit"], 1.0))
    g = r.get("groups") or {"count": 1, "keep": 1}
    return GroupLimitedGLUExperts(c(P["m.router"]), c(P["m.correction"]), c(gu), c(down), r["top"], r.get("identity", 0), g["count"], g["keep"],
                                  r.get("scale", 1.0), K.glu_form(1.702, ml["expert"]["limit"], 1.0), shared)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("ml, D, N", [
    (KH.moe(5, 2, 14, 1, (3, 2), 1.5, 0.7, (10, 1.2)), 36, 50),   # odd sizes, an identity expert, groups, a shared expert
    (KH.moe(6, 3, 64, 2, (4, 2), 2.0, 1.0, (32, 1.0)), 128, 20),  # sizes of the streaming kernel, few rows
    (KH.moe(6, 3, 64, 2, (4, 2), 2.0, 1.0, (32, 1.0)), 128, 400),  # ... and many
    (KH.moe(3, 1, 16), 48, 33),                                    # top-1, nothing else
    (KH.moe(2, 4, 16, 6, None, 0.5), 64, 64),                      # more identity experts than real ones
])
def test_expert_part_with_identity_experts_against_the_plain_mixture(name, dtype, tol, ml, D, N):
    from jax_llm_examples_b200.parts import Runtime

    torch.manual_seed(D + N)
    r = ml["router"]
    E, total, F = r["experts"], r["experts"] + r.get("identity", 0), ml["expert"]["ff"]
    g = lambda *s: (torch.randn(*s) * 0.3).to(dtype).float()  # noqa: E731
    P = {"m.router": g(total, D), "m.correction": g(total) * 0.3}
    for e in range(E):
        P[f"m.e{e}.gate"], P[f"m.e{e}.up"], P[f"m.e{e}.down"] = g(F, D), g(F, D), g(D, F)
    if ml.get("shared"):
        Fs = ml["shared"]["ff"]
        P["m.shared.gate"], P["m.shared.up"], P["m.shared.down"] = g(Fs, D), g(Fs, D), g(D, Fs)
    part = _expert_part(P, ml, dtype)
    h32 = torch.randn(N, D, device=DEV)
    ctx = _ctx(Runtime(dtype, torch.device(DEV)), [N], [0])
    ctx.scratch["record_routing"] = []
    got = H.as_rows_sum(part.forward(ctx, h32.to(dtype), h32))
    assert int(ctx.status) == 0
    used = ctx.scratch["record_routing"][0].cpu().long()
    P64 = {k: v.double() for k, v in P.items()}
    # the experts see the rounded rows, the router and the identity experts the unrounded ones: two plain passes
    hr, hu = h32.to(dtype).double().cpu(), h32.double().cpu()
    s = torch.softmax(hu @ P64["m.router"].T, -1)
    w = torch.gather(s, 1, used)
    w = w / (w.sum(1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    ref = torch.zeros(N, D, dtype=F64)
    for t in range(N):
        for c, wt in zip(used[t].tolist(), w[t]):
            ref[t] += wt * (hu[t] if c >= E else plain.clipped_glu(hr[t:t + 1], P64, f"m.e{c}.", ml["expert"]["limit"])[0])
    if ml.get("shared"):
        ref += plain.clipped_glu(hr, P64, "m.shared.", ml["shared"]["limit"])
    _close(got, ref, tol, name)
    own, _ = plain.route(hu, P64, "m.", r)
    same = (torch.sort(used, 1).values == torch.sort(own, 1).values).all(1)
    assert same.float().mean() >= 0.97
    if r.get("identity"):
        assert (used >= E).any(), "no token took an identity expert: the case is not covered"


# --------------------------------------------------------------------------------------- parts alone
def _retention_part(wd, m, eps, dtype):
    from jax_llm_examples_b200.parts import RetentionMixer, rotary_frequencies

    d = lambda k: wd[k].to(DEV)  # noqa: E731
    rot = m.get("rot")
    f = rotary_frequencies(rot["base"], rot["dims"]).to(DEV) if rot else None
    return RetentionMixer(torch.cat([d("q"), d("k"), d("v"), d("g")]), d("o"), torch.tensor(m["decay"], device=DEV), m["heads"], m["dim"], m["vdim"],
                          eps, k_scale=m["dim"] ** -0.5, inv_freq=f, rot_dims=rot["dims"] if rot else 0)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m, D", [
    ({"heads": 4, "dim": 5, "vdim": 9, "decay": [0.9, 0.97, 0.99, 1.0], "rot": {"base": 50.0, "dims": 4}}, 36),
    ({"heads": 1, "dim": 40, "vdim": 64, "decay": [0.98], "rot": {"base": 10000.0, "dims": 40}}, 64),
    ({"heads": 2, "dim": 128, "vdim": 128, "decay": [0.999, 0.9]}, 48),
    ({"heads": 6, "dim": 32, "vdim": 1, "decay": [0.5, 0.7, 0.9, 0.95, 0.99, 1.0], "rot": {"base": 1e6, "dims": 2}}, 24),
])
def test_retention_part_in_portions_token_by_token_and_in_a_batch(name, dtype, tol, m, D):
    """Three sequences of unequal length fed in different cuts as one batch per step (portions, two tokens, single
    tokens), with slots that are not in order: against the plain recurrence per sequence."""
    from jax_llm_examples_b200.parts import LayerCache, Runtime

    torch.manual_seed(m["heads"] * 7 + D)
    eps = 1e-5
    Hh, dk, dv = m["heads"], m["dim"], m["vdim"]
    g = lambda *s: (torch.randn(*s) * 0.3).to(dtype)  # noqa: E731
    wd = {"q": g(Hh * dk, D), "k": g(Hh * dk, D), "v": g(Hh * dv, D), "g": g(Hh * dv, D), "o": g(D, Hh * dv)}
    mixer = _retention_part(wd, m, eps, dtype)
    rt = Runtime(dtype, torch.device(DEV))
    seqs = [torch.randn(n, D).to(dtype) for n in (37, 9, 20)]
    cuts = [[20, 2, 1, 1, 13], [1, 1, 1, 6], [5, 15]]
    state = torch.zeros(5, Hh, dk, dv, device=DEV)
    state[3] = 99.0  # a slot that no sequence uses
    fwd = lambda ctx, rows: H.as_rows_sum(mixer.forward(ctx, rows.to(DEV), LayerCache(None, None, False, state, (state,))))  # noqa: E731
    got = _run_in_cuts(rt, seqs, cuts, [4, 0, 2], fwd, 5)
    for s, o in zip(seqs, got):
        ref = plain.retention_mixer(s.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
        _close(o, ref, tol, name)
    assert torch.equal(state[3], torch.full_like(state[3], 99.0))


def test_retention_keeps_a_far_token_by_its_decay():
    """Made so that a fault shows: token 0 writes a marker along a key that only the last query asks for; the last token's
    own write puts a known amount beside it, so that the per-head norm cannot hide the marker.  With a decay of 1 the
    marker arrives undiminished 700 tokens later (in one prompt, in portions, and through decoded tokens); with 0.999 it
    arrives as 0.999^700 of it."""
    from jax_llm_examples_b200.parts import LayerCache, RetentionMixer, Runtime

    D = dk = dv = 16
    T = 701
    eye = torch.eye(D)
    shift = torch.roll(eye, 4, 0)  # value entry c + 4 = hidden entry c
    gate = torch.zeros(D, D)
    gate[:, 3] = 4.0               # every gate channel = 4 * hidden entry 3
    rt = Runtime(torch.float32, torch.device(DEV))
    hs = torch.zeros(T, D)
    hs[:, 5] = 0.01
    hs[0, 3], hs[0, 5] = 1.0, 0.0                   # token 0: key e3, value e7
    hs[T - 1, 3], hs[T - 1, 4], hs[T - 1, 5] = 1.0, 1.0, 0.0  # the last token: query and key e3 + e4, value e7 + e8
    w_in = torch.cat([eye, eye, shift, gate]).to(DEV)
    for decay in (1.0, 0.999):
        mixer = RetentionMixer(w_in, eye.to(DEV), torch.tensor([decay], device=DEV), 1, dk, dv, 1e-12, k_scale=1.0)
        m = {"heads": 1, "dim": dk, "vdim": dv, "decay": [decay]}
        P = {"m.q": eye.double(), "m.k": eye.double() * dk ** 0.5, "m.v": shift.double(), "m.g": gate.double(), "m.o": eye.double()}
        ref = plain.retention_mixer(hs.double(), P, "m.", m, 1e-12)  # (the plain mixer scales k by dk^-1/2: undone in m.k)
        # before the norm o = (decay^700 + 2) e7 + 2 e8: the marker is the ratio of the two entries
        assert float(ref[-1, 7] / ref[-1, 8]) == pytest.approx((decay ** 700 + 2.0) / 2.0, rel=1e-9)
        for cuts in ([T], [400, 299, 2], [690] + [1] * 11):
            state = torch.zeros(1, 1, dk, dv, device=DEV)
            at, o = 0, None
            for n in cuts:
                ctx = _ctx(rt, [n], [at])
                o = H.as_rows_sum(mixer.forward(ctx, hs[at:at + n].to(DEV), LayerCache(None, None, False, state, (state,))))
                at += n
            assert float(o[-1, 7] / o[-1, 8]) == pytest.approx((decay ** 700 + 2.0) / 2.0, rel=2e-5), f"decay {decay}, cuts {cuts[:3]}"
            _close(o[-1], ref[-1], 2e-5, f"decay {decay}")
            assert float(state[0, 0, 3, 7]) == pytest.approx(decay ** 700 + 1.0, rel=1e-4)


def _normed_part(wd, m, eps, dtype):
    from jax_llm_examples_b200.parts import GatedPagedAttention, rotary_frequencies, yarn_frequencies

    d = lambda k: wd[k].to(DEV)  # noqa: E731
    rot, f, amp = m.get("rot"), None, 1.0
    if rot is not None:
        sc = rot.get("scaling")
        if sc is None:
            f = rotary_frequencies(rot["base"], rot["dims"]).to(DEV)
        else:
            f, amp = yarn_frequencies(rot["base"], rot["dims"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
            f = f.to(DEV)
    return GatedPagedAttention(torch.cat([d("q"), d("k"), d("v")]), d("o"), m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps,
                               q_norm_weight=d("q.norm"), k_norm_weight=d("k.norm"), norm="whole", inv_freq=f, rot_dims=rot["dims"] if rot else 0,
                               rot_amplitude=amp, window=m["mask"]["size"], gate="none",
                               padded_dim=GatedPagedAttention.padded_size(m["dim"], m["vdim"], dtype))


def _biased_part(wd, m, eps, dtype, own=True, keep=None):
    from jax_llm_examples_b200.models.koduzen import distance_slopes
    from jax_llm_examples_b200.parts import GatedPagedAttention

    d = lambda k: wd[k].to(DEV)  # noqa: E731
    qt = m.get("q_temp")
    return GatedPagedAttention(torch.cat([d("q"), d("k"), d("v")]) if own else d("q"), d("o"), m["heads"], m["kv_heads"], m["dim"], m["vdim"],
                               m["scale"], eps, window=m["mask"]["size"], gate="none", sink=d("sink"), slopes=distance_slopes(m["heads"]).to(DEV),
                               query_temperature=(qt["coef"], qt["every"]) if qt else None, projects_kv=own, keep_window=keep,
                               padded_dim=GatedPagedAttention.padded_size(m["dim"], m["vdim"], dtype))


def _attention_in_portions(mixer, rt, hs, dtype, portions, page=16, pages=None, table=None, writes=True):
    from jax_llm_examples_b200.parts import LayerCache

    need = mixer.kv_need()
    if pages is None:
        pages = torch.zeros(40, 2, need.num_kv_heads, page, need.head_dim, device=DEV, dtype=dtype)
        width = (hs.shape[0] + page - 1) // page
        table = torch.randperm(40)[:width].reshape(1, width).to(torch.int32).to(DEV)
    outs = []
    for lo, hi in portions:
        ctx = _ctx(rt, [hi - lo], [lo], planners=mixer.step_planners(), page_size=page)
        outs.append(H.as_rows_sum(mixer.forward(ctx, hs[lo:hi].to(DEV), LayerCache(pages, table, writes, None))))
        assert int(ctx.status) == 0
    return torch.cat(outs), pages, table


PORTIONS = ((0, 21), (21, 43), (43, 45), (45, 46), (46, 47))
LONG_PORTIONS = ((0, 70), (70, 150), (150, 152), (152, 153), (153, 154))


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m, portions", [
    ({"heads": 3, "kv_heads": 1, "dim": 12, "vdim": 7, "mask": {"size": 11}, "scale": 0.3,
      "rot": {"base": 40.0, "dims": 8, "scaling": {"factor": 4.0, "original": 30, "fast": 4.0, "slow": 1.0}}}, PORTIONS),
    ({"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "mask": {"size": 20}, "scale": 0.1, "rot": {"base": 10000.0, "dims": 64}}, PORTIONS),
    ({"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 40, "mask": {"size": 1000}, "scale": 0.2}, PORTIONS),
    ({"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "mask": {"size": 90}, "scale": 0.05,
      "rot": {"base": 500000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 64, "fast": 8.0, "slow": 2.0}}}, LONG_PORTIONS),
    ({"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 32, "mask": {"size": 1}, "scale": 0.05, "rot": {"base": 100.0, "dims": 2}}, PORTIONS),
])
def test_attention_normed_over_the_whole_projection_then_rotated(name, dtype, tol, m, portions):
    """The ``attention`` mixer as a part: ONE norm over all heads of q (and of k) with a weight, the rotate-half rotation
    of part of each head with YaRN frequencies and amplitude, the window; portions that start inside a page, two tokens,
    single tokens; head size 128 on the tcgen05 kernel in bfloat16."""
    from jax_llm_examples_b200.parts import Runtime

    torch.manual_seed(m["heads"])
    D, eps, T = 48, 1e-5, portions[-1][1]
    g = lambda *s: (torch.randn(*s) * 0.3).to(dtype)  # noqa: E731
    Hq, Hkv, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    wd = {"q": g(Hq * dk, D), "k": g(Hkv * dk, D), "v": g(Hkv * dv, D), "o": g(D, Hq * dv),
          "q.norm": (1 + g(Hq * dk)).to(dtype), "k.norm": (1 + g(Hkv * dk)).to(dtype)}
    hs = torch.randn(T, D).to(dtype)
    page = 64 if dk == 128 else 16
    got, _, _ = _attention_in_portions(_normed_part(wd, m, eps, dtype), Runtime(dtype, torch.device(DEV)), hs, dtype, portions, page)
    ref = plain.attention_mixer(hs.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
    _close(got, ref, tol, name)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m, portions", [
    ({"heads": 6, "kv_heads": 2, "dim": 10, "vdim": 6, "mask": {"size": 7}, "scale": 0.4, "q_temp": {"coef": 0.25, "every": 5}}, PORTIONS),
    ({"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "mask": {"size": 20}, "scale": 0.1, "q_temp": {"coef": 0.4, "every": 16}}, PORTIONS),
    ({"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 40, "mask": {"size": 1000}, "scale": 0.2}, PORTIONS),
    ({"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 128, "mask": {"size": 90}, "scale": 0.08, "q_temp": {"coef": 0.3, "every": 64}}, LONG_PORTIONS),
    ({"heads": 2, "kv_heads": 1, "dim": 144, "vdim": 160, "mask": {"size": 30}, "scale": 0.06, "q_temp": {"coef": 1.0, "every": 1}}, PORTIONS),
])
def test_biased_attention_and_a_layer_that_reads_its_keys(name, dtype, tol, m, portions):
    """The ``attention_2`` mixer as a part: a query temperature that steps with the position, a bias per head that grows
    with the distance, a learned sink, the window; then a second part WITHOUT key and value projections reads the pages
    the first one filled, with its own queries, sink, window (longer than the writer's) and temperature."""
    from jax_llm_examples_b200.parts import Runtime

    torch.manual_seed(m["heads"] + 1)
    D, eps, T = 48, 1e-5, portions[-1][1]
    g = lambda *s: (torch.randn(*s) * 0.3).to(dtype)  # noqa: E731
    Hq, Hkv, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    wd = {"q": g(Hq * dk, D), "k": g(Hkv * dk, D), "v": g(Hkv * dv, D), "o": g(D, Hq * dv), "sink": torch.randn(Hq)}
    hs = torch.randn(T, D).to(dtype)
    rt = Runtime(dtype, torch.device(DEV))
    page = 64 if dk == 128 else 16
    P = {"m." + k: v.double() for k, v in wd.items()}
    kv = plain.attention2_keys_values(hs.double(), P, "m.", m)
    got, pages, table = _attention_in_portions(_biased_part(wd, m, eps, dtype), rt, hs, dtype, portions, page)
    _close(got, plain.attention2_mixer(hs.double(), P, "m.", m, kv), tol, name)
    m2 = dict(m, mask={"size": m["mask"]["size"] + 9}, scale=m["scale"] * 0.7, q_temp={"coef": 0.2, "every": 3})
    wd2 = {"q": g(Hq * dk, D), "o": g(D, Hq * dv), "sink": torch.randn(Hq)}
    hs2 = torch.randn(T, D).to(dtype)
    got2, _, _ = _attention_in_portions(_biased_part(wd2, m2, eps, dtype, own=False), rt, hs2, dtype, portions, page, pages, table, writes=False)
    _close(got2, plain.attention2_mixer(hs2.double(), {"m." + k: v.double() for k, v in wd2.items()}, "m.", m2, kv), tol, name + " reader")


def _needle_run(mixer, rt, hs, dtype, qpos, decoded, page):
    from jax_llm_examples_b200.parts import LayerCache

    need = mixer.kv_need()
    pages = torch.zeros(12, 2, 1, page, need.head_dim, device=DEV, dtype=dtype)
    table = torch.randperm(12)[:7].reshape(1, 7).to(torch.int32).to(DEV)
    cuts = [(0, qpos), (qpos, qpos + 1)] if decoded else [(0, qpos + 1)]
    out = ctx = None
    for lo, hi in cuts:
        if hi > lo:
            ctx = _ctx(rt, [hi - lo], [lo], planners=mixer.step_planners(), page_size=page)
            out = H.as_rows_sum(mixer.forward(ctx, hs[lo:hi].to(DEV), LayerCache(pages, table, True, None)))
    return out, ctx


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
@pytest.mark.parametrize("size", [16, 128])  # padded to 64 in bfloat16 (the mma.sync kernels), and the tcgen05 kernel's size
@pytest.mark.parametrize("window", [5, 16, 21, 64, 90, 100])  # 100: the far key is the sequence's first token, 99 back
def test_a_key_just_inside_and_just_outside_the_window(name, dtype, tol, window, size, kind):
    """Made so that a fault shows: q = k = v = the hidden state, and ONE earlier token points where the query points, with
    a score that outweighs everything but the query's own; its value carries a marker.  window - 1 tokens back it shares
    the weight with the query itself; window tokens back it is gone.  In a prompt portion and for a token decoded
    alone; edges at and across page borders; for both windowed mixers (the biased one with its sink and slope)."""
    from jax_llm_examples_b200.models.koduzen import distance_slopes
    from jax_llm_examples_b200.parts import GatedPagedAttention, Runtime

    torch.manual_seed(window)
    D = dk = dv = size
    rt = Runtime(dtype, torch.device(DEV))
    eye = torch.eye(D)
    qkv = torch.cat([eye, eye, eye]).to(dtype).to(DEV)
    pad = GatedPagedAttention.padded_size(dk, dv, dtype)
    if kind == "attention_2":
        mixer = GatedPagedAttention(qkv, eye.to(dtype).to(DEV), 1, 1, dk, dv, 8.0, 1e-6, window=window, gate="none", sink=torch.zeros(1, device=DEV),
                                    slopes=distance_slopes(1).to(DEV), query_temperature=(0.1, 50), padded_dim=pad)
    else:
        ones = torch.ones(D, device=DEV)
        mixer = GatedPagedAttention(qkv, eye.to(dtype).to(DEV), 1, 1, dk, dv, 48.0 / D, 1e-6, q_norm_weight=ones, k_norm_weight=ones, norm="whole",
                                    window=window, gate="none", padded_dim=pad)
    page = 64 if size == 128 else 16
    for qpos, decoded in ((99, False), (99, True), (70, False), (window - 1, False), (window, True)):
        for back, seen in ((window - 1, True), (window, False)):
            if qpos - back < 0 or qpos >= 100 or back == 0:
                continue
            hs = torch.randn(100, D) * 0.05
            direction = torch.zeros(D)
            direction[3] = 4.0
            hs[qpos] = direction
            hs[qpos - back] = direction + torch.nn.functional.one_hot(torch.tensor(8), D).float()
            out, ctx = _needle_run(mixer, rt, hs.to(dtype), dtype, qpos, decoded, page)
            if size == 128 and dtype == torch.bfloat16 and not decoded and qpos >= 63:
                assert any("tc" in kinds for kinds in ctx.scratch.get("attention_kernels", ())), "the tcgen05 kernel did not run"
            marker = float(out[-1, 8])
            assert (marker > 0.12) == seen and (seen or abs(marker) < 0.03), \
                f"{name} {kind} window {window}: query {qpos} ({'decoded' if decoded else 'prompt'}), key {back} back: marker {marker:.3f}"


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("size, heads", [(16, 4), (128, 2)])
def test_sink_slope_and_query_temperature_made_to_show(name, dtype, tol, size, heads):
    """All keys and queries equal (so every score is the same number c * t(p)), values that name their position: the
    weights are then exp(-slope_h * distance) against exp(sink_h - c t(p)), in closed form, per head; the temperature
    t(p) steps at multiples of ``every``.  In a prompt and for tokens decoded alone."""
    from jax_llm_examples_b200.models.koduzen import distance_slopes
    from jax_llm_examples_b200.parts import GatedPagedAttention, Runtime

    T, window, every, coef, scale = 80, 12, 16, 0.5, 0.25
    dk = dv = size
    D = heads * dv  # the hidden width holds every head's output; the first `size` entries feed q, k and v
    rt = Runtime(dtype, torch.device(DEV))
    # q = k = e_0 for every token (hidden entry 0 is 1); v = the hidden state, whose entry 1 + (p mod 8) marks the position
    hs = torch.zeros(T, D)
    hs[:, 0] = 1.0
    for p in range(T):
        hs[p, 1 + p % 8] = 1.0
    wq = torch.zeros(heads * dk, D)
    wk, wv = torch.zeros(dk, D), torch.eye(D)[:dv]
    wk[0, 0] = 2.0
    for a in range(heads):
        wq[a * dk, 0] = 2.0
    sink = torch.tensor([0.5 * (a + 1) for a in range(heads)])
    wo = torch.eye(D)
    mixer = GatedPagedAttention(torch.cat([wq, wk, wv]).to(dtype).to(DEV), wo.to(dtype).to(DEV), heads, 1, dk, dv, scale, 1e-6, window=window,
                                gate="none", sink=sink.to(DEV), slopes=distance_slopes(heads).to(DEV), query_temperature=(coef, every),
                                padded_dim=GatedPagedAttention.padded_size(dk, dv, dtype))
    page = 64 if size == 128 else 16
    for portions in (((0, T),), ((0, 64), (64, 70)) + tuple((p, p + 1) for p in range(70, T))):
        got, _, _ = _attention_in_portions(mixer, rt, hs.to(dtype), dtype, portions, page)
        for p in (0, 14, 15, 16, 31, 32, 47, 48, 63, 64, 70, 79):
            t = 1.0 + coef * math.log(math.floor((p + 1) / every) + 1.0)
            c = 4.0 * scale * t
            for a in range(heads):
                slope = 2.0 ** (-8.0 * (a + 1) / heads)
                js = range(max(0, p - window + 1), p + 1)
                w = {j: math.exp(c - slope * (p - j)) for j in js}
                den = sum(w.values()) + math.exp(float(sink[a]))
                for mark in range(8):
                    want = sum(v for j, v in w.items() if j % 8 == mark) / den
                    assert abs(float(got[p, a * dv + 1 + mark]) - want) < (2e-5 if dtype == torch.float32 else 1.5e-2), \
                        f"{name}: position {p} head {a} mark {mark}: {float(got[p, a * dv + 1 + mark]):.4f} for {want:.4f}"


# --------------------------------------------------------------------------------------- whole models, by traces
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("koduzen")
    return {n: KH.make_dir(root / n, n, seed=i + 1) for i, n in enumerate(KH.CONFIGS)}


def _engine(folder, dtype, max_tokens=512, page_size=16, max_slots=4, **kw):
    import jax_llm_examples_b200 as J

    return J.Engine(J.load_model(folder, dtype, DEV), max_tokens=max_tokens, page_size=page_size, max_slots=max_slots, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(KH.CONFIGS))
def test_every_kind_of_cut_against_the_plain_implementation(folders, name, dtype):
    """Whole prompts; most of a prompt and then 40 tokens one by one; portions down to two tokens; up to four live
    requests mixed, in a pool too small for all of them, so that pages and slots are used again.  Every position's
    logits are compared, the first tokens of a sequence included."""
    vocab = KH.config(name)["vocab"]
    rng = random.Random(7)
    requests = H.random_requests(rng, vocab, [61, 1, 2, 33, 17, 90, 5])
    engine = _engine(folders[name], dtype, max_tokens=16 * 16)
    for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                  H.trace_mixed(requests, rng, max_live=4)):
        got, routing = H.run_trace(engine, steps, record_routing=True)
        assert len(got) == sum(len(t) for t in requests.values())
        KH.compare(folders[name], requests, got, routing, dtype)
        assert engine.manager.free_slots() == 4 and all(engine.manager.free_pages(g) == engine.num_pages for g in range(len(engine.manager.groups)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_size_128_on_pages_of_64_tokens(folders, dtype):
    """Pages of 64 tokens, as a server has them: in bfloat16 the portions of 64 tokens and more of the layers with head
    size 128 run on the tcgen05 kernel (with the distance bias, the sink, the temperature, and a reader of another
    layer's pages), shorter ones on the mma.sync kernel, single tokens on the split-KV kernel, all in one step."""
    name = "wide"
    vocab = KH.config(name)["vocab"]
    rng = random.Random(13)
    requests = H.random_requests(rng, vocab, [200, 70, 131, 3])
    engine = _engine(folders[name], dtype, max_tokens=12 * 64, page_size=64)
    for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=20), H.trace_portions(requests, rng),
                  H.trace_mixed(requests, rng, max_live=4)):
        got, routing = H.run_trace(engine, steps, record_routing=True)
        KH.compare(folders[name], requests, got, routing, dtype, stray=2 if dtype == "bfloat16" else 0)
    if dtype == "bfloat16":
        assert any("tc" in kinds for kinds in engine.attention_kernels_seen), "the tcgen05 kernel did not run"


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5, 7, 8, 9, 10])
def test_configurations_drawn_at_random_under_every_kind_of_cut(seed, tmp_path):
    """Sizes, head counts, orders of layers, windows, rotations, routers and stream counts that nobody chose, in both
    precisions: whole prompts, a decoded tail, portions and mixed batches against the plain implementation.
    (Seed 6 is left out: one of its requests opens with a token whose retention query and key are orthogonal to within
    6e-4 of their lengths.  A sequence's first output is (q . k) v, and the per-head norm divides its size away, so
    that row hangs on the sign of a sum that bfloat16 cannot tell from zero; in float32 the seed passes.)"""
    rng = random.Random(seed)
    cfg = KH.random_config(rng)
    folder = KH.write_model(tmp_path / "m", cfg, seed)
    requests = H.random_requests(rng, cfg["vocab"], [70, 3, 130, 21, 45])
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folder, dtype, max_tokens=20 * 16)
        for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                      H.trace_mixed(requests, rng, max_live=4)):
            got, routing = H.run_trace(engine, steps, record_routing=True)
            KH.compare(folder, requests, got, routing, dtype, stray=4 if dtype == "bfloat16" else 0)


@pytest.mark.parametrize("seed", [1, 4, 9])
def test_mid_size_configurations_on_pages_of_64_tokens(seed, tmp_path):
    """Widths of 192 to 512, head sizes up to 128, dozens of experts, windows of up to 300 tokens, prompts of up to 700
    tokens on pages of 64: whole prompts, a decoded tail, portions and mixed batches against the plain implementation.
    Weights are drawn with a spread of 0.9 / sqrt(width) (what the tiny configurations have at their widths); the
    float32 cap is 1e-4 here: rows are sums of up to 512 terms through up to seven layers."""
    import jax_llm_examples_b200 as J

    rng = random.Random(1000 + seed)
    cfg = KH.mid_size_config(rng)
    folder = J.write_random_model(tmp_path / "m", cfg, seed, norm_noise=0.1, std=0.9 / cfg["width"] ** 0.5)
    requests = H.random_requests(rng, cfg["vocab"], [700, 330, 97, 23, 1, 260])
    saved = dict(KH.TOL), dict(KH.TOL_MEAN)
    KH.TOL["float32"], KH.TOL_MEAN["float32"] = 1e-4, 2e-5
    try:
        for dtype in ("float32", "bfloat16"):
            engine = _engine(folder, dtype, max_tokens=1536, page_size=64, max_seq_len=1536)
            for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                          H.trace_mixed(requests, rng, max_live=4)):
                got, routing = H.run_trace(engine, steps, record_routing=True)
                KH.compare(folder, requests, got, routing, dtype, stray=6 if dtype == "bfloat16" else 0)
    finally:
        KH.TOL.update(saved[0]), KH.TOL_MEAN.update(saved[1])


@pytest.mark.parametrize("name", list(KH.CONFIGS))
def test_logits_do_not_depend_on_the_cut_or_on_the_batch(folders, name):
    """float32: the same request whole, token by token, in portions, and beside three other requests gives the same
    logits to within rounding of a sum's order (far below the tolerance against the plain implementation)."""
    vocab = KH.config(name)["vocab"]
    rng = random.Random(11)
    requests = H.random_requests(rng, vocab, [70, 23, 41, 9])
    engine = _engine(folders[name], "float32")
    whole, _ = H.run_trace(engine, H.trace_whole(requests), record_routing=False)
    for steps in (H.trace_tail_decode(requests, tail=70), H.trace_portions(requests, rng), H.trace_mixed(requests, rng)):
        got, _ = H.run_trace(engine, steps, record_routing=False)
        worst = max(KH.row_err(got[k], whole[k]) for k in whole)
        assert worst < 2e-6, f"{name}: logits moved by {worst:.2e} with the cut"


@pytest.mark.parametrize("name", ["small", "wide", "recurrent"])
def test_decoding_through_replayed_graphs_equals_decoding_without(folders, name):
    """bfloat16: decode-only steps are captured in CUDA graphs and replayed; states and pages are found by slot and table
    on the device, so the replayed steps must give what the same steps give launched one kernel at a time."""
    vocab = KH.config(name)["vocab"]
    rng = random.Random(5)
    requests = H.random_requests(rng, vocab, [50, 37])
    outs = []
    for graphs in (True, False):
        engine = _engine(folders[name], "bfloat16", use_graphs=graphs)
        got, _ = H.run_trace(engine, H.trace_tail_decode(requests, tail=30), record_routing=False)
        assert (engine.graph_replays > 0) == graphs
        outs.append(got)
    worst = max(KH.row_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst < 2e-2, f"{name}: replayed steps differ by {worst:.2e}"


def test_long_decoding_and_slots_used_again(folders):
    """300 tokens one by one after a short prompt, in both precisions: the retention states and the windows' pages (old
    ones are given back on the way, those that a second layer reads only when its longer window has passed) are carried
    over hundreds of steps; then the same slot and pages serve another request, which must not see what the first left."""
    name = "small"
    vocab = KH.config(name)["vocab"]
    rnd = random.Random(3)
    toks = [rnd.randrange(vocab) for _ in range(320)]
    other = [rnd.randrange(vocab) for _ in range(25)]
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folders[name], dtype, max_tokens=320, max_slots=1)
        for req in ({"a": toks}, {"b": other}):
            got, routing = H.run_trace(engine, H.trace_tail_decode(req, tail=300), record_routing=True)
            KH.compare(folders[name], req, got, routing, dtype, stray=3 if dtype == "bfloat16" else 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_portions(folders, dtype):
    """560 tokens in one step beside a short request, and the same in two portions cut inside the windows: against the
    plain implementation at places near the start, around the windows' edges, in the middle and at the end, and
    against each other."""
    import jax_llm_examples_b200 as J

    name = "wide"
    vocab = KH.config(name)["vocab"]
    rng = random.Random(5)
    toks, other = [rng.randrange(vocab) for _ in range(560)], [rng.randrange(vocab) for _ in range(30)]
    want = [0, 1, 2, 23, 24, 25, 39, 40, 41, 255, 256, 299, 300, 311, 312, 511, 512, 558, 559]
    engine = _engine(folders[name], dtype, max_tokens=1024)
    engine.record_routing = True
    a, b = engine.new_request(), engine.new_request()
    whole = engine.step([J.StepEntry(a, toks, want), J.StepEntry(b, other, [29])]).cpu().numpy().copy()
    routed = KH.routed_layers(folders[name])
    forced = {layer: c.cpu()[:560] for layer, c in zip(routed, engine.last_routing)}
    engine.finish(a), engine.finish(b)
    engine.record_routing = False
    a = engine.new_request()
    first = engine.step([J.StepEntry(a, toks[:300], [w for w in want if w < 300])]).cpu().numpy().copy()
    second = engine.step([J.StepEntry(a, toks[300:], [w - 300 for w in want if w >= 300])]).cpu().numpy().copy()
    engine.check_status()
    engine.finish(a)
    parts = np.concatenate([first, second])
    ref, other_choices = KH.plain_logits(folders[name], toks, forced)
    assert other_choices <= KH.OTHER_CHOICES[dtype]
    for k, w in enumerate(want):
        assert KH.row_err(whole[k], ref[w]) < KH.TOL[dtype], f"{dtype}: position {w} of the whole prompt"
        if dtype == "float32":
            assert KH.row_err(parts[k], ref[w]) < KH.TOL[dtype], f"{dtype}: position {w} of the prompt in portions"
            assert KH.row_err(whole[k], parts[k]) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide", "recurrent"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    """The framework's own entry point: prompts of unequal length under a small token budget per step, so that
    prompt portions run beside decoded tokens."""
    import jax_llm_examples_b200 as J

    vocab = KH.config(name)["vocab"]
    prompts = [[(7 * i + 3 * j) % vocab for i in range(n)] for j, n in enumerate((29, 3, 12))]
    model = J.load_model(folders[name], dtype, DEV)
    got = J.generate(model, prompts, J.SamplingParams(max_new_tokens=10), page_size=16, max_tokens_per_step=16)
    for p, g in zip(prompts, got):
        assert len(g) == 10
        KH.greedy_checked(folders[name], p, g, dtype)


def test_command_line_generates_from_a_preset_and_from_a_folder(folders, capsys):
    from jax_llm_examples_b200.main import main

    assert main(["--preset", "koduzen_tiny", "--random-prompts", "2", "--prompt-len", "9", "--max-new-tokens", "4"]) == 0
    assert capsys.readouterr().out.count("-" * 80) == 2
    assert main(["--model", str(folders["recurrent"]), "--dtype", "float32", "--prompt-ids", "1,2,3,4,5", "--max-new-tokens", "5",
                 "--page-size", "16"]) == 0
    ids = [int(t) for t in capsys.readouterr().out.splitlines()[1].split()]
    KH.greedy_checked(folders["recurrent"], [1, 2, 3, 4, 5], ids, "float32")


def test_trace_replay_program_on_a_koduzen_folder(folders, tmp_path):
    """bin/trace_run picks the model class by config.json and writes the wanted logits."""
    name, dtype = "padded", "float32"
    vocab = KH.config(name)["vocab"]
    toks = [(5 * i + 2) % vocab for i in range(21)]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:13], "want": [0, 12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[13:20], "want": []}, {"id": "b", "tokens": toks[:2], "want": [1]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[20:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(H.ROOT, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref, _ = KH.plain_logits(folders[name], toks)
    rows = {0: [0, 12], 1: [1], 2: [20]}
    for step, places in rows.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)
        for g, pl in zip(got, places):
            assert KH.row_err(g, ref[pl]) < KH.TOL[dtype]
