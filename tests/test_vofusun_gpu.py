"""Vofusun on the GPU against the plain implementation: each mechanism alone (kernel or part against the plain
function of the same name), inputs made so that a fault shows (a far token, a key that is written twice, a window's and a
chunk's edge, the sink's share), then whole models through the engine's step function under every kind of cut, batches
against requests alone, pages and slots that are used again, long decoding, and greedy generation through the scheduler.
All configurations are this file's own (``tests/vofusun_helpers.py``)."""

import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests import vofusun_helpers as VH
from tests.plain import vofusun_plain as plain
from tests.test_makisun_gpu import _run_in_cuts
from tests.test_tebivik_gpu import _close, _ctx

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 3e-2)]


def _i32(v):
    return torch.tensor(v, device=DEV, dtype=torch.int32)


# ------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("ahead", [False, True])
@pytest.mark.parametrize("dk, dv, Hh, G", [(1, 1, 1, 1), (9, 5, 2, 2), (16, 8, 4, 2), (33, 70, 2, 1), (128, 128, 2, 2), (200, 40, 3, 1), (256, 33, 2, 2), (300, 36, 1, 1), (512, 8, 2, 1)])
def test_delta_scan_sizes_and_a_batch_of_unequal_requests(dk, dv, Hh, G, ahead):
    """Other sizes (one channel; three warps; more rows than a lane's registers at the smallest build; no multiple of
    anything; several heads on one key head) and three requests of unequal length in one launch, from states that are not
    zero, against the plain recurrence on each alone.  The products between a group's keys and queries are made in the
    scan's blocks or by a launch ahead of it."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(dk)
    lens = [19, 1, 40]
    N = sum(lens)
    q, k = torch.randn(N, G, dk, device=DEV), torch.nn.functional.normalize(torch.randn(N, G, dk, device=DEV), dim=-1)
    v, beta, decay = torch.randn(N, Hh, dv, device=DEV), torch.rand(N, Hh, device=DEV), torch.rand(N, Hh, device=DEV) * 0.5 + 0.5
    slots = [2, 0, 1]
    state = torch.randn(4, Hh, dk, dv, device=DEV) * 0.3
    before = state.clone()
    o = torch.empty(N, Hh, dv, device=DEV)
    extra = (_i32([0] * 19 + [1] + [2] * 40), torch.empty(N * G * 2 * K.DELTA_GROUP, device=DEV)) if ahead else ()
    K.delta_scan(q, k, v, beta, decay, state, _i32([0, 19, 20, 60]), _i32(slots), o, *extra)
    assert torch.equal(state[3], before[3])
    c = lambda t: t.double().cpu()
    at = 0
    for r, n in enumerate(lens):
        sl = slice(at, at + n)
        want, S = plain.delta_recurrence(c(q[sl]), c(k[sl]), c(v[sl]), c(beta[sl]), c(decay[sl]), c(before[slots[r]]))
        _close(o[sl], want, 2e-5, f"request {r}")
        _close(state[slots[r]], S, 2e-5, f"state of request {r}")
        at += n


def test_delta_scan_keeps_a_far_token_and_corrects_a_key_that_is_written_again():
    """Made so that a fault shows.  Head 1 never decays.  Along key direction e0 it is written ONCE with a full step, at
    token 3; 700 tokens later a query along e0 must read that value exactly, through portions of many sizes and a state
    carried across steps.  Along e1 it is written at token 10 and AGAIN at token 600, full steps: the second write must
    replace the first (a rule that only adds outer products would return their sum); a half step at token 650 must land
    half way between.  Along e2 the state of head 0 decays by 1/2 per token: written d tokens ago it reads 2^-d of it,
    and the token's own write is read undecayed."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(0)
    Hh, G, dk, dv, T = 2, 2, 5, 37, 704
    q, k = torch.zeros(T, G, dk, device=DEV), torch.zeros(T, G, dk, device=DEV)
    v = torch.randn(T, Hh, dv, device=DEV)
    beta, decay = torch.zeros(T, Hh, device=DEV), torch.ones(T, Hh, device=DEV)
    e = torch.eye(dk, device=DEV)
    k[3, 1], beta[3, 1] = e[0], 1.0
    q[703, 1] = e[0]
    k[10, 1], beta[10, 1] = e[1], 1.0
    k[600, 1], beta[600, 1] = e[1], 1.0
    q[640, 1] = e[1]
    k[650, 1], beta[650, 1] = e[1], 0.5
    q[651, 1] = e[1]
    decay[:, 0] = 0.5
    k[690, 0], beta[690, 0] = e[2], 1.0
    k[700, 0], beta[700, 0], q[700, 0] = e[2], 0.25, e[2]
    state = torch.zeros(4, Hh, dk, dv, device=DEV)
    state[2] = 99.0  # another request's slot: must stay as it is
    o = torch.empty(T, Hh, dv, device=DEV)
    cuts = [1, 2, 1, 16, 17, 33, 2, 255, 300, 1, 1, 70, 3, 2]
    assert sum(cuts) == T
    at = 0
    for n in cuts:
        sl = slice(at, at + n)
        K.delta_scan(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), beta[sl].contiguous(), decay[sl].contiguous(), state,
                     _i32([0, n]), _i32([1]), o[sl], _i32([0] * n), torch.empty(n * G * 2 * K.DELTA_GROUP, device=DEV))
        at += n
    assert torch.equal(state[2], torch.full_like(state[2], 99.0)) and float(state[0].abs().max()) == 0.0
    _close(o[703, 1], v[3, 1], 1e-6, "the far token")
    _close(o[640, 1], v[600, 1], 1e-6, "the second write replaces the first")
    _close(o[651, 1], 0.5 * v[600, 1] + 0.5 * v[650, 1], 1e-6, "a half step lands half way")
    old = 0.5 ** 10 * v[690, 0]  # what token 700 finds along e2, after its own decay
    _close(o[700, 0], old + 0.25 * (v[700, 0] - old), 1e-6, "a decayed write, corrected by a quarter step and read at once")
    c = lambda t: t.double().cpu()
    want, S = plain.delta_recurrence(c(q), c(k), c(v), c(beta), c(decay))
    _close(o, want, 1e-5, "all tokens")
    _close(state[1], S, 1e-5, "the state at the end")


@pytest.mark.parametrize("taps, G, Hh, dk, dv, splits, front", [
    (1, 1, 2, 8, 4, 1, 2), (2, 2, 2, 5, 9, 2, 2), (4, 1, 3, 32, 16, 1, 2), (7, 3, 3, 24, 4, 3, 2),
    # rows whose length and offset allow 16-byte loads: four taps, more taps than the move keeps in registers, heads of more
    # than 128 channels (a lane's second round, partly filled)
    (4, 2, 4, 32, 16, 2, 4), (7, 1, 2, 24, 8, 3, 4), (3, 2, 2, 256, 132, 1, 8), (1, 1, 2, 8, 4, 1, 4)])
def test_short_convolution_unit_vectors_and_gates_in_portions(taps, G, Hh, dk, dv, splits, front):
    """The kernel in front of the recurrence, fed two requests in portions (shorter than the taps reach, single tokens,
    long ones) beside each other, from split partial sums: convolution over each request's own time axis with its last
    inputs carried as state, silu, unit vectors (q scaled), the step and the decay, against the plain functions on the
    whole sequences.  A slot of neither request is left alone."""
    from jax_llm_examples_b200.kernels import api as K

    from jax_llm_examples_b200.parts import Runtime

    torch.manual_seed(taps)
    rt = Runtime(torch.float32, torch.device(DEV))
    C = 2 * G * dk + Hh * dv
    F = C + Hh * dv + 2 * Hh  # q, k, v, the output gate's columns (not read here), step, decay
    lens = (37, 12)
    proj = [torch.randn(splits, n, F + front, device=DEV) for n in lens]  # the columns in front belong to something else
    conv_w = torch.randn(C, taps, device=DEV) * 0.5
    rate_log, a_bias = torch.randn(Hh, device=DEV) * 0.5, torch.randn(Hh, device=DEV)
    conv_state = torch.zeros(3, max(taps - 1, 1), C, device=DEV)
    conv_state[0] = 55.0  # a slot of neither request: must stay as it is
    cuts = [[20, 2, 1, 3, 1, 1, 9], [1, 1, 2, 5, 3]]
    slots = [2, 1]
    got = [{n: [] for n in "qkvbd"} for _ in lens]
    at = [0, 0]
    for step in range(7):
        live = [r for r in range(2) if step < len(cuts[r])]
        ns = [cuts[r][step] for r in live]
        rows = torch.cat([proj[r][:, at[r]:at[r] + n] for r, n in zip(live, ns)], dim=1).contiguous()
        N = sum(ns)
        qo, ko = torch.empty(N, G, dk, device=DEV), torch.empty(N, G, dk, device=DEV)
        vo, b, d = torch.empty(N, Hh, dv, device=DEV), torch.empty(N, Hh, device=DEV), torch.empty(N, Hh, device=DEV)
        ctx = _ctx(rt, ns, [at[r] for r in live], [slots[r] for r in live])
        K.conv_unit_prep(K.rows_view(rows, splits, front), C + Hh * dv, C + Hh * dv + Hh, conv_w, conv_state if taps > 1 else None, rate_log,
                         a_bias, ctx.cu_q, ctx.q_start, ctx.slot_ids, ctx.req_of_token, ctx.positions, qo, ko, vo, b, d, "silu", 1e-6,
                         dk ** -0.5)
        o = 0
        for r, n in zip(live, ns):
            for name, t in zip("qkvbd", (qo, ko, vo, b, d)):
                got[r][name].append(t[o:o + n])
            o += n
            at[r] += n
    c = lambda t: t.double().cpu()
    for r, n in enumerate(lens):
        s = c(proj[r].sum(0))[:, front:]
        y = plain.causal_conv_silu(s[:, :C], c(conv_w))
        qr = plain.unit_vector(y[:, :G * dk].view(n, G, dk)) * dk ** -0.5
        kr = plain.unit_vector(y[:, G * dk:2 * G * dk].view(n, G, dk))
        vr = y[:, 2 * G * dk:].view(n, Hh, dv)
        sp = torch.nn.functional.softplus(s[:, C + Hh * dv + Hh:C + Hh * dv + 2 * Hh] + c(a_bias))
        for name, ref in (("q", qr), ("k", kr), ("v", vr), ("b", torch.sigmoid(s[:, C + Hh * dv:C + Hh * dv + Hh])),
                          ("d", torch.exp(-torch.exp(c(rate_log)) * sp))):
            _close(torch.cat(got[r][name]), ref, 5e-6, f"request {r}: {name}")
        if taps > 1:
            _close(conv_state[slots[r]], s[n - (taps - 1):, :C], 1e-6, f"request {r}: the last inputs")
    assert torch.equal(conv_state[0], torch.full_like(conv_state[0], 55.0))


# --------------------------------------------------------------------------------------- parts alone
def _window_part(wd, m, eps, dtype):
    from jax_llm_examples_b200.parts import GatedPagedAttention

    d = lambda k: wd[k].to(DEV)
    return GatedPagedAttention(torch.cat([d("q"), d("k"), d("v")]), d("o"), m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps,
                               window=m["mask"]["size"], gate="none", sink=torch.zeros(m["heads"], device=DEV),
                               padded_dim=GatedPagedAttention.padded_size(m["dim"], m["vdim"], dtype))


def _chunk_part(wd, m, eps, dtype):
    from jax_llm_examples_b200.parts import GatedPagedAttention, rotary_frequencies, wavelength_scaled_frequencies

    d = lambda k: wd[k].to(DEV)
    rot, f = m.get("rot"), None
    if rot is not None:
        sc = rot.get("scaling")
        f = (rotary_frequencies(rot["base"], rot["dims"]) if sc is None else
             wavelength_scaled_frequencies(rot["base"], rot["dims"], sc["factor"], sc["low"], sc["high"], sc["original"])).to(DEV)
    return GatedPagedAttention(torch.cat([d("q"), d("k"), d("g")]), d("o"), m["heads"], m["kv_heads"], m["dim"], m["dim"], m["scale"], eps,
                               inv_freq=f, rot_dims=rot["dims"] if rot else 0, pairing="pairs", norm="after", chunk=m["mask"]["size"],
                               values_are_keys=True, gate="channel", sink=torch.zeros(m["heads"], device=DEV),
                               padded_dim=GatedPagedAttention.padded_size(m["dim"], m["dim"], dtype))


def _attention_in_portions(mixer, rt, hs, dtype, portions, page=16):
    from jax_llm_examples_b200.parts import LayerCache

    need = mixer.kv_need()
    pages = torch.zeros(40, 2, need.num_kv_heads, page, need.head_dim, device=DEV, dtype=dtype)
    width = (hs.shape[0] + page - 1) // page
    table = torch.randperm(40)[:width].reshape(1, width).to(torch.int32).to(DEV)
    outs = []
    for lo, hi in portions:
        ctx = _ctx(rt, [hi - lo], [lo], planners=mixer.step_planners(), page_size=page)
        outs.append(H.as_rows_sum(mixer.forward(ctx, hs[lo:hi].to(DEV), LayerCache(pages, table, True, None))))
        assert int(ctx.status) == 0
    return torch.cat(outs)


PORTIONS = ((0, 21), (21, 43), (43, 45), (45, 46), (46, 47))


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 6, "kv_heads": 2, "dim": 10, "vdim": 6, "mask": {"size": 7}, "scale": 0.4},
    {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "mask": {"size": 20}, "scale": 0.1},
    {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 40, "mask": {"size": 1000}, "scale": 0.2},
    {"heads": 3, "kv_heads": 3, "dim": 128, "vdim": 32, "mask": {"size": 1}, "scale": 0.05},
    {"heads": 2, "kv_heads": 1, "dim": 144, "vdim": 160, "mask": {"size": 30}, "scale": 0.06},  # above every tensor-core size
])
def test_window_attention_with_a_sink_over_scattered_pages(name, dtype, tol, m):
    """The ``attention`` mixer as a part: no rotation, no norm, no gate, the sink in every softmax; a prompt portion, one
    that starts inside a page, two tokens, and single tokens; window edges across page borders; values of another size
    than keys in one padded page layout; a window of one token (the query sees itself and the sink)."""
    from jax_llm_examples_b200.parts import Runtime

    torch.manual_seed(m["heads"])
    D, eps, T = 48, 1e-5, 47
    g = lambda *s: torch.randn(*s) * 0.3
    Hq, Hkv, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    wd = {k: v.to(dtype) for k, v in {"q": g(Hq * dk, D), "k": g(Hkv * dk, D), "v": g(Hkv * dv, D), "o": g(D, Hq * dv)}.items()}
    hs = torch.randn(T, D).to(dtype)
    got = _attention_in_portions(_window_part(wd, m, eps, dtype), Runtime(dtype, torch.device(DEV)), hs, dtype, PORTIONS)
    ref = plain.window_attention(hs.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
    _close(got, ref, tol, name)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 3, "kv_heads": 1, "dim": 12, "mask": {"size": 11}, "scale": 0.3,
     "rot": {"base": 40.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 30}}},
    {"heads": 4, "kv_heads": 2, "dim": 64, "mask": {"size": 16}, "scale": 0.11, "rot": {"base": 10000.0, "dims": 64}},
    {"heads": 2, "kv_heads": 2, "dim": 16, "mask": {"size": 1}, "scale": 0.25},
    {"heads": 2, "kv_heads": 1, "dim": 128, "mask": {"size": 1000}, "scale": 0.09,
     "rot": {"base": 5e5, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}},
])
def test_chunk_attention_whose_values_are_its_keys(name, dtype, tol, m):
    """The ``attention_2`` mixer as a part: neighbours rotated as pairs (part of the head, the whole head, or none), every
    band of the frequency scaling, q and k divided by their root mean square AFTER the rotation, the values the keys as
    they were BEFORE both, the chunk's edge inside portions and at their seams, the sink, a gate per output channel."""
    from jax_llm_examples_b200.parts import Runtime

    torch.manual_seed(m["dim"])
    D, eps, T = 40, 1e-5, 47
    g = lambda *s: torch.randn(*s) * 0.3
    Hq, Hkv, dk = m["heads"], m["kv_heads"], m["dim"]
    wd = {k: v.to(dtype) for k, v in {"q": g(Hq * dk, D), "k": g(Hkv * dk, D), "g": g(Hq * dk, D), "o": g(D, Hq * dk)}.items()}
    hs = torch.randn(T, D).to(dtype)
    got = _attention_in_portions(_chunk_part(wd, m, eps, dtype), Runtime(dtype, torch.device(DEV)), hs, dtype, PORTIONS)
    ref = plain.chunk_attention(hs.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
    _close(got, ref, tol, name)


def test_wavelength_scaled_frequencies_in_all_three_bands():
    from jax_llm_examples_b200.parts import rotary_frequencies, wavelength_scaled_frequencies

    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    ref = plain.scaled_frequencies(5e5, 32, sc)
    got = wavelength_scaled_frequencies(5e5, 32, 8.0, 1.0, 4.0, 64).double()
    base = rotary_frequencies(5e5, 32).double()
    kinds = {("kept" if abs(float(r / b) - 1) < 1e-9 else "divided" if abs(float(r / b) - 1 / 8) < 1e-9 else "blend") for r, b in zip(ref, base)}
    assert kinds == {"kept", "divided", "blend"}
    assert float(((got - ref) / ref).abs().max()) < 1e-6


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
@pytest.mark.parametrize("size", [16, 128])  # padded to 64 in bfloat16 (the mma.sync kernels), and the tcgen05 kernel's size
@pytest.mark.parametrize("window", [5, 16, 21, 64])
def test_a_key_just_inside_and_just_outside_the_window_with_a_sink(name, dtype, tol, window, size):
    """Made so that a fault shows: q = k = v = the hidden state, and ONE earlier token points where the query points, with
    a score that outweighs everything (the sink too); its value carries a marker.  window - 1 tokens back it shares the
    weight with the query itself; window tokens back it is gone.  In a prompt portion and for a token decoded alone;
    edges at and across page borders."""
    from jax_llm_examples_b200.parts import GatedPagedAttention, Runtime

    torch.manual_seed(window)
    D = dk = dv = size
    rt = Runtime(dtype, torch.device(DEV))
    eye = torch.eye(D)
    mixer = GatedPagedAttention(torch.cat([eye, eye, eye]).to(dtype).to(DEV), eye.to(dtype).to(DEV), 1, 1, dk, dv, 8.0, 1e-6,
                                window=window, gate="none", sink=torch.zeros(1, device=DEV),
                                padded_dim=GatedPagedAttention.padded_size(dk, dv, dtype))
    page = 64 if size == 128 else 16
    for qpos, decoded in ((99, False), (99, True), (70, False), (window - 1, False), (window, True)):
        for back, seen in ((window - 1, True), (window, False)):
            if qpos - back < 0:
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
            assert (marker > 0.4) == seen and (seen or abs(marker) < 0.05), \
                f"{name} window {window}: query {qpos} ({'decoded' if decoded else 'prompt'}), key {back} back: marker {marker:.3f}"


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("size", [16, 128])
@pytest.mark.parametrize("chunk", [5, 16, 21, 64])
def test_a_key_at_the_chunks_first_place_and_the_one_before_it(name, dtype, tol, chunk, size):
    """Made so that a fault shows: the query and ONE earlier token point the same way, every other token the opposite way
    (after the division by the root mean square their scores are -20 against +20).  At the first place of the query's
    chunk the token takes about a third of the weight, and its value (the key as projected) carries a marker; one place
    earlier it belongs to the chunk before and must be gone, also when that place lies in the same page or portion.
    Chunks count from position 0 although the portion that holds the query starts elsewhere."""
    from jax_llm_examples_b200.parts import GatedPagedAttention, Runtime

    torch.manual_seed(chunk)
    D = dk = size
    rt = Runtime(dtype, torch.device(DEV))
    eye = torch.eye(D)
    w_in = torch.cat([eye, eye, torch.zeros(D, D)]).to(dtype).to(DEV)  # q = k = h; gate logits 0: every channel halved
    f = torch.tensor([0.3], device=DEV)  # entries 0 and 1 turn with the position; the direction and the marker do not
    mixer = GatedPagedAttention(w_in, eye.to(dtype).to(DEV), 1, 1, dk, dk, 20.0 / D, 1e-6, inv_freq=f, rot_dims=2, pairing="pairs",
                                norm="after", chunk=chunk, values_are_keys=True, gate="channel", sink=torch.zeros(1, device=DEV),
                                padded_dim=GatedPagedAttention.padded_size(dk, dk, dtype))
    page = 64 if size == 128 else 16
    for qpos, decoded in ((99, False), (99, True), (70, False), (chunk, True), (chunk, False), (2 * chunk - 1, True), (2 * chunk + 1, False)):
        first = qpos // chunk * chunk
        for at, seen in ((first, True), (first - 1, False)):
            if at < 0 or at >= qpos or qpos >= 100:
                continue
            hs = torch.randn(100, D) * 0.05
            hs[:, 3], hs[:, 8] = -4.0, 0.0  # nobody else carries the marker (the query's own value has nearly all the weight)
            hs[qpos, 3] = 4.0
            hs[at, 3], hs[at, 8] = 4.0, 1.0
            out, _ = _needle_run(mixer, rt, hs.to(dtype), dtype, qpos, decoded, page)
            marker = 2.0 * float(out[-1, 8])
            assert (marker > 0.25) == seen and (seen or abs(marker) < 0.05), \
                f"{name} chunk {chunk}: query {qpos} ({'decoded' if decoded else 'prompt'}), key at {at}: marker {marker:.3f}"


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("kind", ["window", "chunk"])
def test_the_sinks_share_of_the_softmax(name, dtype, tol, kind):
    """A query that sees one key only (itself: a window or a chunk of one token) with score ln 3 keeps 3/4 of the value:
    the sink takes the rest.  Without the sink it would be all of it.  At the first token of a sequence, inside a
    portion, and decoded alone."""
    from jax_llm_examples_b200.parts import GatedPagedAttention, Runtime

    D = 16
    rt = Runtime(dtype, torch.device(DEV))
    eye = torch.eye(D)
    ln3 = float(np.log(3.0))
    if kind == "window":
        mixer = GatedPagedAttention(torch.cat([eye, eye, eye]).to(dtype).to(DEV), eye.to(dtype).to(DEV), 1, 1, D, D, ln3 / 4.0, 1e-6,
                                    window=1, gate="none", sink=torch.zeros(1, device=DEV),
                                    padded_dim=GatedPagedAttention.padded_size(D, D, dtype))
        share = 0.75
    else:  # q and k become unit-rms vectors: q . k = D
        mixer = GatedPagedAttention(torch.cat([eye, eye, torch.zeros(D, D)]).to(dtype).to(DEV), eye.to(dtype).to(DEV), 1, 1, D, D,
                                    ln3 / D, 0.0, norm="after", chunk=1, values_are_keys=True, gate="channel",
                                    sink=torch.zeros(1, device=DEV), padded_dim=GatedPagedAttention.padded_size(D, D, dtype))
        share = 0.75 * 0.5
    hs = torch.zeros(40, D)
    hs[:, 5] = 2.0  # |h|^2 = 4
    hs[:, 9] = torch.arange(40) * 1e-4  # tells the tokens apart; too small to move the score
    got = _attention_in_portions(mixer, rt, hs.to(dtype), dtype, ((0, 1), (1, 30), (30, 32), (32, 33), (33, 40)))
    _close(got[:, 5], torch.full((40,), 2.0 * share), 1e-4 if dtype == torch.float32 else 1e-2, f"{name} {kind}")


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("Hh, G, dk, dv, D, taps", [(4, 2, 5, 9, 36, 3), (1, 1, 40, 64, 64, 4), (2, 2, 128, 128, 48, 2), (6, 2, 33, 1, 24, 1),
                                                    (2, 1, 16, 16, 32, 7)])
def test_gated_delta_rule_part_in_portions_and_token_by_token(name, dtype, tol, Hh, G, dk, dv, D, taps):
    """The ``delta`` mixer as a part: two requests of unequal length side by side, in long portions, portions shorter than
    the convolution reaches, and single tokens; then one request token by token; against the plain mixer on the whole
    sequences.  Slots that belong to no request stay zero."""
    from jax_llm_examples_b200.parts import GatedDeltaRule, LayerCache, Runtime

    torch.manual_seed(Hh * 10 + taps)
    eps = 1e-5
    rt = Runtime(dtype, torch.device(DEV))
    g = lambda *s: torch.randn(*s) * 0.3
    m = {"heads": Hh, "kv_heads": G, "dim": dk, "vdim": dv, "conv": taps}
    w = {"q": g(G * dk, D), "k": g(G * dk, D), "v": g(Hh * dv, D), "g": g(Hh * dv, D), "b": g(Hh, D), "a": g(Hh, D),
         "q.conv": g(G * dk, taps), "k.conv": g(G * dk, taps), "v.conv": g(Hh * dv, taps), "A_log": g(Hh), "dt_bias": g(Hh),
         "norm": 1 + 0.2 * torch.randn(dv), "o": g(D, Hh * dv)}
    wd = {k: v.to(dtype) for k, v in w.items()}
    d = lambda k: wd[k].to(DEV)
    mixer = GatedDeltaRule(torch.cat([d(s) for s in "qkvgba"]), torch.cat([d(s + ".conv") for s in "qkv"]), d("A_log"), d("dt_bias"),
                           d("norm"), d("o"), Hh, G, dk, dv, eps)
    needs = mixer.state_needs()
    assert len(needs) == (2 if taps > 1 else 1) and needs[-1].shape == (Hh, dk, dv) and all(n.dtype == torch.float32 for n in needs)
    seqs = [torch.randn(70, D).to(dtype), torch.randn(13, D).to(dtype)]
    P = {"m." + k: v.double() for k, v in wd.items()}
    ref = [plain.delta_mixer(s.double(), P, "m.", m, eps) for s in seqs]
    states = tuple(torch.zeros(4, *n.shape, device=DEV) for n in needs)

    def fwd(ctx, rows):
        return H.as_rows_sum(mixer.forward(ctx, rows.to(DEV), LayerCache(None, None, True, states[0], states)))

    got = _run_in_cuts(rt, seqs, [[40, 2, 1, 1, 17, 1, 8], [1, 1, 2, 9]], [3, 1], fwd, 7)
    for r in range(2):
        _close(got[r], ref[r], tol, f"{name} request {r}")
    assert all(float(s[0].abs().max()) == 0.0 and float(s[2].abs().max()) == 0.0 for s in states)
    for s in states:
        s.zero_()
    got = _run_in_cuts(rt, seqs[1:], [[1] * 13], [2], fwd, 13)
    _close(got[0], ref[1], tol, f"{name} token by token")


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
def test_a_pass_of_the_loop_opens_with_the_embedding_added_once_more(name, dtype, tol, tmp_path):
    """A looped stretch that starts after layer 0 and one that is the whole model: the residual stream after EVERY layer
    run against the plain implementation's (a pass after the first starts from x + the embedding's output, added once,
    and each run has a cache or state of its own), for a whole prompt and for the same prompt in portions."""
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.parts.base import as_rows

    for cname in ("small", "padded"):
        folder = VH.make_dir(tmp_path / cname, cname, seed=21)
        cfg, P = VH.plain_model(str(folder))
        model = J.load_model(folder, name, DEV)
        runs = plain.layer_order(cfg)
        assert len(model.schedule) == len(runs) + sum(1 for _, opens in runs if opens)
        seen = []

        def watch(block):
            inner = block.forward

            def forward(ctx, x, delta, cache):
                d = inner(ctx, x, delta, cache)
                r = as_rows(d)
                seen.append((x.float() + r.data.float().reshape(r.splits, -1, x.shape[-1]).sum(0)).cpu())
                return d
            block.forward = forward

        for b in model.blocks:
            if b.mixer is not None:
                watch(b)
        engine = J.Engine(model, max_tokens=128, page_size=16, max_slots=2, use_graphs=False)
        toks = [(5 * i + 1) % cfg["vocab"] for i in range(29)]
        with torch.no_grad():
            _, after = plain.forward(cfg, P, toks)
        for cuts in ([(0, 29)], [(0, 9), (9, 11), (11, 12), (12, 29)]):
            a = engine.new_request()
            seen.clear()
            for lo, hi in cuts:
                engine.step([J.StepEntry(a, toks[lo:hi], [hi - lo - 1])])
            engine.finish(a)
            assert len(seen) == len(runs) * len(cuts)
            for run in range(len(runs)):
                got = torch.cat([seen[c * len(runs) + run] for c in range(len(cuts))])
                _close(got, after[run], 4 * tol, f"{name} {cname}: after layer run {run} ({len(cuts)} portions)")


# --------------------------------------------------------------------------------------- whole models, by traces
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("vofusun")
    return {n: VH.make_dir(root / n, n, seed=i + 1) for i, n in enumerate(VH.CONFIGS)}


def _engine(folder, dtype, max_tokens=512, page_size=16, max_slots=4, **kw):
    import jax_llm_examples_b200 as J

    return J.Engine(J.load_model(folder, dtype, DEV), max_tokens=max_tokens, page_size=page_size, max_slots=max_slots, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(VH.CONFIGS))
def test_every_kind_of_cut_against_the_plain_implementation(folders, name, dtype):
    """Whole prompts; most of a prompt and then 40 tokens one by one; portions down to two tokens; up to four live
    requests mixed, in a pool too small for all of them, so that pages and slots are used again.  Every position's
    logits are compared, the first tokens of a sequence included."""
    vocab = VH.config(name)["vocab"]
    rng = random.Random(7)
    requests = H.random_requests(rng, vocab, [61, 1, 2, 33, 17, 90, 5])
    engine = _engine(folders[name], dtype, max_tokens=16 * 16)
    for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                  H.trace_mixed(requests, rng, max_live=4)):
        got, _ = H.run_trace(engine, steps, record_routing=False)
        assert len(got) == sum(len(t) for t in requests.values())
        VH.compare(folders[name], requests, got, dtype)
        assert engine.manager.free_slots() == 4 and all(engine.manager.free_pages(g) == engine.num_pages for g in range(len(engine.manager.groups)))


@pytest.mark.parametrize("seed", [0, 1, 3, 5, 7, 8, 11, 13])
def test_configurations_drawn_at_random_under_every_kind_of_cut(seed, tmp_path):
    """Sizes, head counts, orders of layers, windows, chunks, taps, rotations and loops that nobody chose, in both precisions:
    whole prompts, a decoded tail, portions and mixed batches against the plain implementation."""
    import jax_llm_examples_b200 as J

    rng = random.Random(seed)
    cfg = VH.random_config(rng)
    folder = J.write_random_model(tmp_path / "m", cfg, seed, norm_noise=0.1, std=0.15)
    requests = H.random_requests(rng, cfg["vocab"], [70, 3, 130, 21, 45])
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folder, dtype, max_tokens=20 * 16)
        for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                      H.trace_mixed(requests, rng, max_live=4)):
            got, _ = H.run_trace(engine, steps, record_routing=False)
            VH.compare(folder, requests, got, dtype, stray=4 if dtype == "bfloat16" else 0)


@pytest.mark.parametrize("name", list(VH.CONFIGS))
def test_logits_do_not_depend_on_the_cut_or_on_the_batch(folders, name):
    """float32: the same request whole, token by token, in portions, and beside three other requests gives the same
    logits to within rounding of a sum's order (far below the tolerance against the plain implementation)."""
    vocab = VH.config(name)["vocab"]
    rng = random.Random(11)
    requests = H.random_requests(rng, vocab, [70, 23, 41, 9])
    engine = _engine(folders[name], "float32")
    whole, _ = H.run_trace(engine, H.trace_whole(requests), record_routing=False)
    for steps in (H.trace_tail_decode(requests, tail=70), H.trace_portions(requests, rng), H.trace_mixed(requests, rng)):
        got, _ = H.run_trace(engine, steps, record_routing=False)
        worst = max(VH.row_err(got[k], whole[k]) for k in whole)
        assert worst < 2e-6, f"{name}: logits moved by {worst:.2e} with the cut"


@pytest.mark.parametrize("name", ["small", "wide", "recurrent"])
def test_decoding_through_replayed_graphs_equals_decoding_without(folders, name):
    """bfloat16: decode-only steps are captured in CUDA graphs and replayed; states and pages are found by slot and table
    on the device, so the replayed steps must give what the same steps give launched one kernel at a time."""
    vocab = VH.config(name)["vocab"]
    rng = random.Random(5)
    requests = H.random_requests(rng, vocab, [50, 37])
    outs = []
    for graphs in (True, False):
        engine = _engine(folders[name], "bfloat16", use_graphs=graphs)
        got, _ = H.run_trace(engine, H.trace_tail_decode(requests, tail=30), record_routing=False)
        assert (engine.graph_replays > 0) == graphs
        outs.append(got)
    worst = max(VH.row_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst < (1e-6 if name == "recurrent" else 2e-2), f"{name}: replayed steps differ by {worst:.2e}"


def test_long_decoding_and_slots_used_again(folders):
    """300 tokens one by one after a short prompt, in both precisions: the delta rule's states, the window's pages (old
    ones are given back on the way) and the chunk's pages (a chunk's pages are given back when the next one opens) are
    carried over hundreds of steps and many windows and chunks; then the same slot and pages serve another request,
    which must not see what the first left."""
    name = "small"
    vocab = VH.config(name)["vocab"]
    rnd = random.Random(3)
    toks = [rnd.randrange(vocab) for _ in range(320)]
    other = [rnd.randrange(vocab) for _ in range(25)]
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folders[name], dtype, max_tokens=320, max_slots=1)
        for req in ({"a": toks}, {"b": other}):
            got, _ = H.run_trace(engine, H.trace_tail_decode(req, tail=300), record_routing=False)
            VH.compare(folders[name], req, got, dtype, stray=3 if dtype == "bfloat16" else 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_portions(folders, dtype):
    """560 tokens in one step beside a short request, and the same in two portions cut inside a window and a chunk:
    against the plain implementation at places near the start, around the window's and the chunk's edges, in the
    middle and at the end, and against each other."""
    import jax_llm_examples_b200 as J

    name = "wide"
    vocab = VH.config(name)["vocab"]
    rng = random.Random(5)
    toks, other = [rng.randrange(vocab) for _ in range(560)], [rng.randrange(vocab) for _ in range(30)]
    want = [0, 1, 2, 23, 24, 25, 39, 40, 41, 255, 256, 299, 300, 311, 312, 511, 512, 558, 559]
    engine = _engine(folders[name], dtype, max_tokens=1024)
    a, b = engine.new_request(), engine.new_request()
    whole = engine.step([J.StepEntry(a, toks, want), J.StepEntry(b, other, [29])]).cpu().numpy().copy()
    engine.finish(a), engine.finish(b)
    a = engine.new_request()
    first = engine.step([J.StepEntry(a, toks[:300], [w for w in want if w < 300])]).cpu().numpy().copy()
    second = engine.step([J.StepEntry(a, toks[300:], [w - 300 for w in want if w >= 300])]).cpu().numpy().copy()
    engine.check_status()
    engine.finish(a)
    parts = np.concatenate([first, second])
    ref = VH.plain_logits(folders[name], toks)
    for k, w in enumerate(want):
        assert VH.row_err(whole[k], ref[w]) < VH.TOL[dtype], f"{dtype}: position {w} of the whole prompt"
        assert VH.row_err(parts[k], ref[w]) < VH.TOL[dtype], f"{dtype}: position {w} of the prompt in portions"
        if dtype == "float32":
            assert VH.row_err(whole[k], parts[k]) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide", "recurrent"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    """The framework's own entry point: prompts of unequal length under a small token budget per step, so that
    prompt portions run beside decoded tokens."""
    import jax_llm_examples_b200 as J

    vocab = VH.config(name)["vocab"]
    prompts = [[(7 * i + 3 * j) % vocab for i in range(n)] for j, n in enumerate((29, 3, 12))]
    model = J.load_model(folders[name], dtype, DEV)
    got = J.generate(model, prompts, J.SamplingParams(max_new_tokens=10), page_size=16, max_tokens_per_step=16)
    for p, g in zip(prompts, got):
        assert len(g) == 10
        VH.greedy_checked(folders[name], p, g, dtype)


def test_command_line_generates_from_a_preset_and_from_a_folder(folders, capsys):
    from jax_llm_examples_b200.main import main

    assert main(["--preset", "vofusun_tiny", "--random-prompts", "2", "--prompt-len", "9", "--max-new-tokens", "4"]) == 0
    assert capsys.readouterr().out.count("-" * 80) == 2
    assert main(["--model", str(folders["recurrent"]), "--dtype", "float32", "--prompt-ids", "1,2,3,4,5", "--max-new-tokens", "5",
                 "--page-size", "16"]) == 0
    ids = [int(t) for t in capsys.readouterr().out.splitlines()[1].split()]
    VH.greedy_checked(folders["recurrent"], [1, 2, 3, 4, 5], ids, "float32")


def test_trace_replay_program_on_a_vofusun_folder(folders, tmp_path):
    """bin/trace_run picks the model class by config.json and writes the wanted logits."""
    name, dtype = "padded", "float32"
    vocab = VH.config(name)["vocab"]
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
    ref = VH.plain_logits(folders[name], toks)
    rows = {0: [0, 12], 1: [1], 2: [20]}
    for step, places in rows.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)
        for g, pl in zip(got, places):
            assert VH.row_err(g, ref[pl]) < VH.TOL[dtype]
