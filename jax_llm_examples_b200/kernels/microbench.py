"""Microbenchmarks of single kernels at model sizes, with the bytes and FLOPs they must move.

    python -m jax_llm_examples_b200.kernels.microbench attention_decode --batch 8 --context 8192
    python -m jax_llm_examples_b200.kernels.microbench attention_prefill --tokens 2048
    python -m jax_llm_examples_b200.kernels.microbench gemm --rows 8 --n 16384 --k 5120 [--experts 16] [--swiglu]
    python -m jax_llm_examples_b200.kernels.microbench decay_scan --tokens 2048 --requests 1 --heads 16 [--read-before]
    python -m jax_llm_examples_b200.kernels.microbench delta_scan --tokens 2048 --requests 1 --heads 16 [--key-heads 8]

The reference benchmarks its kernels the same way, from ``__main__`` blocks in the kernel files
(llama4/llama4_jax/ragged_attention.py:299-418, llama4/llama4_jax/decode_ragged_dot.py:239-291).
Timing: CUDA events around one launch, after warm-up, with a write larger than L2 between launches;
the median of the repetitions is reported.  Sizes default to the Scout layer sizes.
"""

from __future__ import annotations

import argparse
import json
import random

import torch

from . import api as K


def _time(fn, reps: int, flush: torch.Tensor | None) -> float:
    for _ in range(3):
        fn()
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return sorted(times)[len(times) // 2] * 1e-3


def _paged(batch: int, context: int, hkv: int, dh: int, page: int, dev: str):
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    pages = (torch.randn(n_pages, 2, hkv, page, dh, device=dev) * 0.5).bfloat16()
    table = torch.arange(n_pages, device=dev, dtype=torch.int32).view(batch, pages_per).contiguous()
    return pages, table


def attention_decode(a) -> dict:
    dev = "cuda"
    pages, table = _paged(a.batch, a.context, a.kv_heads, a.head_dim, a.page_size, dev)
    q = torch.randn(a.batch, a.heads, a.head_dim, device=dev).bfloat16()
    out = torch.empty_like(q)
    pos = torch.full((a.batch,), a.context - 1, device=dev, dtype=torch.int32)
    req = torch.arange(a.batch, device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    keys, splits = K.attention_decode_plan(a.context, a.chunk, 0, a.batch * a.kv_heads)
    if a.split_keys:
        keys, splits = a.split_keys, -(-a.context // a.split_keys) + 1
    part_o = torch.empty(a.batch * a.heads * splits * a.head_dim, device=dev)
    part_ml = torch.empty(a.batch * a.heads * splits * 2, device=dev)

    def run():
        K.attention_decode(q, pages, table, req, pos, out, a.head_dim ** -0.5, a.chunk, 0, 0.0, 1.0, part_o, part_ml, splits,
                           keys, status)

    t = _time(run, a.reps, _flush(a))
    nbytes = a.batch * a.context * 2 * a.kv_heads * a.head_dim * 2
    assert int(status) == 0
    return {"kernel": "attention_decode", "batch": a.batch, "context": a.context, "split_keys": keys, "splits": splits,
            "us": round(t * 1e6, 1), "GB": round(nbytes / 1e9, 3), "GB/s": round(nbytes / t / 1e9, 1)}


def attention_prefill(a) -> dict:
    dev = "cuda"
    T = a.tokens
    pages, table = _paged(1, T, a.kv_heads, a.head_dim, a.page_size, dev)
    q = torch.randn(T, a.heads, a.head_dim, device=dev).bfloat16()
    out = torch.empty_like(q)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    req = torch.zeros(T, device=dev, dtype=torch.int32)
    rows = 128 if a.tc else 16
    tiles = torch.tensor([(t, min(rows, T - t)) for t in range(0, T, rows)][::-1], device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    fn = K.attention_prefill_tc if a.tc else K.attention_prefill

    def run():
        fn(q, pages, table, req, pos, out, tiles, tiles.shape[0], a.head_dim ** -0.5, a.chunk, 0, 0.0, 1.0, status)

    t = _time(run, a.reps, _flush(a))
    flops = 4 * a.heads * a.head_dim * T * (T + 1) / 2
    assert int(status) == 0
    return {"kernel": "attention_prefill_tc" if a.tc else "attention_prefill", "tokens": T, "us": round(t * 1e6, 1), "TFLOP": round(flops / 1e12, 4),
            "TFLOP/s": round(flops / t / 1e12, 1)}


def gemm(a) -> dict:
    dev = "cuda"
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    x = torch.randn(a.rows, a.k, device=dev).bfloat16()
    E = a.experts
    w = (torch.randn(max(E, 1), a.n, a.k, device=dev) * 0.05).bfloat16()
    offsets, used, tiles = None, 1, None
    hint = a.hint or (min(a.rows, 2 * -(-a.rows // E)) if E else 0)
    if E:
        # rows spread over the groups at random; the sort kernel gives the offsets and, as in the engine, the
        # list of row tiles that hold rows
        rng = random.Random(0)
        choice = torch.tensor([rng.randrange(E) for _ in range(a.rows)], device=dev, dtype=torch.int32).view(-1, 1)
        offsets = torch.empty(E + 1, device=dev, dtype=torch.int32)
        pair, pos = torch.empty(a.rows, device=dev, dtype=torch.int32), torch.empty(a.rows, device=dev, dtype=torch.int32)
        tile_rows = K.gemm_stream_token_tile(hint)
        tiles = (torch.empty(2 * (-(-a.rows // tile_rows) + E), device=dev, dtype=torch.int32), torch.empty(1, device=dev, dtype=torch.int32))
        K.expert_sort(choice, offsets, pair, pos, E, status, 0, tile_rows, *tiles)
        used = int((offsets[1:] > offsets[:-1]).sum())
    else:
        w = w[0]
    mode = K.GEMM_SWIGLU if a.swiglu else K.GEMM_PLAIN
    out = torch.empty(a.rows, a.n // 2 if a.swiglu else a.n, device=dev, dtype=torch.bfloat16 if a.swiglu else torch.float32)
    scratch = torch.empty(a.splits * a.rows * a.n, device=dev) if a.splits > 1 else None

    def run():
        K.gemm_stream(x, w, out, status, offsets=offsets, rows_hint=hint, splits=a.splits, scratch=scratch, mode=mode, tiles=tiles)

    t = _time(run, a.reps, _flush(a))
    nbytes = used * a.n * a.k * 2 + a.rows * a.k * 2 + out.numel() * out.element_size()
    flops = 2 * a.rows * a.n * a.k
    assert int(status) == 0
    return {"kernel": "gemm_stream", "rows": a.rows, "n": a.n, "k": a.k, "experts": E, "experts_used": used if E else None,
            "splits": a.splits, "swiglu": a.swiglu, "us": round(t * 1e6, 1), "GB/s": round(nbytes / t / 1e9, 1),
            "TFLOP/s": round(flops / t / 1e12, 1)}


def decay_scan(a) -> dict:
    """The decayed linear-attention recurrence: ``requests`` requests of ``tokens`` tokens each in one launch."""
    dev = "cuda"
    N, H, dk, dv = a.requests * a.tokens, a.heads, a.dim, a.vdim
    q, k = torch.randn(N, H, dk, device=dev), torch.randn(N, H, dk, device=dev) * dk ** -0.5
    d, v = torch.rand(N, H, dk, device=dev) * 0.5 + 0.5, torch.randn(N, H, dv, device=dev)
    bonus = torch.randn(H, dk, device=dev) if a.read_before else None
    state, o = torch.zeros(a.requests, H, dk, dv, device=dev), torch.empty(N, H, dv, device=dev)
    cu = (torch.arange(a.requests + 1, device=dev, dtype=torch.int32) * a.tokens).contiguous()
    slots = torch.arange(a.requests, device=dev, dtype=torch.int32)

    def run():
        K.decay_scan(q, k, d, v, bonus, state, cu, slots, o, not a.read_before)

    t = _time(run, a.reps, _flush(a))
    rows, states = N * H * (3 * dk + 2 * dv) * 4, a.requests * H * dk * dv * 8
    return {"kernel": "decay_scan", "requests": a.requests, "tokens": a.tokens, "heads": H, "dim": dk, "vdim": dv,
            "read": "before the update, with a bonus" if a.read_before else "after the update", "us": round(t * 1e6, 1),
            "ns_per_token": round(t * 1e9 / a.tokens, 1), "bytes": rows + states, "GB/s": round((rows + states) / t / 1e9, 1),
            "GFLOP/s": round(N * H * dk * dv * 5 / t / 1e9, 1)}


def delta_scan(a) -> dict:
    """The gated delta rule's recurrence: ``requests`` requests of ``tokens`` tokens each in one launch."""
    dev = "cuda"
    N, H, G, dk, dv = a.requests * a.tokens, a.heads, a.key_heads or a.heads, a.dim, a.vdim
    q = torch.nn.functional.normalize(torch.randn(N, G, dk, device=dev), dim=-1) * dk ** -0.5
    k, v = torch.nn.functional.normalize(torch.randn(N, G, dk, device=dev), dim=-1), torch.randn(N, H, dv, device=dev)
    beta, decay = torch.rand(N, H, device=dev), torch.rand(N, H, device=dev) * 0.1 + 0.9
    state, o = torch.zeros(a.requests, H, dk, dv, device=dev), torch.empty(N, H, dv, device=dev)
    cu = (torch.arange(a.requests + 1, device=dev, dtype=torch.int32) * a.tokens).contiguous()
    slots = torch.arange(a.requests, device=dev, dtype=torch.int32)
    req = torch.arange(a.requests, device=dev, dtype=torch.int32).repeat_interleave(a.tokens).contiguous()
    scratch = None if a.products_in_block else torch.empty(N * G * 2 * K.DELTA_GROUP, device=dev)

    def run():
        K.delta_scan(q, k, v, beta, decay, state, cu, slots, o, req, scratch)

    t = _time(run, a.reps, _flush(a))
    rows, states = N * (2 * G * dk + 2 * H * dv + 2 * H) * 4, a.requests * H * dk * dv * 8
    return {"kernel": "delta_scan", "requests": a.requests, "tokens": a.tokens, "heads": H, "key_heads": G, "dim": dk, "vdim": dv,
            "us": round(t * 1e6, 1), "ns_per_token": round(t * 1e9 / a.tokens, 1), "bytes": rows + states,
            "GB/s": round((rows + states) / t / 1e9, 1), "GFLOP/s": round(N * H * dk * dv * 7 / t / 1e9, 1)}


def conv_unit_prep(a) -> dict:
    """The kernel in front of the delta rule's recurrence: ``requests`` requests of ``tokens`` tokens each in one launch."""
    dev = "cuda"
    N, H, G, dk, dv, taps = a.requests * a.tokens, a.heads, a.key_heads or a.heads, a.dim, a.vdim, a.taps
    C = 2 * G * dk + H * dv
    F = C + H * dv + 2 * H
    proj = torch.randn(1, N, F, device=dev)
    conv_w = torch.randn(C, taps, device=dev) * 0.5
    conv_state = torch.zeros(a.requests, max(taps - 1, 1), C, device=dev)
    rate_log, a_bias = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
    cu = (torch.arange(a.requests + 1, device=dev, dtype=torch.int32) * a.tokens).contiguous()
    slots = torch.arange(a.requests, device=dev, dtype=torch.int32)
    req = slots.repeat_interleave(a.tokens).contiguous()
    start = torch.full((a.requests,), 100, device=dev, dtype=torch.int32)
    pos = (torch.arange(a.tokens, device=dev, dtype=torch.int32).repeat(a.requests) + 100).contiguous()
    qo, ko = torch.empty(N, G, dk, device=dev), torch.empty(N, G, dk, device=dev)
    vo, beta, decay = torch.empty(N, H, dv, device=dev), torch.empty(N, H, device=dev), torch.empty(N, H, device=dev)

    def run():
        K.conv_unit_prep(K.rows_view(proj, 1, 0), C + H * dv, C + H * dv + H, conv_w, conv_state if taps > 1 else None, rate_log, a_bias,
                         cu, start, slots, req, pos, qo, ko, vo, beta, decay, "silu", 1e-6, dk ** -0.5)

    t = _time(run, a.reps, _flush(a))
    moved = N * (2 * C + 4 * H) * 4
    return {"kernel": "conv_unit_prep", "requests": a.requests, "tokens": a.tokens, "heads": H, "key_heads": G, "dim": dk, "vdim": dv,
            "taps": taps, "us": round(t * 1e6, 1), "bytes": moved, "GB/s": round(moved / t / 1e9, 1)}


def stream_mix_norm(a) -> dict:
    """The kernel between two sublayers of a model with several residual rows per token: write-back with mixing, the next
    read and its norm, for ``tokens`` rows of ``streams`` x ``width``."""
    from . import api as K

    N, S, D = a.tokens, a.streams, a.width
    x = torch.randn(N, S * D, device="cuda")
    y = torch.randn(a.splits, N, D, device="cuda")
    mix, write, read, gamma = torch.randn(S, S, device="cuda"), torch.randn(S, device="cuda"), torch.randn(S, device="cuda"), torch.randn(D, device="cuda")
    out = torch.empty(N, D, device="cuda", dtype=torch.bfloat16)
    t = _time(lambda: K.stream_mix_norm(x, S, y=y, y_splits=a.splits, mix=mix, write=write, read=read, gamma=gamma, eps=1e-6, out=out),
              a.reps, _flush(a))
    moved = N * D * (8 * S + 4 * a.splits + 2)  # the rows read and written, the partials read, the normed row written
    return {"kernel": "stream_mix_norm", "tokens": N, "streams": S, "width": D, "splits": a.splits, "us": round(t * 1e6, 1), "bytes": moved,
            "GB/s": round(moved / t / 1e9, 1)}


def _flush(a):
    return None if a.no_flush else torch.empty(256 * 1024 * 1024 // 4, device="cuda")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("attention_decode", "attention_prefill", "gemm", "decay_scan", "delta_scan", "conv_unit_prep", "stream_mix_norm"):
        p = sub.add_parser(name)
        p.add_argument("--reps", type=int, default=10)
        p.add_argument("--no-flush", action="store_true", help="do not flush L2 between launches")
        if name == "conv_unit_prep":
            p.add_argument("--taps", type=int, default=4)
        if name == "stream_mix_norm":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--streams", type=int, default=2)
            p.add_argument("--width", type=int, default=4096)
            p.add_argument("--splits", type=int, default=1)
        if name in ("delta_scan", "conv_unit_prep"):
            p.add_argument("--key-heads", type=int, default=0, help="heads of q and k (0: as many as value heads)")
        if name == "delta_scan":
            p.add_argument("--products-in-block", action="store_true", help="no launch ahead for the products between a group's keys and queries")
        if name in ("decay_scan", "delta_scan", "conv_unit_prep"):
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--requests", type=int, default=1)
            p.add_argument("--heads", type=int, default=16)
            p.add_argument("--dim", type=int, default=128)
            p.add_argument("--vdim", type=int, default=128)
        if name == "decay_scan":
            p.add_argument("--read-before", action="store_true", help="o from the state before the update, with a bonus (time mixing)")
        if name.startswith("attention"):
            p.add_argument("--heads", type=int, default=40)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--page-size", type=int, default=64)
            p.add_argument("--chunk", type=int, default=0)
        if name == "attention_decode":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=8192)
            p.add_argument("--split-keys", type=int, default=0, help="keys per split (a multiple of 64) instead of the planned size")
        if name == "attention_prefill":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--tc", action="store_true", help="the tcgen05 kernel (128-token tiles) instead of the mma.sync one")
        if name == "gemm":
            p.add_argument("--rows", type=int, default=8)
            p.add_argument("--n", type=int, default=16384)
            p.add_argument("--k", type=int, default=5120)
            p.add_argument("--experts", type=int, default=0, help="0: one dense weight; else rows are spread over this many groups")
            p.add_argument("--splits", type=int, default=1)
            p.add_argument("--hint", type=int, default=0, help="rows per group that the token tile is sized for (0: twice the mean)")
            p.add_argument("--swiglu", action="store_true", help="fused SiLU(gate) * up epilogue")
    a = ap.parse_args(argv)
    print(json.dumps({"attention_decode": attention_decode, "attention_prefill": attention_prefill, "gemm": gemm, "decay_scan": decay_scan,
                      "delta_scan": delta_scan, "conv_unit_prep": conv_unit_prep, "stream_mix_norm": stream_mix_norm}[a.what](a)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
