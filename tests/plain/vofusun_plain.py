"""A plain, slow Vofusun: one function per mechanism, float64 on the CPU, token by token where the design is a recurrence.

It shares nothing with the package: its own config reading (plain dictionaries), its own safetensors reader, its own
formulas.  ``forward`` runs whole sequences; the tests compare the engine's logits, however its steps were cut, with these.

Notation: h [T, D] rows of one sequence; W [out, in] applied as ``h @ W.T``; P maps tensor names to float64 tensors.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def read_safetensors(path) -> dict:
    """name -> float64 tensor (integers stay integers): 8 bytes of header length, a JSON header, then the data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    types = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32,
             "I64": torch.int64}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=types[meta["dtype"]]).reshape(meta["shape"])
        out[name] = t.to(F64) if t.is_floating_point() else t
    return out


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def unit_vector(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softmax_with_sink(s):
    """p_j = exp(s_j) / (1 + sum_i exp(s_i)): one more term of score zero in the denominator, which carries no value."""
    m = torch.clamp(s.max(), min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum())


def scaled_frequencies(base, dims, scaling):
    """f_i = base^(-2i/dims), short wavelengths kept, long ones divided by ``factor``, a linear blend between."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_pairs(x, positions, freqs):
    """x [T, heads, d]: entries (2i, 2i+1), i < len(freqs), are turned by position * f_i; the rest pass unchanged."""
    n = freqs.numel()
    if n == 0:
        return x
    a = positions.to(F64)[:, None, None] * freqs[None, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., 2 * n:]], dim=-1)


def masked_attention(q, k, v, scale, sees):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; ``sees(i, j)`` for j <= i.  Softmax with the sink."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        keys = [j for j in range(i + 1) if sees(i, j)]
        for a in range(H):
            g = a // (H // G)
            p = softmax_with_sink((k[keys, g] @ q[i, a]) * scale)
            out[i, a] = p @ v[keys, g]
    return out


def window_attention(h, P, p, m, eps):
    """The ``attention`` mixer: no positions in the scores, a sliding window, the sink."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ P[p + "q"].T).view(T, H, d)
    k = (h @ P[p + "k"].T).view(T, G, d)
    v = (h @ P[p + "v"].T).view(T, G, dv)
    span = m["mask"]["size"]
    out = masked_attention(q, k, v, m["scale"], lambda i, j: i - j < span)
    return out.reshape(T, H * dv) @ P[p + "o"].T


def chunk_attention(h, P, p, m, eps):
    """The ``attention_2`` mixer: values are the keys as projected; q and k are turned, then divided by their root mean
    square; queries see their own chunk; the sink; a sigmoid gate on every output channel."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ P[p + "q"].T).view(T, H, d)
    k = (h @ P[p + "k"].T).view(T, G, d)
    v = k.clone()
    rot = m.get("rot")
    if rot is not None:
        f = scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        pos = torch.arange(T)
        q, k = rotate_pairs(q, pos, f), rotate_pairs(k, pos, f)
    q, k = rms_divide(q, eps), rms_divide(k, eps)
    size = m["mask"]["size"]
    out = masked_attention(q, k, v, m["scale"], lambda i, j: i // size == j // size)
    out = out.reshape(T, H * d) * torch.sigmoid(h @ P[p + "g"].T)
    return out @ P[p + "o"].T


def causal_conv_silu(x, w):
    """x [T, C], w [C, taps]: y_t = silu(sum_j w[:, j] x_(t - taps + 1 + j)), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return silu(y)


def decay_and_step(h, P, p):
    """Per token and head: the state's decay g = exp(-exp(A_log) softplus(W_a h + dt_bias)) and the step beta = sigmoid(W_b h)."""
    decay = torch.exp(-torch.exp(P[p + "A_log"]) * torch.nn.functional.softplus(h @ P[p + "a"].T + P[p + "dt_bias"]))
    return decay, torch.sigmoid(h @ P[p + "b"].T)


def delta_recurrence(q, k, v, beta, decay, S=None):
    """q, k [T, G, d]; v [T, H, dv]; beta, decay [T, H].  Token by token and head by head: decay the state, correct what
    it says about k towards v by the step beta, then read it with q.  Returns o [T, H, dv] and the last state [H, d, dv]."""
    T, G, d = q.shape
    H, dv = v.shape[1], v.shape[2]
    S = torch.zeros(H, d, dv, dtype=F64) if S is None else S.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = decay[t, a] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, g])
            S[a] = S[a] + torch.outer(k[t, g], u)
            o[t, a] = S[a].T @ q[t, g]
    return o, S


def delta_mixer(h, P, p, m, eps):
    """The gated delta rule behind short convolutions, with a normed and gated read-out."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ P[p + "q"].T, P[p + "q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ P[p + "k"].T, P[p + "k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ P[p + "v"].T, P[p + "v.conv"]).view(T, H, dv)
    q = unit_vector(q) * d ** -0.5
    k = unit_vector(k)
    decay, beta = decay_and_step(h, P, p)
    o, _ = delta_recurrence(q, k, v, beta, decay)
    o = rms_divide(o, eps) * P[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ P[p + "g"].T)
    return o @ P[p + "o"].T


def dense_mlp(h, P, p):
    return (silu(h @ P[p + "gate"].T) * (h @ P[p + "up"].T)) @ P[p + "down"].T


MIXERS = {"attention": window_attention, "delta": delta_mixer, "attention_2": chunk_attention}


def layer_order(config: dict):
    """(layer index, opens a pass after the first) in the order the layers run."""
    n, loop = len(config["layers"]), config.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    lo, hi, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(lo)]
    for t in range(times):
        order += [(i, t > 0 and i == lo) for i in range(lo, hi)]
    return order + [(i, False) for i in range(hi, n)]


def forward(config: dict, P: dict, tokens):
    """logits [T, vocab] and the residual stream after every layer run [runs, T, D]."""
    eps = config["norm"]["eps"]
    x0 = P["embed"][torch.as_tensor(tokens, dtype=torch.int64)] * config["embedding"]["scale"]
    x = x0.clone()
    after = []
    for i, opens in layer_order(config):
        L, p = config["layers"][i], f"l{i}."
        if opens:
            x = x + x0
        h = rms_divide(x, eps) * P[p + "norm1"]
        x = x + MIXERS[L["type"]](h, P, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            h = rms_divide(x, eps) * P[p + "norm2"]
            x = x + dense_mlp(h, P, p + "mlp.")
        after.append(x.clone())
    logits = (rms_divide(x, eps) * P["final.norm"]) @ P["embed"].T
    return logits, torch.stack(after)
