"""A plain, slow Koduzen: one function per mechanism, float64 on the CPU, token by token where the design is a recurrence.

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


# ------------------------------------------------------------------------------------------------ small pieces
def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_divide(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def plain_frequencies(base, dims):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def yarn_frequencies(base, dims, sc):
    """(frequencies, amplitude): slow-turning pairs are divided by ``factor``, fast ones kept, a linear ramp between
    the two over the pair index; cos and sin are both multiplied by the amplitude."""
    f = plain_frequencies(base, dims)

    def index_of(turns):  # the (real-valued) pair index whose wavelength makes ``turns`` turns over the original length
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)], dtype=F64)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(x, positions, freqs, dims, amplitude=1.0):
    """x [T, heads, d]: entry i < dims/2 is paired with entry i + dims/2; entries from ``dims`` on pass unchanged."""
    half = dims // 2
    if half == 0:
        return x
    a = positions.to(F64)[:, None, None] * freqs[None, None, :]
    c, s = torch.cos(a) * amplitude, torch.sin(a) * amplitude
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_mask(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def softmax_attention(q, k, v, scale, mask, sink=None, bias=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv].  ``bias`` [H, T, T] is taken OFF the scaled scores;
    ``sink`` [H]: one more term exp(sink) in the denominator that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    out = []
    for a in range(H):
        s = (q[:, a] @ k[:, a // per].T) * scale
        if bias is not None:
            s = s - bias[a]
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[a].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[a] - m)
        out.append((e / den) @ v[:, a // per])
    return torch.cat(out, dim=-1)


# ------------------------------------------------------------------------------------------------------ mixers
def retention_recurrence(q, k, v, decay):
    """Per head: S <- decay S + k v^T, o = S^T q, S zero at the start.  q, k [T, H, d]; v [T, H, dv]; decay: H numbers."""
    T, H, d = q.shape
    dv = v.shape[2]
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[a] * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    return o


def retention_mixer(h, P, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ P[p + "q"].T).view(T, H, d)
    k = (h @ P[p + "k"].T).view(T, H, d)
    v = (h @ P[p + "v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot:
        f = plain_frequencies(rot["base"], rot["dims"])
        q, k = rotate_half(q, pos, f, rot["dims"]), rotate_half(k, pos, f, rot["dims"])
    k = k * d ** -0.5
    o = retention_recurrence(q, k, v, m["decay"])
    o = rms_divide(o, eps).reshape(T, H * dv)
    return (o * silu(h @ P[p + "g"].T)) @ P[p + "o"].T


def attention_mixer(h, P, p, m, eps):
    """Windowed softmax attention; q and k normed over the whole projection, then partly rotated (with YaRN)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms_norm(h @ P[p + "q"].T, P[p + "q.norm"], eps).view(T, H, d)
    k = rms_norm(h @ P[p + "k"].T, P[p + "k.norm"], eps).view(T, G, d)
    v = (h @ P[p + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        if rot.get("scaling"):
            f, amp = yarn_frequencies(rot["base"], rot["dims"], rot["scaling"])
        else:
            f, amp = plain_frequencies(rot["base"], rot["dims"]), 1.0
        q, k = rotate_half(q, pos, f, rot["dims"], amp), rotate_half(k, pos, f, rot["dims"], amp)
    a = softmax_attention(q, k, v, m["scale"], window_mask(T, m["mask"]["size"]))
    return a @ P[p + "o"].T


def query_temperature(T, coef, every):
    p = torch.arange(T, dtype=F64)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def distance_bias(T, H):
    """[H, T, T]: slope_h * (i - j), slope_h = 2^(-8 (h + 1) / H)."""
    i = torch.arange(T, dtype=F64)[:, None]
    j = torch.arange(T, dtype=F64)[None, :]
    return torch.stack([2.0 ** (-8.0 * (a + 1) / H) * (i - j) for a in range(H)])


def attention2_keys_values(h, P, p, m):
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    return (h @ P[p + "k"].T).view(T, G, d), (h @ P[p + "v"].T).view(T, G, dv)


def attention2_mixer(h, P, p, m, kv):
    """No rotation: a query temperature by position, a distance bias, a window and a learned sink.  ``kv``: the keys
    and values it attends over (its own, or another layer's)."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    q = (h @ P[p + "q"].T).view(T, H, d)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(T, qt["coef"], qt["every"])[:, None, None]
    k, v = kv
    a = softmax_attention(q, k, v, m["scale"], window_mask(T, m["mask"]["size"]), sink=P[p + "sink"], bias=distance_bias(T, H))
    return a @ P[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def clipped_glu(h, P, p, limit):
    g = torch.clamp(h @ P[p + "gate"].T, max=limit)
    u = torch.clamp(h @ P[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ P[p + "down"].T


def route(h, P, p, r):
    """(chosen [T, top], weights [T, top]) over experts and identity experts together."""
    z = h @ P[p + "router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + P[p + "correction"] if (p + "correction") in P else s
    n = choice.shape[1]
    groups = r.get("groups")
    if groups:
        per = n // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        keep = torch.topk(best, groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, keep, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = torch.topk(choice, r["top"], dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)


def expert_mixture(h, P, p, ml, forced=None):
    """Returns (output, the experts used [T, top], the experts this router chose itself).  ``forced`` [T, top] replaces
    the choice (the tests hand over the engine's, where two scores nearly tie); the weights are this router's."""
    r = ml["router"]
    real = r["experts"]
    own, w = route(h, P, p, r)
    chosen = own
    if forced is not None:
        chosen = forced.to(torch.int64)
        s = torch.softmax(h @ P[p + "router"].T, dim=-1)
        w = torch.gather(s, 1, chosen)
        w = w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c, wt in zip(chosen[t].tolist(), w[t]):
            row = h[t:t + 1]
            y = row if c >= real else clipped_glu(row, P, f"{p}e{c}.", ml["expert"]["limit"])
            out[t] += wt * y[0]
    if ml.get("shared"):
        out = out + clipped_glu(h, P, p + "shared.", ml["shared"]["limit"])
    return out, chosen, own


def feed_forward(h, P, p, ml, forced=None):
    if ml["kind"] == "dense":
        return clipped_glu(h, P, p, ml["limit"]), None, None
    return expert_mixture(h, P, p, ml, forced)


# ------------------------------------------------------------------------------------------------- the decoder
def hyper_sublayer(X, P, p, fn):
    """X [s, T, D]: read u = sum in[s] X_s, y = fn(u), X_t <- sum_s mix[s, t] X_s + out[t] y."""
    u = torch.einsum("s,std->td", P[p + "in"], X)
    y = fn(u)
    return torch.einsum("sr,std->rtd", P[p + "mix"], X) + P[p + "out"][:, None, None] * y[None]


def forward(cfg: dict, P: dict, tokens, forced_choices=None, trace=None):
    """Logits [T, vocab] of one sequence.  ``forced_choices``: {layer: chosen [T, top]}; ``trace``: a list that gets
    (the sum of the streams after the layer, the experts used, the experts its router chose itself) for every layer."""
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams") or 1
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    X = x[None].repeat(S, 1, 1)
    kvs = {}
    for i, L in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", L["mixer"], L["type"]

        def mix(u):
            h = rms_norm(u, P[p + "norm1"], eps)
            if kind == "retention":
                return retention_mixer(h, P, p + "mix.", m, eps)
            if kind == "attention":
                return attention_mixer(h, P, p + "mix.", m, eps)
            if m.get("kv_from") is None:
                kvs[i] = attention2_keys_values(h, P, p + "mix.", m)
            return attention2_mixer(h, P, p + "mix.", m, kvs[i if m.get("kv_from") is None else m["kv_from"]])

        chosen = [None, None]

        def ff(u):
            h = rms_norm(u, P[p + "norm2"], eps)
            y, chosen[0], chosen[1] = feed_forward(h, P, p + "mlp.", L["mlp"], None if forced_choices is None else forced_choices.get(i))
            return y

        if (p + "hc1.in") in P:
            X = hyper_sublayer(X, P, p + "hc1.", mix)
            if L.get("mlp"):
                X = hyper_sublayer(X, P, p + "hc2.", ff)
        else:
            X = X + mix(X[0])[None]
            if L.get("mlp"):
                X = X + ff(X[0])[None]
        if trace is not None:
            trace.append((X.sum(0), chosen[0], chosen[1]))
    return rms_norm(X.sum(0), P["final.norm"], eps) @ P["embed"].T
