"""Python face of the CUDA kernel libraries: loads them with ctypes and launches on torch's
current stream.  There is no fallback: a missing compiler, a failed build or a missing GPU
raises.  Every launch through this module is counted (``launch_count``)."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from .. import tracing
from . import build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {
    1: "a block-table entry pointed outside the page pool",
    2: "a token id was outside the vocabulary",
    4: "a routed expert index was outside the expert count",
    8: "a bounded wait inside a kernel gave up",
}


class KernelError(RuntimeError):
    pass


_libs: dict[str, ctypes.CDLL] = {}
_launches = 0


def launch_count() -> int:
    return _launches


_sm_counts: dict[int, int] = {}


def sm_count() -> int:
    """Multiprocessors of the current device (asked once per device)."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


def library(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        path = build.ensure_built([name])[name]
        lib = ctypes.CDLL(str(path))
        lib.jlx_last_error.restype = ctypes.c_char_p
        _libs[name] = lib
    return lib


def preload(names) -> None:
    """Builds (in parallel) and loads the named libraries."""
    build.ensure_built(list(names))
    for n in names:
        library(n)


def loaded_libraries() -> list[str]:
    return sorted(_libs)


def code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported by the kernels (float32, bfloat16)") from None


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _run(libname: str, fn: str, *args) -> None:
    global _launches
    lib = library(libname)
    timer = tracing.current_timer()
    if timer is None:
        rc = getattr(lib, fn)(*args)
    else:  # Generator(profile="kernels"): CUDA events around the launch
        rc_box = []
        timer.around(fn, lambda: rc_box.append(getattr(lib, fn)(*args)))
        rc = rc_box[0]
    if rc != 0:
        raise KernelError(f"{fn}: {lib.jlx_last_error().decode()}")
    _launches += 1


def _contig(*ts: torch.Tensor | None) -> None:
    for t in ts:
        if t is not None and not t.is_contiguous():
            raise KernelError("a kernel was given a tensor that is not contiguous")


# ------------------------------------------------------------------------------ elementwise
def embed(ids: torch.Tensor, table: torch.Tensor, x_out: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """x_out[n] = scale * table[ids[n]] in float32."""
    _contig(ids, table, x_out)
    V, D = table.shape
    _run("elementwise", "jlx_embed", _ptr(ids), _ptr(table), c_int(code(table.dtype)), _ptr(x_out),
         c_int(ids.numel()), c_int(D), c_int(V), c_float(scale), _ptr(status), _stream())


def _splits(t: torch.Tensor | None, splits: int) -> tuple[int, int]:
    """(split count, elements between partials) of a tensor that may hold split-K partials [splits, ...]."""
    if t is None or splits <= 1:
        return 1, 0
    return splits, t.numel() // splits


DELTA_MAX_TERMS = 3
DELTA_MAX_STREAMS = 64  # rows x split-K partials that one token may add (csrc/elementwise.cu)
DISPATCH_MAX_ROWS, DISPATCH_MAX_PAIRS = 16, 64  # csrc/elementwise.cu


class _DeltaTerm(ctypes.Structure):
    _fields_ = [("p", c_void_p), ("stride", c_longlong), ("index", c_void_p), ("splits", c_int), ("k", c_int), ("base", c_int)]


class _DeltaSpec(ctypes.Structure):
    _fields_ = [("n", c_int), ("t", _DeltaTerm * DELTA_MAX_TERMS)]


class _DispatchArgs(ctypes.Structure):  # DispatchArgs in csrc/elementwise.cu
    _fields_ = [("counter", c_void_p), ("offsets", c_void_p), ("sorted_pair", c_void_p), ("sorted_pos", c_void_p),
                ("tile_list", c_void_p), ("n_tiles", c_void_p), ("a_sorted", c_void_p), ("extra_rows", c_int),
                ("tile_rows", c_int), ("status", c_void_p)]


def add_rmsnorm(x: torch.Tensor, delta, gamma: torch.Tensor | None, eps: float,
                out: torch.Tensor | None, out32: torch.Tensor | None = None, row_index: torch.Tensor | None = None,
                delta_splits: int = 1, w_router: torch.Tensor | None = None, topk_idx: torch.Tensor | None = None,
                topk_w: torch.Tensor | None = None, dispatch=None) -> bool:
    """x (+= delta); out = gamma * x / sqrt(mean(x^2) + eps).  ``delta``: a float32 tensor that may hold
    ``delta_splits`` split-K partials [splits, N, D], added in order; or a list of up to DELTA_MAX_TERMS terms
    ``(data, splits, index, k, base)`` added in the order given: of the float32 partials ``data`` [splits, rows, D]
    token r takes row ``base + r`` or, with ``index`` (int32 [N * k]), the k rows ``index[r * k + j]``.
    With row_index, row n reads source row row_index[n] and x is not written back.  With w_router [E, D] the token
    is routed in the same kernel: topk_idx / topk_w [N, k].  ``dispatch`` (with w_router; an object with the tensors
    counter, offsets, sorted_pair, sorted_pos, a_sorted, status, the optional pair tiles = (tile_list, n_tiles) and
    the numbers extra_rows, tile_rows): what ``expert_sort`` and ``permute_scale`` would write next; the kernel does
    their work too when the step is small enough for that, and the call returns whether it did."""
    terms = [] if delta is None else (list(delta) if isinstance(delta, (list, tuple)) else [(delta, delta_splits, None, 1, 0)])
    _contig(x, gamma, out, out32, row_index, w_router, topk_idx, topk_w, *(t[0] for t in terms), *(t[2] for t in terms))
    D = x.shape[-1]
    n = row_index.numel() if row_index is not None else x.numel() // D
    if x.dtype != torch.float32 or any(t[0].dtype != torch.float32 for t in terms):
        raise KernelError("add_rmsnorm: the residual stream must be float32")
    if gamma is not None and gamma.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the norm weight must be float32")
    if len(terms) > DELTA_MAX_TERMS:
        raise KernelError(f"add_rmsnorm: {len(terms)} terms to add; up to {DELTA_MAX_TERMS} are supported")
    spec = _DeltaSpec()
    spec.n = len(terms)
    for q, (data, splits, index, k_rows, base) in enumerate(terms):
        sp, stride = _splits(data, splits)
        spec.t[q].p, spec.t[q].stride, spec.t[q].splits = data.data_ptr(), stride, sp
        spec.t[q].index, spec.t[q].k, spec.t[q].base = (index.data_ptr() if index is not None else None), k_rows, base
    E = k = 0
    if w_router is not None:
        if w_router.dtype != torch.float32 or topk_idx is None or topk_w is None:
            raise KernelError("router: float32 weight and outputs are needed")
        E, k = w_router.shape[0], topk_idx.shape[1]
    dp, did = None, c_int(0)
    if dispatch is not None and w_router is not None:
        tile_list, n_tiles = dispatch.tiles if dispatch.tiles is not None else (None, None)
        _contig(dispatch.offsets, dispatch.sorted_pair, dispatch.sorted_pos, dispatch.a_sorted, tile_list, n_tiles)
        if out is None or dispatch.a_sorted.dtype != out.dtype:
            raise KernelError("add_rmsnorm: the gathered rows must have the output's type")
        dp = _DispatchArgs(_ptr(dispatch.counter), _ptr(dispatch.offsets), _ptr(dispatch.sorted_pair), _ptr(dispatch.sorted_pos),
                           _ptr(tile_list), _ptr(n_tiles), _ptr(dispatch.a_sorted), dispatch.extra_rows,
                           dispatch.tile_rows if tile_list is not None else 0, _ptr(dispatch.status))
    _run("elementwise", "jlx_add_rmsnorm", _ptr(x), ctypes.byref(spec) if terms else None, _ptr(gamma), c_float(eps),
         _ptr(out), c_int(code(out.dtype) if out is not None else F32), _ptr(out32), _ptr(row_index), c_int(n), c_int(D),
         _ptr(w_router), c_int(E), c_int(k), _ptr(topk_idx), _ptr(topk_w), ctypes.byref(dp) if dp is not None else None,
         ctypes.byref(did), _stream())
    return bool(did.value)


SILU_GLU = (1.0, 0.0, 0.0)  # (alpha, limit, shift) of the gated activation: silu(gate) * up


def glu_form(alpha: float = 1.0, limit: float = 0.0, shift: float = 0.0) -> tuple[float, float, float]:
    """The gated activation  g sigmoid(alpha g) (u + shift)  with g = min(gate, limit), u = clamp(up, -limit, limit)
    when limit > 0: what ``silu_mul`` and the streaming product's epilogue take as ``glu``."""
    if alpha <= 0 or limit < 0:
        raise KernelError(f"gated activation: alpha {alpha} must be positive and limit {limit} not negative (0: none)")
    return (float(alpha), float(limit), float(shift))


def silu_mul(gu: torch.Tensor, out: torch.Tensor, splits: int = 1, interleaved: bool = False, glu=SILU_GLU) -> None:
    """out = silu(gate) * up, or the gated activation ``glu`` (see :func:`glu_form`).  gu: [rows, 2F] (or ``splits``
    float32 partials [splits, rows, 2F]), laid out [gate, up] or, interleaved, in blocks of [16 gate, 16 up]."""
    _contig(gu, out)
    rows, F = out.shape
    sp, stride = _splits(gu, splits)
    _run("elementwise", "jlx_silu_mul", _ptr(gu), c_int(code(gu.dtype)), c_int(sp), c_longlong(stride), _ptr(out),
         c_int(code(out.dtype)), c_int(rows), c_int(F), c_int(int(interleaved)), c_float(glu[0]), c_float(glu[1]), c_float(glu[2]),
         _stream())


# ------------------------------------------------------------------- several residual streams per token
STREAMS_MAX = 16  # csrc/stream_mix.cu


def stream_mix_norm(x: torch.Tensor, streams: int, *, first: torch.Tensor | None = None, y: torch.Tensor | None = None,
                    y_splits: int = 1, mix: torch.Tensor | None = None, write: torch.Tensor | None = None,
                    read: torch.Tensor | None = None, gamma: torch.Tensor | None = None, eps: float = 1e-6,
                    out: torch.Tensor | None = None, out32: torch.Tensor | None = None, row_index: torch.Tensor | None = None,
                    sum_out: torch.Tensor | None = None) -> None:
    """One pass over the S residual streams of every token, x float32 [N, S * D]:
    with a pending sublayer output ``y`` (float32 [N, D] or ``y_splits`` partials):  x_t <- sum_s mix[s, t] x_s + write[t] y;
    then  u = sum_t read[t] x_t  (``read`` None: the plain sum)  and  out / out32 = gamma * u / sqrt(mean(u^2) + eps).
    ``first`` (float32 [N, D]): the streams were never written and all equal this row; they are written, not read.
    With row_index, row n reads source row row_index[n] and x is not written back.  ``sum_out`` [n, D] gets the plain
    sum of the new streams."""
    _contig(x, first, y, mix, write, read, gamma, out, out32, row_index, sum_out)
    S = int(streams)
    if x.dim() != 2 or x.shape[1] % S:
        raise KernelError(f"stream_mix_norm: rows of {x.shape[-1]} do not hold {S} streams")
    D = x.shape[1] // S
    n = row_index.numel() if row_index is not None else x.shape[0]
    if any(t is not None and t.dtype != torch.float32 for t in (x, first, y, mix, write, read, gamma, out32, sum_out)):
        raise KernelError("stream_mix_norm: streams, the pending output, the small weights and the norm weight must be float32")
    if (mix is not None and mix.numel() != S * S) or any(t is not None and t.numel() != S for t in (write, read)):
        raise KernelError(f"stream_mix_norm: {S} streams need a mix matrix of {S} x {S} and read and write weights of {S}")
    if gamma is not None and gamma.numel() != D:
        raise KernelError(f"stream_mix_norm: the norm weight has {gamma.numel()} entries for a width of {D}")
    sp, stride = _splits(y, y_splits)
    _run("stream_mix", "jlx_stream_mix_norm", _ptr(x), _ptr(first), _ptr(y), c_int(sp), c_longlong(stride), _ptr(mix), _ptr(write),
         _ptr(read), _ptr(gamma), c_float(eps), _ptr(out), c_int(code(out.dtype) if out is not None else F32), _ptr(out32),
         _ptr(row_index), _ptr(sum_out), c_int(n), c_int(S), c_int(D), _stream())


# ------------------------------------------------------- grouped norms around a sublayer, biases, short convolution
ACTIVATIONS = {"none": 0, "relu2": 1, "silu": 2, "gelu_tanh": 3, "gelu": 4, "tanh": 5}  # csrc/group_norm.cu ("gelu": the exact, erf form)


def group_norm(x: torch.Tensor, delta: torch.Tensor | None = None, delta_splits: int = 1, delta_bias: torch.Tensor | None = None,
               post_weight: torch.Tensor | None = None, post_groups: int = 1, mult: float = 1.0,
               pre_weight: torch.Tensor | None = None, pre_groups: int = 1, pre_norm: bool = True, eps: float = 1e-6,
               out: torch.Tensor | None = None, out32: torch.Tensor | None = None, row_index: torch.Tensor | None = None,
               post_norm: bool = True) -> None:
    """One pass over each row of the float32 residual x [N, D]:
    x += mult * post_weight * groupnorm(delta + delta_bias) (``delta``: float32 [N, D] or ``delta_splits`` partials of
    it; without post_weight the sum is added as it is; with ``post_norm`` False post_weight is a plain scale per
    channel: x += mult * post_weight * delta), then out / out32 = pre_weight * groupnorm(x) (``pre_norm``
    False: x itself).  groupnorm divides each of ``groups`` equal consecutive parts of a row by
    sqrt(mean(part^2) + eps).  ``out`` may be a view whose rows are longer than D (its row stride is kept).  With
    row_index, row n reads source row row_index[n] and x is not written back."""
    _contig(x, delta, delta_bias, post_weight, pre_weight, out32, row_index)
    N, D = (row_index.numel() if row_index is not None else x.shape[0]), x.shape[1]
    if x.dtype != torch.float32 or any(t is not None and t.dtype != torch.float32 for t in (delta, delta_bias, post_weight, pre_weight)):
        raise KernelError("group_norm: the residual stream, what is added to it and the norm weights must be float32")
    ld_out = D
    if out is not None:
        if out.stride(-1) != 1 or out.shape != (N, D):
            raise KernelError("group_norm: out must be [N, D] with contiguous rows")
        ld_out = out.stride(0) if N > 1 else D
    sp, stride = _splits(delta, delta_splits)
    _run("group_norm", "jlx_group_norm", _ptr(x), _ptr(delta), c_int(sp), c_longlong(stride), _ptr(delta_bias),
         _ptr(post_weight), c_int(post_groups), c_int(int(post_norm)), c_float(mult), _ptr(pre_weight), c_int(pre_groups), c_int(int(pre_norm)),
         c_float(eps), _ptr(out), c_int(code(out.dtype) if out is not None else F32), c_longlong(ld_out), _ptr(out32),
         _ptr(row_index), c_int(N), c_int(D), _stream())


def bias_act(rows: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None, add: torch.Tensor | None = None,
             activation: str = "none", splits: int = 1) -> None:
    """out = activation(rows + bias + add).  rows: [N, F] or ``splits`` float32 partials [splits, N, F]; bias: float32
    [F]; add: float32 [N, F]."""
    _contig(rows, out, bias, add)
    N, F = out.shape
    if any(t is not None and t.dtype != torch.float32 for t in (bias, add)):
        raise KernelError("bias_act: bias and addend must be float32")
    sp, stride = _splits(rows, splits)
    _run("group_norm", "jlx_bias_act", _ptr(rows), c_int(code(rows.dtype)), c_int(sp), c_longlong(stride), _ptr(bias), _ptr(add),
         c_int(ACTIVATIONS[activation]), _ptr(out), c_int(code(out.dtype)), c_int(N), c_int(F), _stream())


def short_conv(h32: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, cu_q: torch.Tensor, q_start: torch.Tensor,
               slot_ids: torch.Tensor, req_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = h[t] + sum_j weight[:, j] * h[t - taps + 1 + j] along each request's time axis (zeros before its start).
    h32: float32 [N, D]; weight: float32 [D, taps]; state: float32 [slots, taps - 1, D], a request's last inputs,
    read for the tokens before this step's and moved on."""
    _contig(h32, weight, state, out)
    N, D = h32.shape
    taps = weight.shape[1]
    if h32.dtype != torch.float32 or weight.dtype != torch.float32 or (state is not None and state.dtype != torch.float32):
        raise KernelError("short_conv: input, weight and state must be float32")
    if weight.shape[0] != D or (state is not None and tuple(state.shape[1:]) != (taps - 1, D)):
        raise KernelError(f"short_conv: shapes do not fit: h {tuple(h32.shape)}, weight {tuple(weight.shape)}")
    _run("group_norm", "jlx_short_conv", _ptr(h32), _ptr(weight), _ptr(state), _ptr(cu_q), _ptr(q_start), _ptr(slot_ids),
         _ptr(req_of_token), _ptr(positions), _ptr(out), c_int(code(out.dtype)), c_int(N), c_int(slot_ids.numel()), c_int(D),
         c_int(taps), _stream())


# ------------------------------------------------------------------------------- recurrences
def _up4(n: int) -> int:
    return -(-n // 4) * 4


def hgrn2_scan_scratch(n_tokens: int, heads: int, dk: int, dv: int, n_segments: int = 0) -> int:
    """float32 elements of scratch that ``hgrn2_scan`` needs: the gated rows and the un-normed outputs, and with
    segments their end/start states, the products of their gates, and the outputs' correction inputs."""
    n = _up4(n_tokens * heads * (2 * dk + dv)) + _up4(n_tokens * heads * dv)
    if n_segments:
        n += _up4(n_segments * heads * dk * dv) + _up4(n_segments * heads * dk) + _up4(n_tokens * heads * dk)
    return n


def hgrn2_scan(qfv: torch.Tensor, splits: int, f_bias: torch.Tensor, lower: torch.Tensor, state: torch.Tensor,
               cu_q: torch.Tensor, slot_ids: torch.Tensor, norm_weight: torch.Tensor | None, eps: float, out: torch.Tensor,
               heads: int, dk: int, dv: int, scratch: torch.Tensor | None = None, segments: torch.Tensor | None = None,
               n_segments: int = 0, segment_tokens: int = 0) -> None:
    """The gated recurrence S = diag(f) S + (1 - f) v^T, o = S^T silu(q) over each request's tokens, then the per-head
    RMS norm of o (three launches: gates, scan, norm).  qfv: float32 [N, 2 H dk + H dv] = [q | f | v] before their
    activations (or ``splits`` partials); state: float32 [slots, H, dk, dv]; out: [N, H dv]; scratch: float32 of
    ``hgrn2_scan_scratch`` elements (made here if not given).
    ``segments`` (int32 [n_segments, 4] = request, first row, end row, flags; at most ``segment_tokens`` rows each, every
    token in exactly one, a request's segments in order): long portions are scanned as several segments at once, each but
    a request's first from a zero state; two more kernels chain the segments' states and correct their outputs.  flags:
    1 = the request's first segment, 2 = the request has several."""
    _contig(qfv, f_bias, lower, state, norm_weight, out, scratch, segments)
    if any(t.dtype != torch.float32 for t in (qfv, f_bias, lower, state)) or (norm_weight is not None and norm_weight.dtype != torch.float32):
        raise KernelError("hgrn2_scan: projections, gate constants, state and norm weight must be float32")
    if tuple(state.shape[1:]) != (heads, dk, dv) or out.shape[1] != heads * dv:
        raise KernelError(f"hgrn2_scan: shapes do not fit: state {tuple(state.shape)}, out {tuple(out.shape)}")
    N = out.shape[0]
    if segments is None:
        n_segments = 0
    elif segments.dtype != torch.int32 or segments.numel() < 4 * n_segments or n_segments <= 0 or segment_tokens <= 0:
        raise KernelError("hgrn2_scan: segments must be int32 [n_segments, 4] with a positive segment size")
    need = hgrn2_scan_scratch(N, heads, dk, dv, n_segments)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=out.device)
    if scratch.dtype != torch.float32 or scratch.numel() < need or scratch.data_ptr() % 16:
        raise KernelError("hgrn2_scan: scratch must be float32, 16-byte aligned, with hgrn2_scan_scratch() elements")
    at = 0

    def cut(n: int):
        nonlocal at
        v = scratch[at:at + n]
        at += _up4(n)
        return v

    gates, o32 = cut(N * heads * (2 * dk + dv)), cut(N * heads * dv)
    seg_state = seg_decay = qd = None
    if n_segments:
        seg_state, seg_decay, qd = cut(n_segments * heads * dk * dv), cut(n_segments * heads * dk), cut(N * heads * dk)
    sp, stride = _splits(qfv, splits)
    global _launches
    _run("recurrent", "jlx_hgrn2_scan", _ptr(qfv), c_int(sp), c_longlong(stride), _ptr(f_bias), _ptr(lower), _ptr(state),
         _ptr(cu_q), _ptr(slot_ids), _ptr(norm_weight), c_float(eps), _ptr(gates), _ptr(o32), _ptr(out), c_int(code(out.dtype)),
         c_int(N), c_int(slot_ids.numel()), c_int(heads), c_int(dk), c_int(dv), c_int(sm_count()),
         _ptr(segments) if n_segments else None, c_int(n_segments), c_int(segment_tokens), _ptr(seg_state), _ptr(seg_decay),
         _ptr(qd), _stream())
    _launches += 2 + (2 if n_segments else 0)  # gates, scan, (chain, correction,) norm


# -------------------------------------------------------------------------- latent attention
def latent_kv_prep(proj: torch.Tensor, splits: int, q_norm_weight: torch.Tensor, kv_norm_weight: torch.Tensor, eps: float,
                   inv_freq: torch.Tensor, rot_dims: int, cq: torch.Tensor, pages: torch.Tensor | None,
                   block_table: torch.Tensor | None, req_of_token: torch.Tensor, positions: torch.Tensor,
                   q_rank: int, rank: int, dr: int, status: torch.Tensor) -> None:
    """From projected rows [N, q_rank + rank + dr] (float32, or partials): cq = weighted RMS norm of the first q_rank
    entries; the page row of the token = [weighted RMS norm of the next rank entries | the last dr entries, rotated].
    pages: [P, 1, 1, page_size, rank + dr]."""
    _contig(proj, q_norm_weight, kv_norm_weight, inv_freq, cq, pages, block_table)
    N = cq.shape[0]
    store = pages is not None
    if store and (pages.dtype != cq.dtype or pages.shape[1:3] != (1, 1) or pages.shape[4] != rank + dr):
        raise KernelError(f"latent_kv_prep: pages {tuple(pages.shape)} do not fit a latent of {rank} + {dr}")
    sp, stride = _splits(proj, splits)
    _run("attention_latent", "jlx_latent_kv_prep", _ptr(proj), c_int(sp), c_longlong(stride), _ptr(q_norm_weight),
         _ptr(kv_norm_weight), c_float(eps), _ptr(inv_freq), c_int(rot_dims), _ptr(cq), _ptr(pages), c_int(code(cq.dtype)),
         _ptr(block_table), c_int(block_table.shape[1] if store else 0), _ptr(req_of_token), _ptr(positions), c_int(N),
         c_int(q_rank), c_int(rank), c_int(dr), c_int(pages.shape[3] if store else 0), c_int(pages.shape[0] if store else 0),
         _ptr(status), _stream())


def latent_q_prep(q: torch.Tensor, splits: int, inv_freq: torch.Tensor, rot_dims: int, positions: torch.Tensor,
                  q_nope: torch.Tensor, q_rot: torch.Tensor, heads: int, dn: int, dr: int, q_full: torch.Tensor | None = None) -> None:
    """q: float32 [N, H (dn + dr)] (or partials) -> q_nope [H, N, dn] (head-major), q_rot float32 [N, H, dr], rotated,
    and optionally q_full [H, N, dn + dr] (both parts, in q_nope's type)."""
    _contig(q, inv_freq, q_nope, q_rot, q_full)
    N = q_rot.shape[0]
    sp, stride = _splits(q, splits)
    _run("attention_latent", "jlx_latent_q_prep", _ptr(q), c_int(sp), c_longlong(stride), _ptr(inv_freq), c_int(rot_dims),
         _ptr(positions), _ptr(q_nope), c_int(code(q_nope.dtype)), _ptr(q_rot), _ptr(q_full), c_int(N), c_int(heads), c_int(dn),
         c_int(dr), _stream())


LATENT_KEY_TILE = 32  # keys per tile of the latent attention kernel: split sizes are multiples of it


def attention_latent(q_lat: torch.Tensor, q_rot: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     req_of_token: torch.Tensor, positions: torch.Tensor, sink: torch.Tensor | None, out_lat: torch.Tensor,
                     scale: float, status: torch.Tensor, rows: torch.Tensor | None = None, n_rows: int = 0, splits: int = 1,
                     split_keys: int = 0, part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None) -> None:
    """Causal attention in the latent space with an optional per-head sink.  q_lat: float32 [H, N, rank]; q_rot:
    float32 [N, H, dr]; pages: [P, 1, 1, page_size, rank + dr]; out_lat: [H, N, rank].
    rows / n_rows: serve these token rows only (int32).  splits > 1: the keys are cut into ranges of ``split_keys``
    (a multiple of LATENT_KEY_TILE), a block each, and a second kernel adds the ranges' results; part_acc: float32
    [served * H * splits * rank], part_ml: float32 [served * H * splits * 2]."""
    _contig(q_lat, q_rot, pages, block_table, sink, out_lat, rows, part_acc, part_ml)
    H, N, rank = q_lat.shape
    dr = q_rot.shape[2]
    if q_lat.dtype != torch.float32 or q_rot.dtype != torch.float32 or (sink is not None and sink.dtype != torch.float32):
        raise KernelError("attention_latent: queries and sinks must be float32")
    if pages.shape[4] != rank + dr:
        raise KernelError("attention_latent: cache rows and queries disagree in size")
    served = n_rows if rows is not None else N
    if splits > 1 and (part_acc is None or part_ml is None or part_acc.numel() < served * H * splits * rank
                       or part_ml.numel() < served * H * splits * 2):
        raise KernelError("attention_latent: scratch for the partial results is missing or too small")
    global _launches
    _run("attention_latent", "jlx_attention_latent", _ptr(q_lat), _ptr(q_rot), _ptr(pages), c_int(code(pages.dtype)),
         _ptr(block_table), c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), _ptr(sink), _ptr(out_lat),
         c_int(code(out_lat.dtype)), c_int(N), c_int(H), c_int(rank), c_int(dr), c_int(pages.shape[3]), c_int(pages.shape[0]),
         c_float(scale), _ptr(rows), c_int(n_rows), c_int(splits), c_int(split_keys), _ptr(part_acc), _ptr(part_ml),
         _ptr(status), _stream())
    _launches += int(splits > 1)  # the combine kernel


def latent_gather(pages: torch.Tensor, block_table_row: torch.Tensor, c: torch.Tensor, kr: torch.Tensor, status: torch.Tensor) -> None:
    """The first L cached rows of one request (its block-table row) as two dense matrices: c [L, rank], kr [L, dr]."""
    _contig(pages, block_table_row, c, kr)
    L, rank = c.shape
    dr = kr.shape[1]
    if pages.shape[4] != rank + dr or c.dtype != pages.dtype or kr.dtype != pages.dtype:
        raise KernelError("latent_gather: cache rows and outputs disagree")
    _run("attention_latent", "jlx_latent_gather", _ptr(pages), c_int(code(pages.dtype)), _ptr(block_table_row), _ptr(c), _ptr(kr),
         c_int(L), c_int(rank), c_int(dr), c_int(pages.shape[3]), c_int(pages.shape[0]), _ptr(status), _stream())


def latent_key_assemble(kv_up: torch.Tensor, kr: torch.Tensor, k: torch.Tensor, heads: int, dn: int) -> None:
    """k[h, t] = [kv_up[t, h dn : (h + 1) dn] | kr[t]].  kv_up: [L, >= H dn] with contiguous rows; kr: [L, dr]; k: [H, L, dn + dr]."""
    _contig(kr, k)
    L, dr = kr.shape
    if kv_up.stride(1) != 1 or tuple(k.shape) != (heads, L, dn + dr) or kv_up.dtype != k.dtype:
        raise KernelError("latent_key_assemble: shapes or types do not fit")
    _run("attention_latent", "jlx_latent_key_assemble", _ptr(kv_up), c_longlong(kv_up.stride(0)), _ptr(kr), _ptr(k),
         c_int(code(k.dtype)), c_int(L), c_int(heads), c_int(dn), c_int(dr), _stream())


def causal_sink_softmax(scores: torch.Tensor, sink: torch.Tensor | None, scale: float, q_start: int, probs: torch.Tensor) -> None:
    """probs[h, i, j] = softmax over j <= q_start + i of scale * scores[h, i, j], the denominator also holding
    exp(sink[h]); 0 beyond the causal edge.  scores: float32 [H, T, L]; probs: [H, T, L]."""
    _contig(scores, sink, probs)
    H, T, L = scores.shape
    if scores.dtype != torch.float32 or probs.shape != scores.shape:
        raise KernelError("causal_sink_softmax: float32 scores and probabilities of the same shape are needed")
    _run("attention_latent", "jlx_causal_sink_softmax", _ptr(scores), _ptr(sink), c_float(scale), c_int(q_start), _ptr(probs),
         c_int(code(probs.dtype)), c_int(H), c_int(T), c_int(L), _stream())


def heads_to_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """x: [H, N, d] -> out: [N, H * d]."""
    _contig(x, out)
    H, N, d = x.shape
    _run("attention_latent", "jlx_heads_to_rows", _ptr(x), _ptr(out), c_int(code(x.dtype)), c_int(N), c_int(H), c_int(d), _stream())


# ------------------------------------------------------ linear attention with a decay per key channel
class _RowsView(ctypes.Structure):  # RowsView in csrc/decay_scan.cu, RopeRowsView in csrc/rope_kv.cu
    _fields_ = [("p", c_void_p), ("split_stride", c_longlong), ("ld", c_longlong), ("splits", c_int), ("pad_", c_int)]


def rows_view(data: torch.Tensor, splits: int = 1, col: int = 0, row: int = 0) -> _RowsView:
    """Columns from ``col`` on (rows from ``row`` on) of float32 projected rows [N, F] or split-K partials [splits, N, F]."""
    if data.dtype != torch.float32 or not data.is_contiguous() or not data.is_cuda:
        raise KernelError("projected rows must be contiguous float32 on the GPU")
    F = data.shape[-1]
    sp, stride = _splits(data, splits)
    v = _RowsView()
    v.p, v.split_stride, v.ld, v.splits = data.data_ptr() + 4 * (row * F + col), stride, F, sp
    v.keep = data  # the view holds an address: the rows must live as long as it does
    return v


def token_shift_blend(h32: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, slot_ids: torch.Tensor,
                      req_of_token: torch.Tensor, out: torch.Tensor, group_offsets: torch.Tensor | None = None) -> None:
    """out[m, n] = h[n] + (h_prev[n] - h[n]) * mu[m], h_prev the request's previous token: the row before, or for a
    step's first token of a request its state (float32 [slots, D], zeros at the start), which then becomes the
    step's last row of the request.  h32: float32 [N, D]; mu: float32 [M, D]; out: [M, N, D].  ``group_offsets`` (int32
    [M + 1]) gets the row offsets m * N of the blends in ``out`` seen as [M N, D]."""
    _contig(h32, mu, state, out)
    N, D = h32.shape
    M = mu.shape[0]
    if any(t.dtype != torch.float32 for t in (h32, mu, state)) or tuple(out.shape) != (M, N, D) or tuple(state.shape[1:]) != (D,):
        raise KernelError("token_shift_blend: float32 rows, blend weights and state [slots, D] and out [M, N, D] are needed")
    _run("decay_scan", "jlx_token_shift_blend", _ptr(h32), _ptr(mu), _ptr(state), _ptr(cu_q), _ptr(slot_ids), _ptr(req_of_token),
         _ptr(out), c_int(code(out.dtype)), c_int(N), c_int(slot_ids.numel()), c_int(D), c_int(M), _ptr(group_offsets), _stream())


DECAY_FORMS = {"double_exp": 0, "sigmoid_power": 1, "head_constant": 2}  # csrc/decay_scan.cu


def decay_prep(q: _RowsView, k: _RowsView, v: _RowsView, z: _RowsView | None, z_bias: torch.Tensor | None, form: str, tau: float,
               q_scale: float, qo: torch.Tensor, ko: torch.Tensor, do: torch.Tensor, vo: torch.Tensor, heads: int, dk: int,
               dv: int, head_decay: torch.Tensor | None = None, k_scale: float = 1.0, inv_freq: torch.Tensor | None = None,
               rot_dims: int = 0, positions: torch.Tensor | None = None) -> None:
    """qo = q_scale * q, ko = k_scale * k, vo = v, do = the decay of every key channel: exp(-exp(z + bias)) ("double_exp"),
    sigmoid(z + bias)^(1 / tau) ("sigmoid_power") or ``head_decay[h]`` ("head_constant": float32 [H], no z), all float32
    [N, H, dk] ([N, H, dv] for vo), from projected rows.  With ``rot_dims`` > 0, q and k are first turned on their first
    rot_dims entries (entry i with i + rot_dims / 2) by the angle positions[n] * inv_freq[i]."""
    _contig(z_bias, qo, ko, do, vo, head_decay, inv_freq, positions)
    N = qo.shape[0]
    if any(t.dtype != torch.float32 for t in (qo, ko, do, vo)) or any(
            t is not None and t.dtype != torch.float32 for t in (z_bias, head_decay, inv_freq)):
        raise KernelError("decay_prep: float32 outputs, bias, decays and frequencies are needed")
    if form == "head_constant" and (head_decay is None or head_decay.numel() != heads):
        raise KernelError(f"decay_prep: a constant decay per head needs {heads} numbers")
    if rot_dims and (inv_freq is None or inv_freq.numel() != rot_dims // 2 or positions is None):
        raise KernelError(f"decay_prep: {rot_dims} rotated entries need {rot_dims // 2} frequencies and the tokens' positions")
    _run("decay_scan", "jlx_decay_prep", ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(z) if z is not None else None,
         _ptr(z_bias), c_int(DECAY_FORMS[form]), c_float(tau), c_float(q_scale), _ptr(qo), _ptr(ko), _ptr(do), _ptr(vo), c_int(N),
         c_int(heads), c_int(dk), c_int(dv), _ptr(head_decay), c_float(k_scale), _ptr(inv_freq), c_int(rot_dims), _ptr(positions),
         _stream())


def decay_scan(q: torch.Tensor, k: torch.Tensor, d: torch.Tensor, v: torch.Tensor, bonus: torch.Tensor | None, state: torch.Tensor,
               cu_q: torch.Tensor, slot_ids: torch.Tensor, o: torch.Tensor, read_after_update: bool) -> None:
    """S <- diag(d_t) S + k_t v_t^T over each request's tokens, in order.  ``read_after_update``: o_t = S_t^T q_t; else
    o_t = (S_(t-1) + diag(bonus) k_t v_t^T)^T q_t.  q, k, d: float32 [N, H, dk]; v, o: [N, H, dv]; bonus: [H, dk];
    state: float32 [slots, H, dk, dv]."""
    _contig(q, k, d, v, bonus, state, o)
    N, H, dk = q.shape
    dv = v.shape[2]
    if any(t.dtype != torch.float32 for t in (q, k, d, v, state, o)) or (bonus is not None and bonus.dtype != torch.float32):
        raise KernelError("decay_scan: everything is float32")
    if tuple(state.shape[1:]) != (H, dk, dv) or tuple(o.shape) != (N, H, dv) or (bonus is not None and bonus.numel() != H * dk):
        raise KernelError(f"decay_scan: shapes do not fit: q {tuple(q.shape)}, v {tuple(v.shape)}, state {tuple(state.shape)}")
    _run("decay_scan", "jlx_decay_scan", _ptr(q), _ptr(k), _ptr(d), _ptr(v), _ptr(bonus), _ptr(state), _ptr(cu_q), _ptr(slot_ids),
         _ptr(o), c_int(slot_ids.numel()), c_int(H), c_int(dk), c_int(dv), c_int(int(read_after_update)), _stream())


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor | None, per_head: bool, gate: _RowsView | None, eps: float, mult: float,
                   out: torch.Tensor) -> None:
    """out[n, h dv + c] = mult * o[n, h, c] / sqrt(mean_c(o[n, h]^2) + eps) * weight * silu(gate[n, h dv + c]).
    o: float32 [N, H, dv]; weight: float32 [H dv] (``per_head``) or [dv] (shared by the heads) or None; out: [N, H dv],
    possibly a column range of wider rows."""
    _contig(o, weight)
    N, H, dv = o.shape
    if o.dtype != torch.float32 or (weight is not None and (weight.dtype != torch.float32 or weight.numel() != (H * dv if per_head else dv))):
        raise KernelError("head_norm_gate: float32 rows and a weight of H * dv (per head) or dv entries are needed")
    if out.shape != (N, H * dv) or out.stride(1) != 1:
        raise KernelError("head_norm_gate: out must be [N, H * dv] with contiguous rows")
    _run("decay_scan", "jlx_head_norm_gate", _ptr(o), _ptr(weight), c_int(int(per_head)), ctypes.byref(gate) if gate is not None else None,
         c_float(eps), c_float(mult), _ptr(out), c_int(code(out.dtype)), c_longlong(out.stride(0) if N > 1 else H * dv), c_int(N),
         c_int(H), c_int(dv), _stream())


# ------------------------------------------------------------------------------ the gated delta rule
CONV_ACTIVATIONS = {"none": 0, "silu": 1}  # csrc/delta_rule.cu


def conv_unit_prep(proj: _RowsView, b_col: int, a_col: int, conv_w: torch.Tensor, conv_state: torch.Tensor | None,
                   rate_log: torch.Tensor, a_bias: torch.Tensor, cu_q: torch.Tensor, q_start: torch.Tensor, slot_ids: torch.Tensor,
                   req_of_token: torch.Tensor, positions: torch.Tensor, qo: torch.Tensor, ko: torch.Tensor, vo: torch.Tensor,
                   beta: torch.Tensor, decay: torch.Tensor, activation: str, unit_eps: float, q_scale: float) -> None:
    """From projected float32 rows whose first C = 2 G dk + H dv columns are the q, k and v channels: each channel
    through a short causal convolution over its request's time axis (``conv_w`` float32 [C, taps], the last column the
    current token's; ``conv_state`` float32 [slots, taps - 1, C] = a request's last inputs, read and moved on) and the
    activation; q and k heads made unit vectors, x / sqrt(sum x^2 + unit_eps), q times ``q_scale``; beta = sigmoid of
    the H columns from ``b_col``; decay = exp(-exp(rate_log) * softplus(columns from a_col + a_bias)).
    qo, ko: float32 [N, G, dk]; vo: [N, H, dv]; beta, decay: [N, H]."""
    _contig(conv_w, conv_state, rate_log, a_bias, qo, ko, vo, beta, decay)
    N, G, dk = qo.shape
    _, H, dv = vo.shape
    C, taps = conv_w.shape
    if any(t.dtype != torch.float32 for t in (conv_w, rate_log, a_bias, qo, ko, vo, beta, decay)) or \
            (conv_state is not None and conv_state.dtype != torch.float32):
        raise KernelError("conv_unit_prep: everything is float32")
    if C != 2 * G * dk + H * dv or rate_log.numel() != H or a_bias.numel() != H or tuple(beta.shape) != (N, H) \
            or tuple(decay.shape) != (N, H) or (conv_state is not None and tuple(conv_state.shape[1:]) != (taps - 1, C)):
        raise KernelError(f"conv_unit_prep: shapes do not fit: conv {tuple(conv_w.shape)} for {G} x {dk} keys and {H} x {dv} values")
    _run("delta_rule", "jlx_conv_unit_prep", ctypes.byref(proj), c_int(b_col), c_int(a_col), _ptr(conv_w), _ptr(conv_state),
         _ptr(rate_log), _ptr(a_bias), _ptr(cu_q), _ptr(q_start), _ptr(slot_ids), _ptr(req_of_token), _ptr(positions), _ptr(qo),
         _ptr(ko), _ptr(vo), _ptr(beta), _ptr(decay), c_int(N), c_int(slot_ids.numel()), c_int(G), c_int(H), c_int(dk), c_int(dv),
         c_int(taps), c_int(CONV_ACTIVATIONS[activation]), c_float(unit_eps), c_float(q_scale), _stream())


DELTA_GROUP = 8  # tokens that delta_scan walks together (csrc/delta_rule.cu)


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
               cu_q: torch.Tensor, slot_ids: torch.Tensor, o: torch.Tensor, req_of_token: torch.Tensor | None = None,
               scratch: torch.Tensor | None = None) -> None:
    """Over each request's tokens, in order:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    q, k: float32 [N, G, dk] (head h reads key head h // (H / G)); v, o: [N, H, dv]; beta, decay: [N, H];
    state: float32 [slots, H, dk, dv].  With `req_of_token` [N] and `scratch` (float32, N * G * 2 * DELTA_GROUP elements) a
    step that holds prompts makes the products between a group's keys and queries once per key head, ahead of the scan."""
    _contig(q, k, v, beta, decay, state, o)
    N, G, dk = q.shape
    _, H, dv = v.shape
    if any(t.dtype != torch.float32 for t in (q, k, v, beta, decay, state, o)):
        raise KernelError("delta_scan: everything is float32")
    if tuple(state.shape[1:]) != (H, dk, dv) or tuple(o.shape) != (N, H, dv) or tuple(k.shape) != (N, G, dk) or H % G:
        raise KernelError(f"delta_scan: shapes do not fit: q {tuple(q.shape)}, v {tuple(v.shape)}, state {tuple(state.shape)}")
    ahead = req_of_token is not None and scratch is not None
    if ahead and (scratch.dtype != torch.float32 or scratch.numel() < N * G * 2 * DELTA_GROUP or not scratch.is_contiguous()):
        raise KernelError(f"delta_scan: the scratch holds {scratch.numel()} elements; {N * G * 2 * DELTA_GROUP} float32 are needed")
    _run("delta_rule", "jlx_delta_scan", _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), _ptr(state), _ptr(cu_q), _ptr(slot_ids),
         _ptr(req_of_token) if ahead else None, _ptr(scratch) if ahead else None, _ptr(o), c_int(N), c_int(slot_ids.numel()), c_int(G),
         c_int(H), c_int(dk), c_int(dv), _stream())


# ---------------------------------- weighted q/k norm + rotate-half rotation + page write; gated attention heads
ROPE_PAIRINGS = {"halves": 0, "pairs": 1}  # csrc/rope_kv.cu
ROPE_NORMS = {"none": 0, "before": 1, "after": 2, "whole": 3}


def rope_norm_kv_store(proj: _RowsView, k_col: int, v_col: int, q_out: torch.Tensor, pages: torch.Tensor | None,
                       block_table: torch.Tensor | None, req_of_token: torch.Tensor, positions: torch.Tensor,
                       q_norm_weight: torch.Tensor | None, k_norm_weight: torch.Tensor | None, eps: float,
                       inv_freq: torch.Tensor | None, rot_dims: int, Hq: int, Hkv: int, dk: int, dv: int, status: torch.Tensor,
                       pairing: str = "halves", norm: str = "before", amplitude: float = 1.0) -> None:
    """From projected float32 rows (q heads from the view's first column, k heads from column k_col, v heads of dv
    entries from v_col; v_col = k_col stores the keys as projected as values): q and k RMS-normed over dk (``norm``:
    "none", "before" or "after" the rotation; with a weight where one is given), their first rot_dims entries rotated
    (``pairing`` "halves": entry i with i + rot_dims / 2; "pairs": entry 2i with 2i + 1); q into q_out [N, Hq, dpad],
    k and v into the token's cache row (pages [P, 2, Hkv, page_size, dpad]), all padded with zeros to dpad.
    ``norm`` "whole": before the rotation, over all heads of q (of k) at once, the weights [Hq dk] and [Hkv dk].
    ``amplitude`` multiplies both the cosine and the sine of every angle."""
    _contig(q_out, pages, block_table, q_norm_weight, k_norm_weight, inv_freq)
    N, _, dpad = q_out.shape
    if norm == "whole" and (q_norm_weight is None or k_norm_weight is None or q_norm_weight.numel() != Hq * dk or k_norm_weight.numel() != Hkv * dk):
        raise KernelError(f"rope_norm_kv_store: a norm over the whole projection needs weights of {Hq * dk} and {Hkv * dk} entries")
    store = pages is not None
    if store and (pages.dtype != q_out.dtype or tuple(pages.shape[1:3]) != (2, Hkv) or pages.shape[4] != dpad):
        raise KernelError(f"rope_norm_kv_store: pages {tuple(pages.shape)} do not fit {Hkv} heads padded to {dpad}")
    _run("rope_kv", "jlx_rope_half_kv_store", ctypes.byref(proj), c_int(k_col), c_int(v_col), _ptr(q_out), _ptr(pages),
         c_int(code(q_out.dtype)), _ptr(block_table), c_int(block_table.shape[1] if store else 0), _ptr(req_of_token),
         _ptr(positions), _ptr(q_norm_weight), _ptr(k_norm_weight), c_float(eps), _ptr(inv_freq), c_int(rot_dims),
         c_int(ROPE_PAIRINGS[pairing]), c_int(ROPE_NORMS[norm]), c_int(N), c_int(Hq), c_int(Hkv), c_int(dk), c_int(dv), c_int(dpad),
         c_int(pages.shape[3] if store else 0), c_int(pages.shape[0] if store else 0), c_int(int(store)), _ptr(status),
         c_float(amplitude), _stream())


def rope_half_kv_store(proj: _RowsView, k_col: int, v_col: int, q_out: torch.Tensor, pages: torch.Tensor | None,
                       block_table: torch.Tensor | None, req_of_token: torch.Tensor, positions: torch.Tensor,
                       q_norm_weight: torch.Tensor | None, k_norm_weight: torch.Tensor | None, eps: float,
                       inv_freq: torch.Tensor | None, rot_dims: int, Hq: int, Hkv: int, dk: int, dv: int, status: torch.Tensor) -> None:
    """:func:`rope_norm_kv_store` in the form "a weighted norm (where both weights are given) before a rotation in halves"."""
    if (q_norm_weight is None) != (k_norm_weight is None):
        raise KernelError("rope_half_kv_store: q and k are normed both or neither")
    rope_norm_kv_store(proj, k_col, v_col, q_out, pages, block_table, req_of_token, positions, q_norm_weight, k_norm_weight, eps,
                       inv_freq, rot_dims, Hq, Hkv, dk, dv, status, "halves", "none" if q_norm_weight is None else "before")


def head_gate(attn: torch.Tensor, gate: _RowsView | None, mult: float, out: torch.Tensor, dv: int, per_channel: bool = False) -> None:
    """out[n, h dv + c] = mult * sigmoid(gate[n, h]) * attn[n, h, c] for c < dv (``per_channel``: gate[n, h dv + c], a gate
    for every output channel).  attn: [N, Hq, dpad]; gate: float32 projected rows (None: no gate); out: [N, Hq dv],
    possibly a column range of wider rows."""
    _contig(attn)
    N, Hq, dpad = attn.shape
    if out.shape != (N, Hq * dv) or out.stride(1) != 1 or out.dtype != attn.dtype:
        raise KernelError("head_gate: out must be [N, Hq * dv] of the attention's type with contiguous rows")
    _run("rope_kv", "jlx_head_gate", _ptr(attn), ctypes.byref(gate) if gate is not None else None, c_int(int(per_channel)),
         c_float(mult), _ptr(out), c_int(code(attn.dtype)), c_longlong(out.stride(0) if N > 1 else Hq * dv), c_int(N), c_int(Hq),
         c_int(dv), c_int(dpad), _stream())


# ------------------------------------------------------------------- position encoding + cache
def rope_kv_store(qkv: torch.Tensor, q_out: torch.Tensor, pages: torch.Tensor | None, block_table: torch.Tensor | None,
                  req_of_token: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None, l2norm: bool,
                  eps: float, Hq: int, Hkv: int, dh: int, status: torch.Tensor, splits: int = 1) -> None:
    """qkv: [N, (Hq + 2 Hkv) * dh] projected rows, or ``splits`` float32 partials of them.
    pages: [num_pages, 2, Hkv, page_size, dh] or None (a layer that writes no cache)."""
    _contig(qkv, q_out, pages, block_table, inv_freq)
    store = pages is not None
    N = q_out.shape[0]
    sp, stride = _splits(qkv, splits)
    _run("rope_kv", "jlx_rope_kv_store", _ptr(qkv), c_int(code(qkv.dtype)), c_int(sp), c_longlong(stride), _ptr(q_out),
         _ptr(pages), c_int(code(q_out.dtype)), _ptr(block_table), c_int(block_table.shape[1] if store else 0),
         _ptr(req_of_token), _ptr(positions), _ptr(inv_freq), c_int(int(l2norm)), c_float(eps), c_int(N), c_int(Hq),
         c_int(Hkv), c_int(dh), c_int(pages.shape[3] if store else 0), c_int(pages.shape[0] if store else 0),
         c_int(int(store)), _ptr(status), _stream())


def kv_store(k: torch.Tensor, v: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
             req_of_token: torch.Tensor, positions: torch.Tensor, status: torch.Tensor) -> None:
    _contig(k, v, pages, block_table)
    N, Hkv, dh = k.shape
    _run("rope_kv", "jlx_kv_store", _ptr(k), _ptr(v), _ptr(pages), c_int(code(k.dtype)), _ptr(block_table),
         c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), c_int(N), c_int(Hkv), c_int(dh),
         c_int(pages.shape[3]), c_int(pages.shape[0]), _ptr(status), _stream())


# ---------------------------------------------------------------------------------- attention
def attention_generic(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                      positions: torch.Tensor, out: torch.Tensor, scale: float, chunk: int, window: int,
                      attn_scale: float, floor_scale: float, status: torch.Tensor, sink: torch.Tensor | None = None,
                      slopes: torch.Tensor | None = None) -> None:
    """q: [N, Hq, dh]; pages: [P, 2, Hkv, page, dh]; out: [N, Hq, dh].  ``sink``: float32 [Hq] or None; with it the
    softmax's denominator has one more term exp(sink[h]) that carries no value.  ``slopes``: float32 [Hq] or None; with
    it slopes[h] * (query position - key position) is taken off every scaled score (all four attention kernels take both)."""
    _contig(q, pages, block_table, out)
    _check_sink(sink, q.shape[1])
    _check_sink(slopes, q.shape[1], "slopes")
    N, Hq, dh = q.shape
    P, _, Hkv, page_size, dh2 = pages.shape
    if dh2 != dh or pages.dtype != q.dtype:
        raise KernelError("attention: cache pages and queries disagree in head size or element type")
    _run("attention_generic", "jlx_attention_generic", _ptr(q), _ptr(pages), c_int(code(q.dtype)), _ptr(block_table),
         c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), _ptr(out), c_int(N), c_int(Hq), c_int(Hkv),
         c_int(dh), c_int(page_size), c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale),
         c_float(floor_scale), _ptr(sink), _ptr(slopes), _ptr(status), _stream())


def _check_sink(sink: torch.Tensor | None, Hq: int, what: str = "sink") -> None:
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != Hq or not sink.is_contiguous()):
        raise KernelError(f"attention: the {what} must be float32 [{Hq}], one number per query head")


def attention_mma_supported(q_dtype: torch.dtype, Hq: int, Hkv: int, dh: int, decode: bool) -> bool:
    if q_dtype != torch.bfloat16:
        return False
    return bool(library("attention_mma").jlx_attention_mma_supported(c_int(Hq), c_int(Hkv), c_int(dh), c_int(int(decode))))


def attention_decode_plan(max_kv_len: int, chunk: int, window: int, pairs: int) -> tuple[int, int]:
    """(keys per split, splits) for a decode launch over `pairs` (request, KV head) pairs."""
    lib = library("attention_mma")
    keys = int(lib.jlx_attention_decode_split_keys(c_int(max_kv_len), c_int(chunk), c_int(window), c_int(pairs)))
    return keys, int(lib.jlx_attention_decode_splits(c_int(max_kv_len), c_int(chunk), c_int(window), c_int(keys)))


def attention_decode(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, scale: float, chunk: int, window: int, attn_scale: float,
                     floor_scale: float, part_o: torch.Tensor, part_ml: torch.Tensor, max_splits: int, split_keys: int,
                     status: torch.Tensor, rows: torch.Tensor | None = None, n_rows: int = 0,
                     sink: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> None:
    """Split-KV attention for one query token per request (tensor cores, bfloat16).
    part_o: float32 [N * Hq * max_splits * dh]; part_ml: float32 [N * Hq * max_splits * 2].
    rows / n_rows: work on these token rows only (int32, the first n_rows entries): the single decoded tokens of
    a step that also holds prompt portions; N is then n_rows."""
    _contig(q, pages, block_table, out, part_o, part_ml, rows)
    N, Hq, dh = q.shape
    _check_sink(sink, Hq)
    _check_sink(slopes, Hq, "slopes")
    if rows is not None:
        N = n_rows
    P, _, Hkv, page_size, _ = pages.shape
    if part_o.numel() < N * Hq * max_splits * dh or part_ml.numel() < N * Hq * max_splits * 2:
        raise KernelError("attention_decode: scratch for the partial results is too small")
    _run("attention_mma", "jlx_attention_decode", _ptr(q), _ptr(pages), _ptr(block_table), c_int(block_table.shape[1]),
         _ptr(req_of_token), _ptr(positions), _ptr(out), c_int(N), c_int(Hq), c_int(Hkv), c_int(dh), c_int(page_size),
         c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale), c_float(floor_scale), _ptr(part_o),
         _ptr(part_ml), c_int(max_splits), c_int(split_keys), _ptr(rows), _ptr(sink), _ptr(slopes), _ptr(status), _stream())


def attention_prefill(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                      positions: torch.Tensor, out: torch.Tensor, tiles: torch.Tensor, n_tiles: int, scale: float,
                      chunk: int, window: int, attn_scale: float, floor_scale: float, status: torch.Tensor,
                      sink: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> None:
    """Flash attention over the paged cache for prompt portions (tensor cores, bfloat16).
    tiles: int32 [n_tiles, 2] = (first token row, count <= 16), each within one request."""
    _contig(q, pages, block_table, out, tiles)
    N, Hq, dh = q.shape
    _check_sink(sink, Hq)
    _check_sink(slopes, Hq, "slopes")
    P, _, Hkv, page_size, _ = pages.shape
    _run("attention_mma", "jlx_attention_prefill", _ptr(q), _ptr(pages), _ptr(block_table), c_int(block_table.shape[1]),
         _ptr(req_of_token), _ptr(positions), _ptr(out), _ptr(tiles), c_int(n_tiles), c_int(Hq), c_int(Hkv), c_int(dh),
         c_int(page_size), c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale),
         c_float(floor_scale), _ptr(sink), _ptr(slopes), _ptr(status), _stream())


def attention_prefill_tc_supported(q_dtype: torch.dtype, Hq: int, Hkv: int, dh: int, page_size: int) -> bool:
    if q_dtype != torch.bfloat16:
        return False
    return bool(library("attention_tc").jlx_attention_prefill_tc_supported(c_int(Hq), c_int(Hkv), c_int(dh), c_int(page_size)))


def attention_prefill_tc(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                         positions: torch.Tensor, out: torch.Tensor, tiles: torch.Tensor, n_tiles: int, scale: float,
                         chunk: int, window: int, attn_scale: float, floor_scale: float, status: torch.Tensor,
                         sink: torch.Tensor | None = None, slopes: torch.Tensor | None = None) -> None:
    """Flash attention for prompt portions on tcgen05 (bfloat16, head size 128, pages of a multiple of 64).
    tiles: int32 [n_tiles, 2] = (first token row, count <= 128), each within one request; only the rows
    of these tiles are written."""
    _contig(q, pages, block_table, out, tiles)
    N, Hq, dh = q.shape
    _check_sink(sink, Hq)
    _check_sink(slopes, Hq, "slopes")
    P, _, Hkv, page_size, _ = pages.shape
    _run("attention_tc", "jlx_attention_prefill_tc", _ptr(q), _ptr(pages), _ptr(block_table), c_int(block_table.shape[1]),
         _ptr(req_of_token), _ptr(positions), _ptr(out), _ptr(tiles), c_int(n_tiles), c_int(N), c_int(Hq), c_int(Hkv),
         c_int(dh), c_int(page_size), c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale),
         c_float(floor_scale), _ptr(sink), _ptr(slopes), _ptr(status), _stream())


# ------------------------------------------------------------------------------------- GEMMs
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor | None = None) -> None:
    """out = a @ w^T.  a: [M, K]; w: [N, K], or [E, N, K] with row-group offsets [E + 1] on the device."""
    _contig(a, w, out, offsets)
    M, K = a.shape
    if offsets is None:
        N, E, stride = w.shape[0], 0, 0
    else:
        E, N = w.shape[0], w.shape[1]
        stride = N * K
    if w.shape[-1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _run("gemm_simt", "jlx_gemm_simt", _ptr(a), c_int(code(a.dtype)), _ptr(w), c_int(code(w.dtype)), _ptr(out),
         c_int(code(out.dtype)), c_int(M), c_int(N), c_int(K), c_longlong(K), c_longlong(K), c_longlong(N),
         _ptr(offsets), c_int(E), c_longlong(stride), _stream())


def gemm_stream_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


GEMM_PLAIN, GEMM_PARTIALS, GEMM_SWIGLU = 0, 1, 2


def gemm_stream_token_tile(rows_hint: int) -> int:
    """The token-tile width gemm_stream uses for this rows_hint."""
    return int(library("gemm_stream").jlx_gemm_stream_token_tile(c_int(rows_hint)))


def gemm_stream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                offsets: torch.Tensor | None = None, rows_hint: int = 0, splits: int = 1,
                scratch: torch.Tensor | None = None, mode: int = GEMM_PLAIN,
                tiles: tuple[torch.Tensor, torch.Tensor] | None = None, offsets_settled: bool = False, glu=SILU_GLU) -> int:
    """a @ w^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulate).  a: [M, K]; w: [N, K] or,
    with row-group offsets [E + 1], [E, N, K].
    GEMM_PLAIN: out [M, N] bfloat16 or float32; splits > 1 cuts K across blocks (scratch: float32
    [splits * M * N]) and adds the partials.  GEMM_PARTIALS: out is float32 [splits, M, N], left for the
    consumer to add.  GEMM_SWIGLU: w's rows are interleaved [16 gate, 16 up]; out [M, N / 2] =
    silu(gate) * up, or the gated activation ``glu`` (see :func:`glu_form`).  ``tiles`` = (tile_list, n_tiles) from
    expert_sort for the same rows_hint.
    ``offsets_settled``: the kernel launched just before this call on the stream was a grouped gemm_stream over the
    same offsets and tiles (this one then finds its tile and asks for its weights without waiting for that one).
    Returns the split count used."""
    _contig(a, w, out, offsets, scratch)
    M, K = a.shape
    E = w.shape[0] if offsets is not None else 0
    N = w.shape[-2]
    if w.shape[-1] != K or (offsets is None) != (w.dim() == 2):
        raise KernelError(f"gemm_stream: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}")
    want = {GEMM_PLAIN: M * N, GEMM_PARTIALS: splits * M * N, GEMM_SWIGLU: M * (N // 2)}[mode]
    if out.numel() < want:
        raise KernelError(f"gemm_stream: out has {out.numel()} elements, {want} are needed")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_stream: bfloat16 operands and a bfloat16 or float32 result are supported")
    if mode == GEMM_PLAIN and splits > 1 and (scratch is None or scratch.numel() < splits * M * N or scratch.dtype != torch.float32):
        raise KernelError("gemm_stream: split-K needs float32 scratch of splits * M * N elements")
    used = c_int(1)
    _run("gemm_stream", "jlx_gemm_stream", _ptr(a), _ptr(w), _ptr(out), c_int(int(out.dtype == torch.float32)), c_int(M),
         c_int(N), c_int(K), _ptr(offsets), c_int(E), c_int(rows_hint), c_int(splits), _ptr(scratch), c_int(mode),
         _ptr(tiles[0]) if tiles else None, _ptr(tiles[1]) if tiles else None, c_int(int(offsets_settled and offsets is not None)),
         ctypes.byref(used), _ptr(status), c_float(glu[0]), c_float(glu[1]), c_float(glu[2]), _stream())
    return used.value


# --------------------------------------------------------------------------------------- MoE
ROUTER_WEIGHT_FORMS = {"sigmoid": 0, "softmax_of_chosen": 1, "softmax_normalized": 2}  # csrc/moe.cu
ROUTER_MAX_GROUPS = 64


def router(h32: torch.Tensor, w_router: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
           scores_out: torch.Tensor | None = None, many_rows: bool = False, bias: torch.Tensor | None = None,
           weight_form: str = "sigmoid", correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1,
           scale: float = 1.0) -> None:
    """Scores h32 @ w_router^T (+ bias) in 32-bit, top-k of the scores (lower index wins ties); the weights are the
    sigmoid of each chosen score, or (``weight_form`` "softmax_of_chosen") the softmax over the chosen scores only.
    "softmax_normalized": s = softmax of the scores over ALL outputs; the choice is made on s + ``correction`` (float32
    [E]), among the ``keep`` best of ``groups`` equal groups of neighbouring outputs only (a group's score is its largest
    choice score); the weights are the chosen s divided by their sum and multiplied by ``scale``.
    ``many_rows``: the kernel that shares each router row among eight tokens (for prompt portions; its sums
    run in another order than the one-token kernel's)."""
    _contig(h32, w_router, topk_idx, topk_w, scores_out, bias)
    N, D = h32.shape
    E, k = w_router.shape[0], topk_idx.shape[1]
    _contig(correction)
    if h32.dtype != torch.float32 or w_router.dtype != torch.float32 or any(
            t is not None and (t.dtype != torch.float32 or t.numel() != E) for t in (bias, correction)):
        raise KernelError("router: scores are computed from float32 input, weight, bias and correction (one number per output)")
    _run("moe", "jlx_router", _ptr(h32), _ptr(w_router), _ptr(topk_idx), _ptr(topk_w), _ptr(scores_out), c_int(N),
         c_int(D), c_int(E), c_int(k), c_int(int(many_rows)), _ptr(bias), c_int(ROUTER_WEIGHT_FORMS[weight_form]),
         _ptr(correction), c_int(groups), c_int(keep), c_float(scale), _stream())


def expert_sort(topk_idx: torch.Tensor, offsets: torch.Tensor, sorted_pair: torch.Tensor, sorted_pos: torch.Tensor,
                E: int, status: torch.Tensor, extra_rows: int = 0, tile_rows: int = 0,
                tile_list: torch.Tensor | None = None, n_tiles: torch.Tensor | None = None, tile_groups: int = 0) -> None:
    """Counting sort of the (token, choice) pairs by expert.  offsets: [E + 1], or [E + 2] with extra_rows > 0:
    one more group of that many rows appended after the experts.  With tile_rows > 0 also the list of row
    tiles of that height that hold rows: tile_list int32 [(ceil(rows / tile_rows) + groups) * 2], n_tiles [1];
    ``tile_groups`` > 0: tiles of the first so many groups only (the later ones are experts without weights)."""
    _contig(topk_idx, offsets, sorted_pair, sorted_pos, tile_list, n_tiles)
    if offsets.numel() < E + 1 + (extra_rows > 0):
        raise KernelError("expert_sort: offsets too short")
    if tile_rows > 0:
        rows, groups = topk_idx.numel() + extra_rows, E + (extra_rows > 0)
        if tile_list is None or n_tiles is None or tile_list.numel() < 2 * (-(-rows // tile_rows) + groups):
            raise KernelError("expert_sort: tile list too short")
    _run("moe", "jlx_expert_sort", _ptr(topk_idx), _ptr(offsets), _ptr(sorted_pair), _ptr(sorted_pos),
         c_int(topk_idx.numel()), c_int(E), c_int(extra_rows), c_int(tile_rows), _ptr(tile_list), _ptr(n_tiles),
         _ptr(status), c_int(tile_groups), _stream())


def permute_scale(h32: torch.Tensor, sorted_pair: torch.Tensor, topk_w: torch.Tensor | None, a_sorted: torch.Tensor, k: int,
                  extra_rows: int = 0) -> None:
    """a_sorted[i] = weight * h32[token] in expert order (``topk_w`` None: unscaled); then extra_rows unscaled copies
    of h32's rows."""
    _contig(h32, sorted_pair, topk_w, a_sorted)
    P = a_sorted.shape[0] - extra_rows
    _run("moe", "jlx_permute_scale", _ptr(h32), _ptr(sorted_pair), _ptr(topk_w), _ptr(a_sorted),
         c_int(code(a_sorted.dtype)), c_int(P), c_int(extra_rows), c_int(h32.shape[1]), c_int(k), _stream())


def moe_combine(y_sorted: torch.Tensor, shared: torch.Tensor | None, sorted_pos: torch.Tensor, delta: torch.Tensor, k: int,
                shared_splits: int = 1, y_splits: int = 1, extra_base: int = -1, pair_weights: torch.Tensor | None = None,
                topk_idx: torch.Tensor | None = None, n_real: int = 0, h_rows: torch.Tensor | None = None) -> None:
    """delta = the sum of each token's expert rows (+ row extra_base + n of y: an appended shared group)
    (+ shared); y_sorted and shared may be split-K partials.  ``pair_weights`` (float32 [N, k]): each expert row is
    multiplied by its (token, choice) weight as it is added (experts whose OUTPUT is weighted).  With ``topk_idx``
    (int32 [N, k]) a choice >= ``n_real`` is an expert without weights whose output is its input: the token's row of
    ``h_rows`` (float32 [N, D]) takes the place of a row of y."""
    _contig(y_sorted, shared, sorted_pos, delta, pair_weights, topk_idx, h_rows)
    if h_rows is not None and (h_rows.dtype != torch.float32 or h_rows.shape != delta.shape):
        raise KernelError("moe_combine: the input rows must be float32 [N, D]")
    N, D = delta.shape
    sp, stride = _splits(shared, shared_splits)
    ysp, ystride = _splits(y_sorted, y_splits)
    _run("moe", "jlx_moe_combine", _ptr(y_sorted), c_int(ysp), c_longlong(ystride), c_int(extra_base), _ptr(shared),
         c_int(sp), c_longlong(stride), _ptr(sorted_pos), _ptr(delta), c_int(N), c_int(D), c_int(k), _ptr(pair_weights),
         _ptr(topk_idx), c_int(n_real), _ptr(h_rows), _stream())


# ---------------------------------------------------------------------------------- sampling
def sample_max_top_k() -> int:
    return int(library("sampling").jlx_sample_max_top_k())


def argmax(logits: torch.Tensor, out: torch.Tensor, part_v: torch.Tensor, part_i: torch.Tensor) -> None:
    """out[m] = index of the largest logit (lowest index on ties).  part_v (float32), part_i (int32): [M * 32] scratch."""
    _contig(logits, out, part_v, part_i)
    if logits.dtype != torch.float32:
        raise KernelError("argmax: logits must be float32")
    M, V = logits.shape
    if part_v.numel() < 32 * M or part_i.numel() < 32 * M:
        raise KernelError("argmax: scratch too small")
    _run("sampling", "jlx_argmax", _ptr(logits), c_int(M), c_int(V), c_longlong(V), _ptr(part_v), _ptr(part_i), _ptr(out),
         _stream())


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           top_k: torch.Tensor | None = None, streams: torch.Tensor | None = None,
           counters: torch.Tensor | None = None, seed: int = 0) -> None:
    """out[m] = argmax (temperature None or <= 1e-3) or a draw from softmax(logits / temperature)."""
    _contig(logits, out, temperature, top_k, streams, counters)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    M, V = logits.shape
    _run("sampling", "jlx_sample", _ptr(logits), c_int(M), c_int(V), c_longlong(V), _ptr(temperature), _ptr(top_k),
         _ptr(streams), _ptr(counters), c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _ptr(out), _stream())
