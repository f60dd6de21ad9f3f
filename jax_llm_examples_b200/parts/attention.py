"""Attention mixer over the paged cache."""

from __future__ import annotations

import numpy as np
import torch

from ..cache.manager import Retention
from ..kernels import api as K
from ..tracing import scope
from .base import KVNeed, LayerCache, Mixer, PositionEncoding, ProjectedMixer, Rows, Runtime, StepContext, StepShape, register_part
from .linear import linear

# How this part's kernels cut a step's tokens (the planner below is theirs alone; nothing else knows these numbers).
FLASH_TILE = 16  # query rows per block of the mma.sync flash kernel
TC_TILE = 128  # query rows per block of the tcgen05 flash kernel
TC_MIN_TOKENS = 64  # a request that brings at least this many tokens goes to the tcgen05 kernel


def plan_attention_tiles(shape: StepShape) -> dict[str, np.ndarray]:
    """The step's tokens cut for the three attention kernels, once per step on the host.  A step of single
    tokens only needs no lists.  Otherwise, as int32 arrays of (first token row, count) pairs, each within one
    request: ``attn_tiles_all`` = every request that brings several tokens in tiles of FLASH_TILE;
    ``attn_tiles_long`` = requests that bring at least TC_MIN_TOKENS in tiles of TC_TILE; ``attn_tiles_short`` =
    the other requests with several tokens in tiles of FLASH_TILE; and ``attn_single_rows`` = the token rows of
    the requests that bring one token (decoded tokens beside the portions), which the split-KV kernel serves."""
    n_tok = np.asarray(shape.q_lens, dtype=np.int64)
    if n_tok.max() <= 1:
        return {}
    firsts = np.concatenate([[0], np.cumsum(n_tok)[:-1]])

    def cut(rows: int, which) -> np.ndarray:
        t = [(f + o, min(rows, n - o)) for f, n in zip(firsts, n_tok) if which(n) for o in range(0, n, rows)]
        # late tiles of a causal prompt read the most keys: launch them first so that the tail is short
        return np.ascontiguousarray(np.array(t, dtype=np.int32).reshape(-1, 2)[::-1])

    return {
        "attn_tiles_all": cut(FLASH_TILE, lambda n: n > 1),
        "attn_tiles_long": cut(TC_TILE, lambda n: n >= TC_MIN_TOKENS),
        "attn_tiles_short": cut(FLASH_TILE, lambda n: 1 < n < TC_MIN_TOKENS),
        "attn_single_rows": np.ascontiguousarray(firsts[n_tok == 1].astype(np.int32)),
    }


class PagedAttention(Mixer):
    """Grouped-query attention (llama4/llama4_jax/model.py:891-955, 745-794).

    ``w_qkv``: [(Hq + 2 Hkv) * dh, D], the q, k and v projections stacked in that order, each head a
    block of dh rows (HF orientation, chkpt_utils.py:84-89).  ``w_o``: [D, Hq * dh].
    ``chunk``: query and key must lie in the same chunk of that many positions (model.py:738-740);
    ``window``: keys within the last that many positions; None = no such limit.
    ``qk_norm_eps``: eps of the weightless norm of q and k, None = no norm.
    ``sink``: [Hq] or None; with it the softmax's denominator has one more term exp(sink[h]) that carries no value
    (zeros: "one added to the denominator").
    A layer with ``shares_cache`` projects only q and reads pages that another layer wrote.
    """

    kernel_libraries = ("attention_generic", "gemm_simt")
    kernel_libraries_bf16 = ("attention_mma", "attention_tc", "gemm_stream")

    def __init__(self, w_qkv: torch.Tensor, w_o: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PositionEncoding, qk_norm_eps: float | None = None, chunk: int | None = None,
                 window: int | None = None, scale: float | None = None, sink: torch.Tensor | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads are no multiple of {n_kv_heads} KV heads")
        self.sink = self._sink_vector(sink, n_heads)
        rows = (n_heads + 2 * n_kv_heads) * head_dim
        if w_qkv.shape[0] != rows or w_o.shape[1] != n_heads * head_dim or w_o.shape[0] != w_qkv.shape[1]:
            raise ValueError(f"attention weights do not fit: w_qkv {tuple(w_qkv.shape)}, w_o {tuple(w_o.shape)} for "
                             f"{n_heads}/{n_kv_heads} heads of {head_dim}")
        self.w_qkv, self.w_o = w_qkv, w_o
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.chunk, self.window = chunk, window
        self.scale = float(head_dim) ** -0.5 if scale is None else float(scale)  # model.py:774

    sink: torch.Tensor | None = None
    slopes: torch.Tensor | None = None  # [Hq]: slopes[h] * (query position - key position) is taken off the scaled scores

    @staticmethod
    def _sink_vector(sink, n_heads: int, what: str = "sink") -> torch.Tensor | None:
        if sink is None:
            return None
        if sink.numel() != n_heads:
            raise ValueError(f"the {what} has {sink.numel()} entries for {n_heads} query heads")
        return sink.to(torch.float32).contiguous()

    # Head sizes that the tensor-core attention kernels are built for: a model with another head size never
    # asks for them (and so never compiles them).
    MMA_HEAD_SIZES = (64, 128)
    TC_HEAD_SIZES = (128,)

    def required_libraries(self, runtime: Runtime):
        return tuple(n for n in super().required_libraries(runtime)
                     if not (n == "attention_mma" and self.head_dim not in self.MMA_HEAD_SIZES)
                     and not (n == "attention_tc" and self.head_dim not in self.TC_HEAD_SIZES))

    def sub_parts(self):
        return (self.position,)

    def step_planners(self):
        return (plan_attention_tiles,)

    def kv_need(self) -> KVNeed:
        if self.chunk is not None and self.window is None:
            keep = Retention.chunk(self.chunk)
        elif self.window is not None and self.chunk is None:
            keep = Retention.window(self.window)
        else:
            keep = Retention.all()  # both limits at once: keep everything (correct, not minimal)
        return KVNeed(self.n_kv_heads, self.head_dim, keep)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = ctx.runtime
        with scope("qkv_matmul"):  # the scopes carry the reference's names (model.py:906-954)
            qkv = linear(ctx, h, self.w_qkv, rt.dtype, partials=self.position.accepts_partials)
        with scope("rope"):  # with the q/k norm and the cache update (the reference's "cache_update") in one kernel
            q = self.position.encode_and_store(ctx, qkv, self.n_heads, self.n_kv_heads, self.head_dim, cache, self.qk_norm_eps)
        attn_scale, floor_scale = self.position.query_temperature()
        out = torch.empty_like(q)
        with scope("attention"):
            self.attend(ctx, q, cache, out, attn_scale, floor_scale)
        with scope("projection"):
            return linear(ctx, out.view(q.shape[0], -1), self.w_o, torch.float32, partials=True)

    def _split_kv(self, ctx: StepContext, q, cache: LayerCache, out, attn_scale, floor_scale, rows, n_rows: int) -> None:
        """Split-KV attention for requests that bring one token: all rows of q, or the listed ones."""
        chunk, window = self.chunk or 0, self.window or 0
        split_keys, splits = K.attention_decode_plan(ctx.max_kv_len, chunk, window, n_rows * self.n_kv_heads)
        n = n_rows * self.n_heads * splits
        part_o = ctx.workspace.get("attn_part_o", n * self.head_dim, torch.float32)
        part_ml = ctx.workspace.get("attn_part_ml", n * 2, torch.float32)
        K.attention_decode(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, self.scale,
                           chunk, window, attn_scale, floor_scale, part_o, part_ml, splits, split_keys, ctx.status,
                           rows, n_rows, self.sink, self.slopes)

    def attend(self, ctx: StepContext, q, cache: LayerCache, out, attn_scale: float, floor_scale: float) -> None:
        """Tensor-core kernels where they are built (bfloat16, head size 64 or 128, small groups): split-KV for
        requests that bring one token, flash tiles for the others (tcgen05 for long portions of head size 128);
        the generic kernel where those are not built."""
        chunk, window = self.chunk or 0, self.window or 0
        decode = ctx.max_q_len == 1
        if self.head_dim in self.MMA_HEAD_SIZES and K.attention_mma_supported(q.dtype, self.n_heads, self.n_kv_heads,
                                                                              self.head_dim, decode):
            if decode:
                self._split_kv(ctx, q, cache, out, attn_scale, floor_scale, None, q.shape[0])
                return
            tiles_all = ctx.arrays.get("attn_tiles_all")
            if tiles_all is not None:
                count = {name: len(a) for name, a in ctx.host_arrays.items()}
                if count["attn_single_rows"]:
                    # the single decoded tokens of a mixed step go to the split-KV kernel, by their row list
                    self._split_kv(ctx, q, cache, out, attn_scale, floor_scale, ctx.arrays["attn_single_rows"],
                                   count["attn_single_rows"])
                tiles, n_tiles = tiles_all, count["attn_tiles_all"]  # every request that brings more than one token
                if count["attn_tiles_long"] and self.head_dim in self.TC_HEAD_SIZES and K.attention_prefill_tc_supported(
                        q.dtype, self.n_heads, self.n_kv_heads, self.head_dim, cache.pages.shape[3]):
                    # long portions on the tcgen05 kernel (128-token tiles), the short ones below
                    K.attention_prefill_tc(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out,
                                           ctx.arrays["attn_tiles_long"], count["attn_tiles_long"], self.scale, chunk, window,
                                           attn_scale, floor_scale, ctx.status, self.sink, self.slopes)
                    tiles, n_tiles = ctx.arrays["attn_tiles_short"], count["attn_tiles_short"]
                    kinds = ("tc", "flash" if n_tiles else "", "split_kv" if count["attn_single_rows"] else "")
                    ctx.scratch.setdefault("attention_kernels", set()).add(tuple(k for k in kinds if k))
                if n_tiles:
                    K.attention_prefill(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, tiles,
                                        n_tiles, self.scale, chunk, window, attn_scale, floor_scale, ctx.status, self.sink, self.slopes)
                return
        K.attention_generic(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, self.scale,
                            self.chunk or 0, self.window or 0, attn_scale, floor_scale, ctx.status, self.sink, self.slopes)


register_part("mixer", "paged_attention", PagedAttention)


class GatedPagedAttention(ProjectedMixer, PagedAttention):
    """Grouped-query softmax attention over the paged cache in a general form: queries and keys RMS-normed over the head
    (with a weight or without; BEFORE or AFTER the rotation; or not at all), rotated on their first ``rot_dims`` entries
    only (``pairing`` "halves": entry i with i + rot_dims / 2, the rotate-half layout; "pairs": entry 2i with 2i + 1;
    angle position * inv_freq[i]), values of another size than keys, or the keys themselves as projected
    (``values_are_keys``: no value projection), an optional sink in the softmax, and a sigmoid gate on the heads'
    outputs before the output product, one number per token and head (``gate`` "head") or per output channel ("channel"):

        out = W_o [ sigmoid(W_g h)_a * softmax(scale * q_a K^T) V  for every head a ]

    ``w_in``: the q, k, v and gate projections stacked in that order, [Hq dk + Hkv dk + Hkv dv + gate rows, D] (no v rows
    with ``values_are_keys``; no k and v rows with ``projects_kv`` False: the layer reads the pages that another layer
    fills, with its own queries, mask, sink and slopes; gate rows: Hq, Hq dv or none).  ``q_norm_weight`` /
    ``k_norm_weight``: [dk], shared by the heads.  ``norm``: "before", "after" or "none"; None = "before" if a weight is
    given, else "none"; "whole": before the rotation, ONE norm over all heads of q (and one over all of k), weights
    [Hq dk] and [Hkv dk].  ``rot_amplitude`` multiplies the cosine and the sine of every angle (a rotation that also
    stretches the rotated entries).  ``slopes`` [Hq]: slopes[h] * (i - j) is taken off the scaled score of query i and key
    j.  ``query_temperature`` (coef, every): queries at position p are multiplied by 1 + coef * ln(floor((p + 1) / every)
    + 1).  ``keep_window``: pages are kept for a window of at least this many positions (a layer with a longer window
    reads them; 0: for good).  ``window``: a query
    sees itself and the window - 1 positions before it; ``chunk``: the positions of its own chunk.  Keys, queries and
    values are kept at one padded size (``padded_dim`` >= max(dk, dv), zeros beyond their own): one page layout, and the
    attention kernels built for equal sizes, serve both.  It is a :class:`ProjectedMixer`: beside another mixer that
    reads the same input, both share their input and output products."""

    kernel_libraries = ("attention_generic", "gemm_simt", "rope_kv")
    kernel_libraries_bf16 = ("attention_mma", "attention_tc", "gemm_stream")

    def __init__(self, w_in: torch.Tensor, w_o: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int,
                 scale: float, eps: float, q_norm_weight: torch.Tensor | None = None, k_norm_weight: torch.Tensor | None = None,
                 inv_freq: torch.Tensor | None = None, rot_dims: int = 0, window: int | None = None, chunk: int | None = None,
                 gated: bool = True, padded_dim: int | None = None, sink: torch.Tensor | None = None, pairing: str = "halves",
                 norm: str | None = None, values_are_keys: bool = False, gate: str | None = None,
                 rot_amplitude: float = 1.0, slopes: torch.Tensor | None = None, query_temperature: tuple[float, float] | None = None,
                 projects_kv: bool = True, keep_window: int | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads are no multiple of {n_kv_heads} KV heads")
        gate = ("head" if gated else "none") if gate is None else gate
        if gate not in ("none", "head", "channel") or pairing not in K.ROPE_PAIRINGS:
            raise ValueError(f"gate {gate!r} (none, head, channel) or pairing {pairing!r} (halves, pairs) is unknown")
        if values_are_keys and value_dim != head_dim:
            raise ValueError(f"values that are the keys have the keys' size {head_dim}, not {value_dim}")
        gate_rows = {"none": 0, "head": n_heads, "channel": n_heads * value_dim}[gate]
        kv_rows = n_kv_heads * head_dim + (0 if values_are_keys else n_kv_heads * value_dim) if projects_kv else 0
        rows = n_heads * head_dim + kv_rows + gate_rows
        if w_in.shape[0] != rows or w_o.shape[1] != n_heads * value_dim or w_o.shape[0] != w_in.shape[1]:
            raise ValueError(f"attention weights do not fit: w_in {tuple(w_in.shape)}, w_o {tuple(w_o.shape)} for {n_heads}/"
                             f"{n_kv_heads} heads of {head_dim} (values {value_dim}{', the keys' if values_are_keys else ''}"
                             f"{'' if projects_kv else '; keys and values are another layer\'s'}) with gate {gate!r}")
        if rot_dims % 2 or not 0 <= rot_dims <= head_dim or (rot_dims and (inv_freq is None or inv_freq.numel() != rot_dims // 2)):
            raise ValueError(f"{rot_dims} rotated entries of {head_dim} need {rot_dims // 2} frequencies")
        if (q_norm_weight is None) != (k_norm_weight is None):
            raise ValueError("q and k are normed with a weight each, or both without")
        self.norm = ("none" if q_norm_weight is None else "before") if norm is None else norm
        if self.norm not in K.ROPE_NORMS:
            raise ValueError(f"norm {norm!r} is unknown (none, before, after, whole)")
        for w, heads in ((q_norm_weight, n_heads), (k_norm_weight, n_kv_heads)):
            want = heads * head_dim if self.norm == "whole" else head_dim  # "whole": one norm over all heads of the projection
            if w is not None and w.numel() != want:
                raise ValueError(f"a q/k norm weight has {w.numel()} entries; the norm {self.norm!r} of heads of {head_dim} takes {want}")
        if self.norm == "whole" and q_norm_weight is None:
            raise ValueError("the norm over a whole projection takes a weight for q and one for k")
        if not projects_kv and keep_window is not None:
            raise ValueError("a layer that reads another layer's keys and values keeps none itself")
        self.w_in, self.w_o = w_in, w_o
        self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim = n_heads, n_kv_heads, head_dim, value_dim
        self.head_dim = max(head_dim, value_dim) if padded_dim is None else int(padded_dim)  # what the cache and the kernels see
        if self.head_dim < max(head_dim, value_dim):
            raise ValueError(f"padded size {self.head_dim} is below the key or value size")
        f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()  # noqa: E731
        self.q_norm_weight, self.k_norm_weight, self.inv_freq = f32(q_norm_weight), f32(k_norm_weight), f32(inv_freq)
        self.rot_dims, self.eps, self.gate, self.gated = int(rot_dims), float(eps), gate, gate != "none"
        self.pairing, self.values_are_keys = pairing, bool(values_are_keys)
        self.chunk, self.window, self.scale = chunk, window, float(scale)
        self.sink = self._sink_vector(sink, n_heads)
        self.slopes = self._sink_vector(slopes, n_heads, "slope vector")
        self.rot_amplitude = float(rot_amplitude)
        self.q_temperature = (0.0, 1.0) if query_temperature is None else (float(query_temperature[0]), float(query_temperature[1]))
        if self.q_temperature[0] != 0.0 and self.q_temperature[1] <= 0:
            raise ValueError("the query temperature's period must be positive")
        self.projects_kv, self.keep_window = bool(projects_kv), keep_window
        self.position, self.qk_norm_eps = None, None

    def kv_need(self) -> KVNeed:
        need = PagedAttention.kv_need(self)
        if self.keep_window is not None and self.window is not None and self.chunk is None:
            # another layer reads these pages through a longer window (0: without one): keep them that long
            keep = Retention.all() if self.keep_window == 0 else Retention.window(max(self.window, self.keep_window))
            need = KVNeed(need.num_kv_heads, need.head_dim, keep)
        return need

    @staticmethod
    def padded_size(head_dim: int, value_dim: int, dtype: torch.dtype) -> int:
        """The common size of keys and values in the cache: with bfloat16 the next size that the tensor-core
        attention kernels are built for, if there is one; else the larger of the two."""
        d = max(head_dim, value_dim)
        if dtype == torch.bfloat16:
            for size in PagedAttention.MMA_HEAD_SIZES:
                if d <= size:
                    return size
        return d

    def sub_parts(self):
        return ()

    def _attend_rows(self, ctx: StepContext, proj: Rows, col: int, cache: LayerCache) -> torch.Tensor:
        """Norm, rotation and page write of the projected rows, then attention: [N, Hq, padded size]."""
        Hq, Hkv, dk, dv = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim
        n = proj.data.shape[-2]
        k_col = Hq * dk
        v_col = k_col if self.values_are_keys else k_col + Hkv * dk  # the keys as projected stand in for values
        if not self.projects_kv and cache.writes:
            raise RuntimeError("an attention layer without key and value projections was scheduled to fill a cache")
        q = torch.empty((n, Hq, self.head_dim), dtype=ctx.runtime.dtype, device=proj.data.device)
        with scope("rope"):
            K.rope_norm_kv_store(K.rows_view(proj.data, proj.splits, col), k_col, v_col, q,
                                 cache.pages if cache.writes else None, cache.block_table if cache.writes else None,
                                 ctx.req_of_token, ctx.positions, self.q_norm_weight, self.k_norm_weight, self.eps,
                                 self.inv_freq, self.rot_dims, Hq, Hkv, dk, dv, ctx.status, self.pairing, self.norm,
                                 self.rot_amplitude)
        attn = torch.empty_like(q)
        with scope("attention"):
            self.attend(ctx, q, cache, attn, *self.q_temperature)
        return attn

    def core(self, ctx: StepContext, h, proj: Rows, col: int, cache: LayerCache, out: torch.Tensor, mult: float) -> None:
        Hq, Hkv, dk, dv = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim
        gate_col = Hq * dk
        if self.projects_kv:
            gate_col += Hkv * dk + (0 if self.values_are_keys else Hkv * dv)
        attn = self._attend_rows(ctx, proj, col, cache)
        with scope("attention"):
            gate = K.rows_view(proj.data, proj.splits, col + gate_col) if self.gated else None
            K.head_gate(attn, gate, mult, out, dv, per_channel=self.gate == "channel")

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache):
        if self.gated or self.value_dim != self.head_dim:
            return ProjectedMixer.forward(self, ctx, h, cache)
        # no gate and no padding: the heads' outputs are the output product's rows as they lie
        from .base import as_rows

        with scope("qkv_matmul"):
            proj = as_rows(linear(ctx, h, self.w_in, torch.float32, partials=True))
        attn = self._attend_rows(ctx, proj, 0, cache)
        with scope("projection"):
            return linear(ctx, attn.view(attn.shape[0], -1), self.w_o, torch.float32, partials=True)


register_part("mixer", "gated_paged_attention", GatedPagedAttention)
