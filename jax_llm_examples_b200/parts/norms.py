"""Norm parts."""

from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Norm, Rows, RowSum, StepContext, as_rows, register_part


class RMSNorm(Norm):
    """out = weight * x / sqrt(mean(x^2) + eps), mean and division in float32
    (llama4/llama4_jax/model.py:885-888).  ``weight`` None = weightless.  The residual sum x += delta
    runs in the same kernel, and so can the router of a following routed feed-forward."""

    kernel_libraries = ("elementwise",)
    fuses_router = True
    FUSED_ROUTER_MAX_ROWS = 64  # above this many rows (bfloat16) the router runs as its own many-rows kernel

    def __init__(self, weight: torch.Tensor | None, eps: float):
        self.weight = None if weight is None else weight.to(torch.float32).contiguous()
        self.eps = float(eps)

    def forward(self, ctx: StepContext, x, delta, *, out_dtype, want_f32=False, row_index=None, router=None):
        n = x.shape[0] if row_index is None else row_index.numel()
        dev = x.device
        out = torch.empty((n, x.shape[1]), dtype=out_dtype, device=dev)
        out32 = torch.empty((n, x.shape[1]), dtype=torch.float32, device=dev) if want_f32 else None
        # a sum of terms (an expert layer's rows still in expert order) is added term by term in the kernel
        # (the kernel takes so many terms, rows per token and partials; beyond that the sum is made by its producer)
        if isinstance(delta, RowSum) and len(delta.terms) <= K.DELTA_MAX_TERMS and all(t.k <= 16 for t in delta.terms) and \
                sum((t.k if t.index is not None else 1) * t.splits for t in delta.terms) <= K.DELTA_MAX_STREAMS:
            terms = [(t.data, t.splits, t.index, t.k, t.base) for t in delta.terms]
        else:
            d = as_rows(delta)
            terms = None if d is None else [(d.data, d.splits, None, 1, 0)]
        routing = None
        w_router = idx = wt = None
        unfused = False
        if router is not None and x.shape[1] <= 16384:
            w_router, k, *offer = router
            idx = torch.empty((n, k), dtype=torch.int32, device=dev)
            wt = torch.empty((n, k), dtype=torch.float32, device=dev)
            routing = (idx, wt)
            # Prompt portions in bfloat16: the router as a kernel of its own that shares each router row among
            # eight tokens (the fused kernel would fetch all router weights once per token).  The 32-bit path
            # keeps the fused kernel at every size: its sums must not depend on the batch.
            unfused = out_dtype == torch.bfloat16 and n > self.FUSED_ROUTER_MAX_ROWS and x.shape[1] % 4 == 0
            if unfused and out32 is None:
                out32 = torch.empty((n, x.shape[1]), dtype=torch.float32, device=dev)
        # a decode step's few rows: the kernel can also sort the choices and gather the rows for the experts
        dispatch = None
        if routing is not None and not unfused and offer and offer[0] is not None and row_index is None \
                and out_dtype == torch.bfloat16 and n <= K.DISPATCH_MAX_ROWS and n * k <= K.DISPATCH_MAX_PAIRS:
            dispatch = offer[0](ctx, n)
        did = K.add_rmsnorm(x, terms, self.weight, self.eps, out, out32, row_index, 1, None if unfused else w_router, idx, wt,
                            dispatch)
        if did:
            routing = (idx, wt, dispatch)
        if unfused:
            K.router(out32, w_router, idx, wt, many_rows=True)
        return out, out32, routing


register_part("norm", "rms", RMSNorm)


class GroupRMSNorm(Norm):
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, each part is divided by its own
    sqrt(mean(part^2) + eps), and the whole is multiplied by ``weight`` (``groups`` = 1 is the plain RMS norm).

    The pending delta may be a :class:`PostNormed`: a sublayer's output that is itself to be group-normed, scaled
    and then added.  That norm, the residual sum and this norm run in one pass over the row (one kernel)."""

    kernel_libraries = ("group_norm",)

    def __init__(self, weight: torch.Tensor, eps: float, groups: int = 1):
        if weight.numel() % groups:
            raise ValueError(f"{groups} norm groups do not divide the width {weight.numel()}")
        self.weight = weight.to(torch.float32).contiguous()
        self.eps, self.groups = float(eps), int(groups)

    def forward(self, ctx: StepContext, x, delta, *, out_dtype, want_f32=False, row_index=None, router=None):
        """``out_dtype`` None: only the float32 rows are made (for a consumer that takes those)."""
        n = x.shape[0] if row_index is None else row_index.numel()
        out = None if out_dtype is None else torch.empty((n, x.shape[1]), dtype=out_dtype, device=x.device)
        out32 = torch.empty((n, x.shape[1]), dtype=torch.float32, device=x.device) if want_f32 else None
        add_to_residual(x, delta, pre_weight=self.weight, pre_groups=self.groups, eps=self.eps, out=out, out32=out32,
                        row_index=row_index)
        return out, out32, None


def add_to_residual(x: torch.Tensor, delta, *, pre_weight=None, pre_groups: int = 1, pre_norm: bool = True, eps: float = 1e-6,
                    out=None, out32=None, row_index=None) -> None:
    """x += delta, whatever form the pending delta has (None, a tensor, split-K partials, a :class:`PostNormed`, a
    :class:`Scaled`),
    and, in the same pass, out / out32 = the group norm of the new x (``pre_norm`` False: the new x itself)."""
    from .base import PostNormed, Scaled

    if isinstance(delta, Scaled):  # x += scale * delta, channel by channel, in the same pass
        K.group_norm(x, delta.rows.data, delta.rows.splits, None, delta.scale, 1, 1.0, pre_weight, pre_groups, pre_norm, eps,
                     out, out32, row_index, post_norm=False)
        return
    if isinstance(delta, PostNormed):
        if abs(delta.eps - eps) > 0:
            # one kernel takes one eps: norm the delta on its own first
            delta = Rows(delta.materialize(), 1)
        else:
            K.group_norm(x, delta.rows.data, delta.rows.splits, delta.bias, delta.weight, delta.groups, delta.mult,
                         pre_weight, pre_groups, pre_norm, eps, out, out32, row_index)
            return
    d = as_rows(delta)
    if d is not None and d.data.dtype != torch.float32:
        d = Rows(d.data.to(torch.float32), d.splits)
    K.group_norm(x, None if d is None else d.data, 1 if d is None else d.splits, None, None, 1, 1.0,
                 pre_weight, pre_groups, pre_norm, eps, out, out32, row_index)


register_part("norm", "group_rms", GroupRMSNorm)


class StreamRMSNorm(Norm):
    """The norm in front of a sublayer of a model that keeps ``streams`` residual rows per token (x: float32
    [N, streams * D]): the sublayer reads  u = sum_t read[t] x_t  (``read`` None: the plain sum, as the model's final
    norm does) and this part returns  weight * u / sqrt(mean(u^2) + eps).  A pending :class:`StreamMixed` (the output
    of the sublayer before, with its mix matrix and write weights) is written into the streams in the same kernel,
    which is to several streams what the residual-add + norm kernel is to one."""

    kernel_libraries = ("stream_mix",)

    def __init__(self, weight: torch.Tensor | None, eps: float, streams: int, read: torch.Tensor | None = None):
        if not 1 <= streams <= K.STREAMS_MAX:
            raise ValueError(f"{streams} residual streams; 1..{K.STREAMS_MAX} are supported")
        if read is not None and read.numel() != streams:
            raise ValueError(f"the read weights have {read.numel()} entries for {streams} streams")
        self.weight = None if weight is None else weight.to(torch.float32).contiguous()
        self.read = None if read is None else read.to(torch.float32).contiguous()
        self.eps, self.streams = float(eps), int(streams)

    def forward(self, ctx: StepContext, x, delta, *, out_dtype, want_f32=False, row_index=None, router=None):
        from .base import StreamMixed

        if delta is not None and not isinstance(delta, StreamMixed):
            raise TypeError("a norm over several residual streams adds sublayer outputs that come with their mix and write weights")
        n = x.shape[0] if row_index is None else row_index.numel()
        D = x.shape[1] // self.streams
        out = None if out_dtype is None else torch.empty((n, D), dtype=out_dtype, device=x.device)
        out32 = torch.empty((n, D), dtype=torch.float32, device=x.device) if want_f32 else None
        first = ctx.scratch.pop("streams_start", None)  # the embedding's rows, while the streams are still unwritten
        rows = None if delta is None else delta.rows
        K.stream_mix_norm(x, self.streams, first=first, y=None if rows is None else rows.data, y_splits=1 if rows is None else rows.splits,
                          mix=None if delta is None else delta.mix, write=None if delta is None else delta.write, read=self.read,
                          gamma=self.weight, eps=self.eps, out=out, out32=out32, row_index=row_index,
                          sum_out=ctx.scratch.get("stream_sum_probe"))
        return out, out32, None


register_part("norm", "stream_rms", StreamRMSNorm)
