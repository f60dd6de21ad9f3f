"""Mixers that keep a matrix state per head, decayed channel by channel: linear attention as a recurrence.

Both mixers here share one recurrence, S_t = diag(d_t) S_(t-1) + k_t v_t^T with a decay d_t in (0, 1) per key channel
that depends on the token, and one set of kernels (``csrc/decay_scan.cu``); they differ in where the decay comes from,
in when the state is read, and in what surrounds the recurrence.  Decays, state, norms and gates are float32 in both
precisions; bfloat16 rounding happens at the operands of the matrix products only.
"""

from __future__ import annotations

import torch

from ..kernels import api as K
from ..tracing import scope
from .base import LayerCache, Mixer, ProjectedMixer, Rows, StateNeed, StepContext, as_rows, register_part
from .linear import grouped_linear, linear


def _scan(ctx: StepContext, q, k, v, z, z_bias, form: str, tau: float, q_scale: float, bonus, state, heads: int, dk: int, dv: int,
          read_after_update: bool, **prep) -> torch.Tensor:
    """The recurrence over the step's tokens from projected rows (views); returns o float32 [N, H, dv]."""
    n, dev = ctx.n_tokens, state.device
    need = n * heads * (3 * dk + 2 * dv)
    buf = ctx.workspace.get("decay_scan", need, torch.float32) if ctx.workspace is not None else torch.empty(need, dtype=torch.float32, device=dev)
    at = 0

    def cut(*shape):
        nonlocal at
        size = 1
        for s in shape:
            size *= s
        t = buf[at:at + size].view(*shape)
        at += size
        return t

    qo, ko, do, vo, o = cut(n, heads, dk), cut(n, heads, dk), cut(n, heads, dk), cut(n, heads, dv), cut(n, heads, dv)
    K.decay_prep(q, k, v, z, z_bias, form, tau, q_scale, qo, ko, do, vo, heads, dk, dv, **prep)
    K.decay_scan(qo, ko, do, vo, bonus, state, ctx.cu_q, ctx.slot_ids, o, read_after_update)
    return o


class GatedLinearAttention(ProjectedMixer):
    """q = W_q h / sqrt(dk), k = W_k h, v = W_v h; a decay per key channel alpha = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau);
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's o is RMS-normed over dv with a weight shared
    by the heads, multiplied by silu(W_g h) and sent through W_o.

    ``w_in``: [2 H dk + 2 H dv, D] = the q, k, v and gate projections stacked in that order; ``w_a1``: [rank, D];
    ``w_a2``: [H dk, rank]; ``a_bias``: [H dk].  State: float32 [H, dk, dv] per request."""

    kernel_libraries = ("decay_scan", "gemm_simt", "group_norm")
    kernel_libraries_bf16 = ("gemm_stream",)

    def __init__(self, w_in: torch.Tensor, w_a1: torch.Tensor, w_a2: torch.Tensor, a_bias: torch.Tensor, norm_weight: torch.Tensor,
                 w_o: torch.Tensor, heads: int, dim: int, vdim: int, tau: float, eps: float):
        if w_in.shape[0] != 2 * heads * (dim + vdim) or w_o.shape[1] != heads * vdim or w_a2.shape != (heads * dim, w_a1.shape[0]) \
                or a_bias.numel() != heads * dim or norm_weight.numel() != vdim or w_a1.shape[1] != w_in.shape[1]:
            raise ValueError(f"gated linear attention weights do not fit {heads} heads of {dim} x {vdim}: w_in {tuple(w_in.shape)}, "
                             f"a1 {tuple(w_a1.shape)}, a2 {tuple(w_a2.shape)}, o {tuple(w_o.shape)}")
        if tau <= 0:
            raise ValueError("tau must be positive")
        self.w_in, self.w_a1, self.w_a2, self.w_o = w_in, w_a1.contiguous(), w_a2.contiguous(), w_o
        self.a_bias, self.norm_weight = a_bias.to(torch.float32).contiguous(), norm_weight.to(torch.float32).contiguous()
        self.heads, self.dim, self.vdim, self.tau, self.eps = heads, dim, vdim, float(tau), float(eps)

    def state_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def core(self, ctx: StepContext, h, proj: Rows, col: int, cache: LayerCache, out: torch.Tensor, mult: float) -> None:
        H, dk, dv = self.heads, self.dim, self.vdim
        with scope("qkv_matmul"):  # the decay's two small products
            a1 = linear(ctx, h, self.w_a1, ctx.runtime.dtype)
            z = as_rows(linear(ctx, a1, self.w_a2, torch.float32, partials=True))
        view = lambda c: K.rows_view(proj.data, proj.splits, col + c)  # noqa: E731
        with scope("attention"):
            o = _scan(ctx, view(0), view(H * dk), view(2 * H * dk), K.rows_view(z.data, z.splits), self.a_bias, "sigmoid_power",
                      self.tau, float(dk) ** -0.5, None, cache.state, H, dk, dv, True)
            K.head_norm_gate(o, self.norm_weight, False, view(2 * H * dk + H * dv), self.eps, mult, out)


class TimeMixWKV(Mixer):
    """RWKV-style time mixing with a data-dependent decay.  With h' the previous token's input (zeros before the first),
    each of r, k, v, g, w reads its own blend  h + (h' - h) * mu_s;  r, k, v = W_r, W_k, W_v of their blends (H heads of
    dk), gate = silu(W_g blend_g), decay w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0)) per head and key channel;

        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_(t-1) + k_t v_t^T;

    each head's o is divided by its root mean square, the heads are multiplied by ``norm_weight`` [H dk] and the gate
    and go through W_o.

    ``mu``: [5, D] in the order r, k, v, g, w.  ``w_rkvg``: [4, H dk, D].  ``w_w1``: [rank, D]; ``w_w2``: [H dk, rank];
    ``w0``: [H dk]; ``bonus``: [H, dk].  State: the previous input, float32 [D], and S, float32 [H, dk, dk]."""

    kernel_libraries = ("decay_scan", "gemm_simt", "group_norm")
    kernel_libraries_bf16 = ("gemm_stream",)
    needs_f32_input = True
    OVERLAP_MAX_ROWS = 256

    def __init__(self, mu: torch.Tensor, w_rkvg: torch.Tensor, w_w1: torch.Tensor, w_w2: torch.Tensor, w0: torch.Tensor,
                 bonus: torch.Tensor, norm_weight: torch.Tensor, w_o: torch.Tensor, heads: int, dim: int, eps: float):
        D, F = w_o.shape[0], heads * dim
        if tuple(mu.shape) != (5, D) or tuple(w_rkvg.shape) != (4, F, D) or w_w1.shape[1] != D or tuple(w_w2.shape) != (F, w_w1.shape[0]) \
                or w0.numel() != F or bonus.numel() != F or norm_weight.numel() != F or w_o.shape[1] != F:
            raise ValueError(f"time-mix weights do not fit {heads} heads of {dim} at width {D}: mu {tuple(mu.shape)}, rkvg "
                             f"{tuple(w_rkvg.shape)}, w1 {tuple(w_w1.shape)}, w2 {tuple(w_w2.shape)}, o {tuple(w_o.shape)}")
        f32 = lambda t: t.to(torch.float32).contiguous()  # noqa: E731
        self.mu, self.w0, self.bonus, self.norm_weight = f32(mu), f32(w0), f32(bonus).view(heads, dim), f32(norm_weight)
        self.w_rkvg, self.w_w1, self.w_w2, self.w_o = w_rkvg.contiguous(), w_w1.contiguous(), w_w2.contiguous(), w_o
        self.heads, self.dim, self.eps, self.width = heads, dim, float(eps), D

    def state_needs(self):
        return (StateNeed((self.width,), torch.float32), StateNeed((self.heads, self.dim, self.dim), torch.float32))

    def forward(self, ctx: StepContext, h, cache: LayerCache, h32: torch.Tensor | None = None):
        n, D = h32.shape
        H, dk, F = self.heads, self.dim, self.heads * self.dim
        dt = ctx.runtime.dtype
        shift_state, S = cache.states
        blends = torch.empty((5, n, D), dtype=dt, device=h32.device)
        offsets = torch.empty(6, dtype=torch.int32, device=h32.device)  # row offsets of the blends: the groups of the product below
        K.token_shift_blend(h32, self.mu, shift_state, ctx.cu_q, ctx.slot_ids, ctx.req_of_token, blends, offsets)
        def decay_logits():
            w1 = as_rows(linear(ctx, blends[4], self.w_w1, torch.float32, partials=True))
            lora = torch.empty((n, self.w_w1.shape[0]), dtype=dt, device=h32.device)
            K.bias_act(w1.data, lora, None, None, "tanh", w1.splits)
            return as_rows(linear(ctx, lora, self.w_w2, torch.float32, partials=True))

        with scope("qkv_matmul"):
            # In steps of few rows the decay's three small launches run on the second stream beside the projections
            # (a branch of a captured graph): the chain of dependent launches is shorter by them.
            side = None
            if ctx.workspace is not None and h32.is_cuda and n <= self.OVERLAP_MAX_ROWS:
                main, side = torch.cuda.current_stream(), ctx.workspace.side_stream()
                side.wait_stream(main)  # the blends are there
                with torch.cuda.stream(side):
                    z = decay_logits()
                z.data.record_stream(main)  # made on the second stream, read (and freed) on the step's own
            # the four projections, each of its own blend, as one grouped product over the stacked rows
            rkvg = as_rows(grouped_linear(ctx, blends[:4].view(4 * n, D), self.w_rkvg, offsets,
                                          torch.float32, partials=True, largest_group=n))
            if side is None:
                z = decay_logits()
            else:
                torch.cuda.current_stream().wait_stream(side)
        view = lambda i: K.rows_view(rkvg.data, rkvg.splits, 0, i * n)  # noqa: E731
        out = torch.empty((n, F), dtype=dt, device=h32.device)
        with scope("attention"):
            o = _scan(ctx, view(0), view(1), view(2), K.rows_view(z.data, z.splits), self.w0, "double_exp", 1.0, 1.0, self.bonus,
                      S, H, dk, dk, False)
            K.head_norm_gate(o, self.norm_weight, True, view(3), self.eps, 1.0, out)
        with scope("projection"):
            return linear(ctx, out, self.w_o, torch.float32, partials=True)


class RetentionMixer(ProjectedMixer):
    """Linear attention with ONE fixed decay per head and neither softmax nor denominator:

        q = W_q h, k = W_k h (H heads of dk), v = W_v h (H heads of dv); q and k turned by the token's position on their
        first ``rot_dims`` entries (entry i with i + rot_dims / 2, angle position * inv_freq[i]); k times ``k_scale``;
        S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;
        each head's o divided by its root mean square (no weight), times silu(W_g h), through W_o.

    ``w_in``: [2 H dk + 2 H dv, D] = the q, k, v and gate projections stacked in that order; ``decay``: [H] numbers in
    (0, 1].  State: float32 [H, dk, dv] per request, zero at the start.  The recurrence is the decay-scan kernel's with
    a decay that is the same for every key channel of a head and every token."""

    kernel_libraries = ("decay_scan", "gemm_simt")
    kernel_libraries_bf16 = ("gemm_stream",)

    def __init__(self, w_in: torch.Tensor, w_o: torch.Tensor, decay: torch.Tensor, heads: int, dim: int, vdim: int, eps: float,
                 k_scale: float = 1.0, q_scale: float = 1.0, inv_freq: torch.Tensor | None = None, rot_dims: int = 0):
        if w_in.shape[0] != 2 * heads * (dim + vdim) or w_o.shape[1] != heads * vdim or w_o.shape[0] != w_in.shape[1] or decay.numel() != heads:
            raise ValueError(f"retention weights do not fit {heads} heads of {dim} x {vdim}: w_in {tuple(w_in.shape)}, o {tuple(w_o.shape)}, "
                             f"{decay.numel()} decays")
        if rot_dims % 2 or not 0 <= rot_dims <= dim or (rot_dims and (inv_freq is None or inv_freq.numel() != rot_dims // 2)):
            raise ValueError(f"{rot_dims} rotated entries of {dim} need {rot_dims // 2} frequencies")
        self.w_in, self.w_o = w_in, w_o
        self.decay = decay.to(torch.float32).contiguous()
        self.inv_freq = None if inv_freq is None else inv_freq.to(torch.float32).contiguous()
        self.heads, self.dim, self.vdim, self.eps = heads, dim, vdim, float(eps)
        self.k_scale, self.q_scale, self.rot_dims = float(k_scale), float(q_scale), int(rot_dims)

    def state_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def core(self, ctx: StepContext, h, proj: Rows, col: int, cache: LayerCache, out: torch.Tensor, mult: float) -> None:
        H, dk, dv = self.heads, self.dim, self.vdim
        view = lambda c: K.rows_view(proj.data, proj.splits, col + c)  # noqa: E731
        with scope("attention"):
            o = _scan(ctx, view(0), view(H * dk), view(2 * H * dk), None, None, "head_constant", 1.0, self.q_scale, None, cache.state,
                      H, dk, dv, True, head_decay=self.decay, k_scale=self.k_scale, inv_freq=self.inv_freq, rot_dims=self.rot_dims,
                      positions=ctx.positions)
            K.head_norm_gate(o, None, False, view(2 * H * dk + H * dv), self.eps, mult, out)


register_part("mixer", "retention", RetentionMixer)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "time_mix_wkv", TimeMixWKV)
