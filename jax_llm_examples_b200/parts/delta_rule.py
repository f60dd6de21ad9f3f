"""The gated delta rule: a mixer whose matrix state is corrected, not just added to.

Per head, with a decay g in (0, 1) for the whole state and a step size beta in (0, 1), both from the token:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

(the read-out sees the token's own write).  The state is asked to return v when read with k; how far it is moved
towards that is beta.  q, k and v first pass a short causal convolution per channel and an activation; q and k are
then made unit vectors per head.  The convolution's sums, activations, unit norms, gates, decays, the state and every
sum over it are float32 in both precisions; bfloat16 rounding happens at the operands of the matrix products only.
"""

from __future__ import annotations

import torch

from ..kernels import api as K
from ..tracing import scope
from .base import LayerCache, ProjectedMixer, Rows, StateNeed, StepContext, register_part


class GatedDeltaRule(ProjectedMixer):
    """q = W_q h and k = W_k h (G key heads of dk), v = W_v h (H heads of dv; head a reads key head a // (H / G)); each
    channel of q, k, v through a causal convolution over ``taps`` tokens and ``activation``; q and k divided by
    sqrt(sum x^2 + unit_eps), q times ``q_scale`` (default dk^-1/2); beta = sigmoid(W_b h);
    g = exp(-exp(rate_log) * softplus(W_a h + a_bias)); the recurrence above; each head's o divided by its root mean
    square over dv (``eps``), times ``norm_weight`` [dv] (shared by the heads), times silu(W_g h); then W_o.

    ``w_in``: [2 G dk + 2 H dv + 2 H, D] = the q, k, v, gate, beta and decay projections stacked in that order;
    ``conv_weight``: [2 G dk + H dv, taps] for the q, k, v channels in that order, the last column the current token's.
    State per request: the convolution's last taps - 1 inputs, float32 [taps - 1, 2 G dk + H dv] (if taps > 1), and S,
    float32 [H, dk, dv]."""

    kernel_libraries = ("delta_rule", "decay_scan", "gemm_simt")
    kernel_libraries_bf16 = ("gemm_stream",)

    def __init__(self, w_in: torch.Tensor, conv_weight: torch.Tensor, rate_log: torch.Tensor, a_bias: torch.Tensor,
                 norm_weight: torch.Tensor, w_o: torch.Tensor, heads: int, key_heads: int, dim: int, vdim: int, eps: float,
                 activation: str = "silu", unit_eps: float = 1e-6, q_scale: float | None = None):
        C = 2 * key_heads * dim + heads * vdim
        if heads % key_heads:
            raise ValueError(f"{heads} heads are no multiple of {key_heads} key heads")
        if w_in.shape[0] != C + heads * vdim + 2 * heads or w_o.shape[1] != heads * vdim or w_o.shape[0] != w_in.shape[1] \
                or conv_weight.shape[0] != C or rate_log.numel() != heads or a_bias.numel() != heads or norm_weight.numel() != vdim:
            raise ValueError(f"delta-rule weights do not fit {heads} heads ({key_heads} key heads) of {dim} x {vdim}: w_in "
                             f"{tuple(w_in.shape)}, conv {tuple(conv_weight.shape)}, o {tuple(w_o.shape)}")
        if activation not in K.CONV_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is unknown ({', '.join(K.CONV_ACTIVATIONS)})")
        f32 = lambda t: t.to(torch.float32).contiguous()  # noqa: E731
        self.w_in, self.w_o = w_in, w_o
        self.conv_weight, self.rate_log, self.a_bias, self.norm_weight = f32(conv_weight), f32(rate_log), f32(a_bias), f32(norm_weight)
        self.heads, self.key_heads, self.dim, self.vdim = heads, key_heads, dim, vdim
        self.channels, self.taps = C, conv_weight.shape[1]
        self.eps, self.activation, self.unit_eps = float(eps), activation, float(unit_eps)
        self.q_scale = float(dim) ** -0.5 if q_scale is None else float(q_scale)

    def state_needs(self):
        conv = (StateNeed((self.taps - 1, self.channels), torch.float32),) if self.taps > 1 else ()
        return conv + (StateNeed((self.heads, self.dim, self.vdim), torch.float32),)

    def core(self, ctx: StepContext, h, proj: Rows, col: int, cache: LayerCache, out: torch.Tensor, mult: float) -> None:
        H, G, dk, dv, C = self.heads, self.key_heads, self.dim, self.vdim, self.channels
        conv_state, S = (cache.states[0], cache.states[1]) if self.taps > 1 else (None, cache.states[0])
        n, dev = proj.data.shape[-2], out.device
        need = n * (2 * G * K.DELTA_GROUP + 2 * G * dk + 2 * H * dv + 2 * H)
        buf = ctx.workspace.get("delta_rule", need, torch.float32) if ctx.workspace is not None else \
            torch.empty(need, dtype=torch.float32, device=dev)
        at = 0

        def cut(*shape):
            nonlocal at
            size = 1
            for s in shape:
                size *= s
            t = buf[at:at + size].view(*shape)
            at += size
            return t

        products = cut(n, G, 2 * K.DELTA_GROUP)  # first: it is copied 16 bytes at a time
        q, k, v, o = cut(n, G, dk), cut(n, G, dk), cut(n, H, dv), cut(n, H, dv)
        beta, decay = cut(n, H), cut(n, H)
        gate_col = col + C
        with scope("attention"):
            K.conv_unit_prep(K.rows_view(proj.data, proj.splits, col), C + H * dv, C + H * dv + H, self.conv_weight, conv_state,
                             self.rate_log, self.a_bias, ctx.cu_q, ctx.q_start, ctx.slot_ids, ctx.req_of_token, ctx.positions,
                             q, k, v, beta, decay, self.activation, self.unit_eps, self.q_scale)
            K.delta_scan(q, k, v, beta, decay, S, ctx.cu_q, ctx.slot_ids, o, ctx.req_of_token, products)
            K.head_norm_gate(o, self.norm_weight, False, K.rows_view(proj.data, proj.splits, gate_col), self.eps, mult, out)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
