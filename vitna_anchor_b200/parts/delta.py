"""The gated delta rule: a recurrent mixer whose memory is a matrix per head instead of a cache of keys.

With G key heads of size dk, H value heads of size dv (value head h reads key head h // (H / G)) and a short causal
convolution of `taps` weights per channel:

    q, k, v = silu(conv(W_q xn)), silu(conv(W_k xn)), silu(conv(W_v xn))
    q, k    scaled to unit length per head (sqrt(sum x^2 + 1e-6)), q also by dk^-1/2
    beta    = sigmoid(W_b xn)                                   one per value head
    decay   = exp(-exp(A_log) * softplus(W_a xn + dt_bias))     one per value head
    per head, token after token:   S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out     = W_o (o / rms(o) * w_norm * silu(W_g xn))          rms over dv, w_norm [dv] shared by the heads

The six projections are ONE product over their matrices stacked by rows, with float32 results; everything after it is
float32 until the input of the output projection.  A request's state (S of every head, and the last taps-1 inputs of
the convolution) lives in the request's state slot and is carried from step to step, so a prompt may be cut anywhere.
All launches depend on the step's counts and device arrays alone: the part is replayed faithfully from a graph.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import LayerCacheView, StateSpec
from .base import Mixer, StepContext


class GatedDeltaRule(Mixer):
    CHUNKED_FROM = 64       # steps of more tokens than this run the recurrence in chunks

    def __init__(self, hidden: int, num_heads: int, num_key_heads: int, key_dim: int, value_dim: int, taps: int, w_in: torch.Tensor,
                 conv: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, norm_weight: torch.Tensor, wo: torch.Tensor, eps: float):
        """w_in: the projections stacked by rows, q | k | v | g | b | a ([2 G dk + 2 H dv + 2 H, hidden], compute dtype);
        conv float32 [2 G dk + H dv, taps], the q, k and v channels in that order, the last column the current token's."""
        if num_heads % num_key_heads:
            raise ValueError("value heads do not divide into key heads")
        H, G, dk, dv = num_heads, num_key_heads, key_dim, value_dim
        C = 2 * G * dk + H * dv
        if w_in.shape != (C + H * dv + 2 * H, hidden) or conv.shape != (C, taps) or wo.shape != (hidden, H * dv):
            raise ValueError("the delta rule's weights do not fit the head counts")
        if a_log.shape != (H,) or dt_bias.shape != (H,) or norm_weight.shape != (dv,):
            raise ValueError("the delta rule's per-head vectors do not fit the head counts")
        self.hidden, self.H, self.G, self.dk, self.dv, self.taps, self.eps = hidden, H, G, dk, dv, int(taps), float(eps)
        self.w_in, self.wo = w_in.contiguous(), wo.contiguous()
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.conv, self.a_log, self.dt_bias, self.norm_weight = f32(conv), f32(a_log), f32(dt_bias), f32(norm_weight)
        self.channels = C

    def tensors(self):
        return [self.w_in, self.conv, self.a_log, self.dt_bias, self.norm_weight, self.wo]

    def cache_spec(self):
        return StateSpec((ops.delta_state_floats(self.G, self.H, self.dk, self.dv, self.taps),), torch.float32)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if not write_cache:
            raise ValueError("a recurrent mixer has no cache that another run could read")
        T, ws = ctx.num_tokens, ctx.workspace
        proj = ops.linear(xn, self.w_in, ws.rows("delta.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        # a prompt's step takes the chunked form (the exact 32-bit routing keeps one kernel for every step)
        scratch = None
        if (T > self.CHUNKED_FROM and not (ctx.dtype == torch.float32 and ops.float32_exact())
                and ops.delta_chunked_takes(self.G, self.H, self.dk, self.dv, self.taps)):
            scratch = ws.flat(f"delta.chunks/{self.H}/{self.dk}/{self.dv}",
                              ops.delta_chunked_scratch_floats(ws.max_tokens, ws.max_segments, self.H, self.dk, self.dv), torch.float32)
        out = ops.delta_rule(proj, self.conv, self.a_log, self.dt_bias, self.norm_weight, self.eps, ctx.token_seg, ctx.seg_starts,
                             ctx.seg_slots, cache.state, ws.rows("delta.prep", T, ops.delta_prep_width(self.G, self.H, self.dk, self.dv), torch.float32),
                             ws.rows("delta.o", T, self.H * self.dv, torch.float32), ws.rows("delta.out", T, self.H * self.dv, ctx.dtype),
                             self.G, self.H, self.dk, self.dv, self.taps, chunk_scratch=scratch,
                             single_tokens=ctx.decode_only and not (ctx.dtype == torch.float32 and ops.float32_exact()))
        ops.linear(out, self.wo, residual, ops.LINEAR_ACC_F32)


class ChannelDeltaRule(Mixer):
    """The delta rule whose decay differs by head AND key channel, behind two low-rank projections:

        q, k, v, beta   as in GatedDeltaRule
        decay   = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 xn) + dt_bias))      [H, dk]: the rows of S decay at rates of their own
        per head, token after token:   S <- diag(decay) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
        out     = W_o (o / rms(o) * w_norm * sigmoid(W_g2 (W_g1 xn)))

    ONE product makes q | k | v | b | W_a1 xn | W_g1 xn with float32 results; the wide halves W_a2 and W_g2 are applied in float32
    inside the kernel that prepares the recurrence.  The state and its slot are GatedDeltaRule's.  Single decoded tokens take ONE
    kernel for all of it in the serving routings (the exact 32-bit routing keeps one set of kernels for every step)."""

    def __init__(self, hidden: int, num_heads: int, num_key_heads: int, key_dim: int, value_dim: int, taps: int, w_in: torch.Tensor,
                 conv: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, w_a2: torch.Tensor, w_g2: torch.Tensor,
                 norm_weight: torch.Tensor, wo: torch.Tensor, eps: float):
        """w_in: q | k | v | b | a1 | g1 stacked by rows ([2 G dk + H dv + H + ra + rg, hidden], compute dtype); w_a2 [H dk, ra] and
        w_g2 [H dv, rg] (kept in float32, transposed); conv float32 [2 G dk + H dv, taps]; dt_bias [H dk]."""
        if num_heads % num_key_heads:
            raise ValueError("value heads do not divide into key heads")
        H, G, dk, dv = num_heads, num_key_heads, key_dim, value_dim
        C = 2 * G * dk + H * dv
        if w_a2.dim() != 2 or w_g2.dim() != 2 or w_a2.shape[0] != H * dk or w_g2.shape[0] != H * dv:
            raise ValueError("the delta rule's low-rank projections do not fit the head counts")
        ra, rg = w_a2.shape[1], w_g2.shape[1]
        if w_in.shape != (C + H + ra + rg, hidden) or conv.shape != (C, taps) or wo.shape != (hidden, H * dv):
            raise ValueError("the delta rule's weights do not fit the head counts")
        if a_log.shape != (H,) or dt_bias.shape != (H * dk,) or norm_weight.shape != (dv,):
            raise ValueError("the delta rule's per-head vectors do not fit the head counts")
        self.hidden, self.H, self.G, self.dk, self.dv, self.taps, self.eps = hidden, H, G, dk, dv, int(taps), float(eps)
        self.w_in, self.wo = w_in.contiguous(), wo.contiguous()
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.conv, self.a_log, self.dt_bias, self.norm_weight = f32(conv), f32(a_log), f32(dt_bias), f32(norm_weight)
        self.a2t, self.g2t = f32(w_a2.to(torch.float32).t()), f32(w_g2.to(torch.float32).t())

    def tensors(self):
        return [self.w_in, self.conv, self.a_log, self.dt_bias, self.a2t, self.g2t, self.norm_weight, self.wo]

    def cache_spec(self):
        return StateSpec((ops.delta_state_floats(self.G, self.H, self.dk, self.dv, self.taps),), torch.float32)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if not write_cache:
            raise ValueError("a recurrent mixer has no cache that another run could read")
        T, ws = ctx.num_tokens, ctx.workspace
        proj = ops.linear(xn, self.w_in, ws.rows("cdelta.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        serving = not (ctx.dtype == torch.float32 and ops.float32_exact())
        # a prompt's step takes the chunked form (the exact 32-bit routing keeps one set of kernels for every step)
        scratch = None
        if T > GatedDeltaRule.CHUNKED_FROM and serving and ops.delta_chunked_takes(self.G, self.H, self.dk, self.dv, self.taps):
            scratch = ws.flat(f"cdelta.chunks/{self.H}/{self.dk}/{self.dv}",
                              ops.channel_delta_chunked_scratch_floats(ws.max_tokens, ws.max_segments, self.H, self.dk, self.dv), torch.float32)
        out = ops.channel_delta_rule(proj, self.conv, self.a_log, self.dt_bias, self.a2t, self.g2t, self.norm_weight, self.eps, ctx.token_seg,
                                     ctx.seg_starts, ctx.seg_slots, cache.state,
                                     ws.rows("cdelta.prep", T, ops.channel_delta_prep_width(self.G, self.H, self.dk, self.dv), torch.float32),
                                     ws.flat(f"cdelta.groups/{self.H}/{self.dk}", ops.channel_delta_group_floats(ws.max_tokens, self.H, self.dk),
                                             torch.float32),
                                     ws.rows("delta.o", T, self.H * self.dv, torch.float32), ws.rows("delta.out", T, self.H * self.dv, ctx.dtype),
                                     self.G, self.H, self.dk, self.dv, self.taps, single_tokens=ctx.decode_only and serving, chunk_scratch=scratch)
        ops.linear(out, self.wo, residual, ops.LINEAR_ACC_F32)
