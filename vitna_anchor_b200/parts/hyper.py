"""Residual streams joined by hyper-connections.

A token has `streams` residual rows X_0..X_{s-1} instead of one, all equal to the embedding at the start.  A sublayer
f (a mixer or a feed-forward) with a norm w and the weights a [s] (in), M [s, s] (mix, indexed [from, to]) and b [s]
(out) reads one combination of the rows and writes to all of them:

    u = sum_i a_i X_i;    y = f(rms(u) * w);    X_j <- sum_i M[i, j] X_i + b_j y    (every j from the old rows)

The model's output is the sum of the rows.  On the device the rows are one float32 tensor [tokens, s * width].  What
lies between two sublayers is one kernel (ops.hyper_step): the update of the sublayer that has just run, then the next
sublayer's u, normed.  So a block leaves its last update PENDING in the step's context, and the next block's first
step, or the sum at the end, applies it.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..cache.manager import LayerCacheView
from .base import Block, FeedForward, Mixer, Norm, Part, StepContext

_PENDING = "hyper.pending"


class HyperConnection(Part):
    """The weights of one sublayer's connection to the streams."""

    def __init__(self, streams: int, w_in: torch.Tensor, w_mix: torch.Tensor, w_out: torch.Tensor):
        if w_in.shape != (streams,) or w_mix.shape != (streams, streams) or w_out.shape != (streams,):
            raise ValueError("hyper-connection weights do not fit the number of streams")
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.streams, self.w_in, self.w_mix, self.w_out = streams, f32(w_in), f32(w_mix), f32(w_out)

    def tensors(self):
        return [self.w_in, self.w_mix, self.w_out]


def _step(xs: torch.Tensor, ctx: StepContext, streams: int, nxt: Optional[Tuple[HyperConnection, Norm]], sum_out=None):
    """Apply the pending update, if any, and form the next sublayer's normed input (or the sum of the rows)."""
    T, width = xs.shape[0], xs.shape[1] // streams
    y = ctx.workspace.rows("hyper.y", T, width, torch.float32)
    done: Optional[HyperConnection] = ctx.extra.pop(_PENDING, None)
    xn = None
    kw = {}
    if nxt is not None:
        hc, norm = nxt
        nw, eps = norm.as_rms()
        xn = ctx.workspace.rows("block.xn", T, width, ctx.dtype)
        kw = dict(in_w=hc.w_in, norm_w=nw, eps=eps, xn=xn)
    ops.hyper_step(xs, y, streams, mix=None if done is None else done.w_mix, out_w=None if done is None else done.w_out,
                   sum_out=sum_out, **kw)
    return xn, y


class HyperBlock(Block):
    """x has `streams` rows a token; the mixer and (if there is one) the feed-forward each read and write them through a
    connection of their own."""

    def __init__(self, streams: int, mixer_norm: Norm, mixer_hc: HyperConnection, mixer: Mixer, ffn_norm: Optional[Norm] = None,
                 ffn_hc: Optional[HyperConnection] = None, ffn: Optional[FeedForward] = None):
        if mixer_norm.as_rms() is None or (ffn is not None and (ffn_norm is None or ffn_hc is None or ffn_norm.as_rms() is None)):
            raise ValueError("a hyper-connected sublayer needs a norm of the RMS form and a connection")
        self.streams = streams
        self.mixer_norm, self.mixer_hc, self.mixer = mixer_norm, mixer_hc, mixer
        self.ffn_norm, self.ffn_hc, self.ffn = ffn_norm, ffn_hc, ffn

    def tensors(self):
        parts: Sequence[Optional[Part]] = (self.mixer_norm, self.mixer_hc, self.mixer, self.ffn_norm, self.ffn_hc, self.ffn)
        return [t for p in parts if p is not None for t in p.tensors()]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], write_cache: bool = True) -> None:
        xn, y = _step(x, ctx, self.streams, (self.mixer_hc, self.mixer_norm))
        self.mixer.forward(xn, ctx, cache, y, write_cache)
        ctx.extra[_PENDING] = self.mixer_hc
        if self.ffn is not None:
            xn, y = _step(x, ctx, self.streams, (self.ffn_hc, self.ffn_norm))
            self.ffn.forward(xn, ctx, y)
            ctx.extra[_PENDING] = self.ffn_hc


class StreamSum(Part):
    """Ends a model with residual streams: the last pending update, then the sum of the rows as one float32 row a token."""

    def __init__(self, streams: int):
        self.streams = streams

    def forward(self, xs: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, width = xs.shape[0], xs.shape[1] // self.streams
        out = ctx.workspace.rows("hyper.sum", T, width, torch.float32)
        _step(xs, ctx, self.streams, None, sum_out=out)
        return out
