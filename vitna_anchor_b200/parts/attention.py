"""Causal grouped-query attention over the paged cache.

q = Wq xn, k = Wk xn, v = Wv xn (one product over the three matrices stacked
by rows); q and k heads are rotated by the position encoding's tables; k and v
go into the request's pages; every query reads keys 0..its own position (or
the last `window` of them) of its request; the heads are concatenated and the
output projection is added into the residual stream
(engine/src/model.c:912-959).  Query head h reads key-value head
h // (heads / kv_heads); scale = 1/sqrt(head_dim) unless given.

The unrotated form.  A mixer built with any of `v_dim`, `qk_norm_eps`, `q_temp` or `dist_bias` takes positions in
other ways than a rotation (its position encoding must give no tables):

  v_dim         values of another size than the keys; the output projection then reads heads * v_dim columns
  qk_norm_eps   every q and k head is divided by its root mean square, sqrt(mean(x^2) + eps), without a weight
  q_temp        (coef, every): the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1), so that
                the softmax stays as sharp as the context grows
  dist_bias     float32 [distances, heads]: row min(p - j, last) is added to the scaled score of query p and key j
                (`bucketed_distance_bias` spreads a small learned table over the distances)
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache.manager import KVSpec, LayerCacheView
from .base import Mixer, PositionEncoding, StepContext


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of a table of `rows` distance biases for the distance n >= 0: the first rows/2 distances have a row each; the
    other rows widen geometrically so that the last one begins at the distance `far`:
    rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2)), at most rows - 1."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def bucketed_distance_bias(table: torch.Tensor, far: int, distances: int) -> torch.Tensor:
    """float32 [distances, heads]: the learned table [rows, heads] laid out by distance (see distance_bucket), on the
    table's device.  The buckets are worked out once, on the host."""
    rows = table.shape[0]
    if rows < 2 or far <= rows // 2:
        raise ValueError("a table of distance biases needs two rows or more and a far distance beyond its exact rows")
    idx = torch.tensor([distance_bucket(n, rows, far) for n in range(distances)], dtype=torch.long, device=table.device)
    return table.to(torch.float32).index_select(0, idx).contiguous()


class PagedAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, wqkv: torch.Tensor,
                 wo: torch.Tensor, position: Optional[PositionEncoding], window: int = 0, scale: Optional[float] = None, *,
                 v_dim: Optional[int] = None, qk_norm_eps: Optional[float] = None, q_temp: Optional[tuple] = None,
                 dist_bias: Optional[torch.Tensor] = None):
        if num_heads % num_kv_heads:
            raise ValueError("heads do not divide into key-value groups")
        self.vd = int(v_dim) if v_dim else head_dim
        qd, kvd = num_heads * head_dim, num_kv_heads * head_dim
        if wqkv.shape != (qd + kvd + num_kv_heads * self.vd, hidden) or wo.shape != (hidden, num_heads * self.vd):
            raise ValueError("attention weights do not fit the head counts")
        self.hidden, self.nh, self.nkv, self.hd = hidden, num_heads, num_kv_heads, head_dim
        self.qd, self.kvd = qd, kvd
        self.unrotated = v_dim is not None or qk_norm_eps is not None or q_temp is not None or dist_bias is not None
        if self.unrotated and position is not None and position.rotary_tables() is not None:
            raise ValueError("the unrotated form of the attention takes no rotation tables")
        self.qk_norm_eps = -1.0 if qk_norm_eps is None else float(qk_norm_eps)
        self.q_coef, self.q_every = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else (0.0, 1)
        if dist_bias is not None and (dist_bias.dim() != 2 or dist_bias.shape[1] != num_heads or dist_bias.dtype != torch.float32):
            raise ValueError("the distance bias is not a float32 [distances, heads] table")
        self.dist_bias = None if dist_bias is None else dist_bias.contiguous()
        self.wqkv, self.wo = wqkv.contiguous(), wo.contiguous()
        self.position = position
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))

    def tensors(self):
        return [self.wqkv, self.wo]

    def cache_spec(self):
        return KVSpec(self.nkv, self.hd, self.window, self.vd if self.vd != self.hd else 0)

    def fuses_norm(self, norm, ctx: StepContext) -> bool:
        return (not self.unrotated and norm.as_rms() is not None
                and ops.fused_norm_takes(ctx.dtype, ctx.num_tokens, self.hidden, self.qd + 2 * self.kvd))

    def _forward_unrotated(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool) -> None:
        """Projections; unit-RMS q and k, the query's factor and the cache write in one launch; attention with the bias by
        distance; output projection."""
        T, ws = ctx.num_tokens, ctx.workspace
        meta = ctx.groups[cache.group]
        ps = ops._page_size_of(cache.pages, self.nkv, self.hd, self.vd)
        qkv = ops.linear(xn, self.wqkv, ws.rows("att.qkv", T, self.wqkv.shape[0], ctx.dtype), ops.LINEAR_SAME)
        q = ops.qk_norm_store(qkv, ctx.positions, meta.slot_mapping, ws.rows("att.q", T, self.qd, ctx.dtype),
                              cache.pages if write_cache else None, self.nh, self.nkv, self.hd, self.vd, ps, eps=self.qk_norm_eps,
                              q_coef=self.q_coef, q_every=self.q_every)
        att = ops.attention_biased(q, cache.pages, meta, ctx, ws.rows("att.out", T, self.nh * self.vd, ctx.dtype), self.nh, self.nkv,
                                   self.hd, self.vd, ps, self.scale, self.window, self.dist_bias)
        ops.linear(att, self.wo, residual, ops.LINEAR_ACC_F32)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor,
                write_cache: bool = True, norm=None) -> None:
        if self.unrotated:
            return self._forward_unrotated(xn, ctx, cache, residual, write_cache)
        T = ctx.num_tokens
        ws = ctx.workspace
        meta = ctx.groups[cache.group]
        tables = self.position.rotary_tables() if self.position is not None else None
        cos, sin, rot = tables if tables is not None else (None, None, 0)
        q_buf = ws.rows("att.q", T, self.qd, ctx.dtype)
        if norm is not None and rot == self.hd and write_cache:
            # few rows: norm, the three projections, the rotation and the cache write in one launch
            nw, eps = norm.as_rms()
            q = ops.linear_skinny(xn, self.wqkv, q_buf, ops.EPI_ROPE, norm_weight=nw, eps=eps,
                                  rope=(ctx.positions, cos, sin, meta.slot_mapping, cache.pages, self.nh, self.nkv, self.hd))
        elif (norm is None and rot == self.hd and write_cache and xn.stride(0) % 8 == 0 and xn.data_ptr() % 16 == 0
              and ops.skinny_takes(ctx.dtype, T, self.hidden, self.qd + 2 * self.kvd)):
            # a few dozen rows: the norm ran once for all of them; projections, rotation and cache write in one launch
            q = ops.linear_skinny(xn, self.wqkv, q_buf, ops.EPI_ROPE,
                                  rope=(ctx.positions, cos, sin, meta.slot_mapping, cache.pages, self.nh, self.nkv, self.hd))
        elif (norm is None and T > ops.SKINNY_MAX_ROWS and rot == self.hd and self.hd in (64, 128) and write_cache
              and ops.tcgen05_takes(xn, self.wqkv)):
            # prompt-sized batch in bfloat16: the projections, the rotation and the cache write in one tcgen05 kernel
            q = ops.linear_tcgen05_rope(xn, self.wqkv, q_buf, ctx.positions, cos, sin, meta.slot_mapping, cache.pages, self.nh,
                                        self.nkv, self.hd)
        else:
            qkv_buf = ws.rows("att.qkv", T, self.qd + 2 * self.kvd, ctx.dtype)
            if norm is not None:
                nw, eps = norm.as_rms()
                qkv = ops.linear_skinny(xn, self.wqkv, qkv_buf, ops.EPI_SAME, norm_weight=nw, eps=eps)
            else:
                qkv = ops.linear(xn, self.wqkv, qkv_buf, ops.LINEAR_SAME)
            q = ops.rope_store(qkv, ctx.positions, cos, sin, meta.slot_mapping, q_buf, cache.pages if write_cache else None,
                               self.nh, self.nkv, self.hd, rot, cache.pages.shape[3])
        att = ops.attention(q, cache.pages, meta, ctx, ws.rows("att.out", T, self.qd, ctx.dtype), self.nh, self.nkv,
                            self.hd, self.scale, self.window)
        ops.linear(att, self.wo, residual, ops.LINEAR_ACC_F32)
