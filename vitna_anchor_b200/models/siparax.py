"""The Siparax decoder: manifest of its tensors and how its layers are built from the engine's parts.

A small decoder-only language model whose layers each choose between latent attention (queries and keys/values through
narrow latents, one rotated key part shared by the heads, only the latent cached; two forms that differ in the rotation's
pairing, the second with a gate a head and, optionally, reading another layer's cached rows) and the delta rule with a
decay per head and key channel.  Every norm around the sublayers is a layer norm with weight and bias; the embedding is
normed before the first layer; the feed-forward is gated with the tanh form of gelu, or absent; the logits pass a soft cap.

Tensor names: embed, embed.norm(.b), final.norm(.b), head; layer i has l<i>.norm1(.b), l<i>.norm2(.b), l<i>.mix.* and
l<i>.mlp.{gate,up,down}.  Matrices are [out, in].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.siparax import ChannelDeltaSpec, SiparaxConfig
from ..parts.embedding import CappedLMHead, LMHead, NormedEmbedding
from ..parts.registry import make_part
from ..parts.rotary import blended_frequencies
from ..weights.loader import WeightSpec
from .decoder import DecoderModel, LayerRun

UNBOUNDED_POSITIONS = 1 << 24       # nothing of the model is a table over positions; float32 holds these exactly


def siparax_manifest(cfg: SiparaxConfig) -> List[WeightSpec]:
    W = cfg.width
    norm = lambda name: [WeightSpec(name, (W,)), WeightSpec(name + ".b", (W,))]
    m = [WeightSpec("embed", (cfg.vocab, W))] + norm("embed.norm")
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer.mixer
        m += norm(p + "norm1")
        if isinstance(mx, ChannelDeltaSpec):
            qk, v = mx.kv_heads * mx.dim, mx.heads * mx.vdim
            m += [WeightSpec(p + "mix.q", (qk, W)), WeightSpec(p + "mix.q.conv", (qk, mx.conv)),
                  WeightSpec(p + "mix.k", (qk, W)), WeightSpec(p + "mix.k.conv", (qk, mx.conv)),
                  WeightSpec(p + "mix.v", (v, W)), WeightSpec(p + "mix.v.conv", (v, mx.conv)),
                  WeightSpec(p + "mix.b", (mx.heads, W)), WeightSpec(p + "mix.A_log", (mx.heads,)), WeightSpec(p + "mix.norm", (mx.vdim,)),
                  WeightSpec(p + "mix.a1", (None, W), free_size=16), WeightSpec(p + "mix.a2", (mx.heads * mx.dim, None), free_size=16),
                  WeightSpec(p + "mix.dt_bias", (mx.heads * mx.dim,)),
                  WeightSpec(p + "mix.g1", (None, W), free_size=16), WeightSpec(p + "mix.g2", (v, None), free_size=16),
                  WeightSpec(p + "mix.o", (W, v))]
        else:
            H = mx.heads
            m += [WeightSpec(p + "mix.dq", (mx.q_rank, W)), WeightSpec(p + "mix.dq.norm", (mx.q_rank,)),
                  WeightSpec(p + "mix.uq", (H * (mx.dim + mx.rot_dim), mx.q_rank))]
            if mx.kv_from is None:
                m += [WeightSpec(p + "mix.dkv", (mx.kv_rank + mx.rot_dim, W)), WeightSpec(p + "mix.dkv.norm", (mx.kv_rank,))]
            m += [WeightSpec(p + "mix.uk", (H * mx.dim, mx.kv_rank)), WeightSpec(p + "mix.uv", (H * mx.vdim, mx.kv_rank))]
            if mx.gated:
                m.append(WeightSpec(p + "mix.g", (H, W)))
            m.append(WeightSpec(p + "mix.o", (W, H * mx.vdim)))
        if layer.mlp is not None:
            m += norm(p + "norm2")
            m += [WeightSpec(p + "mlp.gate", (layer.mlp.ff, W)), WeightSpec(p + "mlp.up", (layer.mlp.ff, W)),
                  WeightSpec(p + "mlp.down", (W, layer.mlp.ff))]
    m += norm("final.norm") + [WeightSpec("head", (cfg.vocab, W))]
    return m


def is_norm_weight(name: str) -> bool:
    """Tensors that random initialisation makes 1 + noise instead of noise around 0."""
    return name.rsplit(".", 1)[-1] in ("norm1", "norm2", "norm")


def build_siparax(cfg: SiparaxConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> DecoderModel:
    """Matrices go to the device in the compute dtype; norms, the delta rule's per-head vectors, its convolution weights and
    the wide halves of its low-rank projections are float32 in both paths."""
    dev = torch.device(device)
    W = cfg.width

    def mat(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=dtype) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def vec(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=torch.float32) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def norm(name: str):
        return make_part("norm", "layernorm", width=W, eps=cfg.eps, weight=vec(name), bias=vec(name + ".b"))

    blocks, cache_of = [], {}
    schedule: List[LayerRun] = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer.mixer
        if isinstance(mx, ChannelDeltaSpec):
            if weights[p + "mix.a1"].shape[0] != weights[p + "mix.a2"].shape[1] or weights[p + "mix.g1"].shape[0] != weights[p + "mix.g2"].shape[1]:
                raise ValueError(f"layer {i}: the two halves of a low-rank projection differ in rank")
            mixer = make_part("mixer", "channel_delta", hidden=W, num_heads=mx.heads, num_key_heads=mx.kv_heads, key_dim=mx.dim,
                              value_dim=mx.vdim, taps=mx.conv,
                              w_in=mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.b", p + "mix.a1", p + "mix.g1"),
                              conv=vec(p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv"), a_log=vec(p + "mix.A_log"),
                              dt_bias=vec(p + "mix.dt_bias"), w_a2=vec(p + "mix.a2"), w_g2=vec(p + "mix.g2"), norm_weight=vec(p + "mix.norm"),
                              wo=mat(p + "mix.o"), eps=cfg.eps)
            schedule.append(LayerRun(block=i, cache=i))
        else:
            freq, mag = blended_frequencies(mx.rot.base, mx.rot.dims, mx.rot.scaling)
            own = mx.kv_from is None
            mixer = make_part("mixer", "latent_attention", hidden=W, num_heads=mx.heads, dim=mx.dim, rot_dim=mx.rot_dim, v_dim=mx.vdim,
                              kv_rank=mx.kv_rank, q_rank=mx.q_rank, scale=mx.scale, eps=cfg.eps, w_dq=weights[p + "mix.dq"],
                              q_norm=weights[p + "mix.dq.norm"], w_uq=weights[p + "mix.uq"], w_dkv=weights[p + "mix.dkv"] if own else None,
                              kv_norm=weights[p + "mix.dkv.norm"] if own else None, w_uk=weights[p + "mix.uk"], w_uv=weights[p + "mix.uv"],
                              w_o=weights[p + "mix.o"], w_gate=weights[p + "mix.g"] if mx.gated else None, freq=freq, mag=mag,
                              rot_dims=mx.rot.dims, interleaved=mx.interleaved, dtype=dtype, device=dev)
            # a layer that reads another layer's rows runs on that layer's cache and does not write it
            schedule.append(LayerRun(block=i, cache=i if own else mx.kv_from, write_cache=own))
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = make_part("feed_forward", "gated", hidden=W, intermediate=layer.mlp.ff, w_gate_up=mat(p + "mlp.gate", p + "mlp.up"),
                            w_down=mat(p + "mlp.down"), activation="gelu_tanh")
            ffn_norm = norm(p + "norm2")
        blocks.append(make_part("block", "pre_norm", mixer_norm=norm(p + "norm1"), mixer=mixer, ffn_norm=ffn_norm, ffn=ffn))
    # cache layers are numbered without gaps: a layer without rows of its own has none
    used = sorted({r.cache for r in schedule})
    renumber = {c: n for n, c in enumerate(used)}
    schedule = [LayerRun(r.block, renumber[r.cache], r.write_cache) for r in schedule]
    embedding = NormedEmbedding(cfg.vocab, W, mat("embed"), norm("embed.norm"))
    head = LMHead(cfg.vocab, W, mat("head")) if cfg.logit_softcap is None else CappedLMHead(cfg.vocab, W, mat("head"), cfg.logit_softcap)
    return DecoderModel(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=norm("final.norm"), lm_head=head, position=None,
                        dtype=dtype, vocab_size=cfg.vocab, max_positions=UNBOUNDED_POSITIONS, config=cfg)
