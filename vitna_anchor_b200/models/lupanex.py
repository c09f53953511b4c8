"""The Lupanex decoder: manifest of its tensors and how its layers are built from the engine's parts.

A small decoder-only language model whose layers each choose between two mixers: an attention without a rotation
(unit-RMS q and k, a query factor that grows with the position, a learned bias by bucketed distance, values of their
own size) and the gated delta rule (a recurrent matrix state per head behind a short convolution).  The feed-forward
is dense with the erf form of gelu, or absent.  Tokens are embedded as scale * row + a learned row for the position.
With `streams` the residual stream is several rows joined by hyper-connections, else one row with plain pre-norm
sums.  A range of layers may run several times in a row with the same weights, each pass with its own cache or state.

Tensor names: embed, pos, final.norm, head; layer i has l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{up,down} and, with
streams, l<i>.hc{1,2}.{in,mix,out}.  Matrices are [out, in].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.lupanex import LupanexConfig
from ..parts.attention import bucketed_distance_bias
from ..parts.embedding import LMHead, ScaledEmbedding
from ..parts.hyper import HyperConnection, StreamSum
from ..parts.registry import make_part
from ..weights.loader import WeightSpec
from .decoder import DecoderModel, LayerRun


def lupanex_manifest(cfg: LupanexConfig) -> List[WeightSpec]:
    W = cfg.width
    m = [WeightSpec("embed", (cfg.vocab, W)), WeightSpec("pos", (cfg.max_positions, W))]
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer.mixer
        m.append(WeightSpec(p + "norm1", (W,)))
        if mx.kind == "attention":
            m += [WeightSpec(p + "mix.q", (mx.heads * mx.dim, W)), WeightSpec(p + "mix.k", (mx.kv_heads * mx.dim, W)),
                  WeightSpec(p + "mix.v", (mx.kv_heads * mx.vdim, W)), WeightSpec(p + "mix.o", (W, mx.heads * mx.vdim))]
            if mx.bias_max is not None:
                m.append(WeightSpec(p + "mix.rel", (None, mx.heads), free_size=32))      # as many rows as the checkpoint gives
        else:
            qk, v = mx.kv_heads * mx.dim, mx.heads * mx.vdim
            m += [WeightSpec(p + "mix.q", (qk, W)), WeightSpec(p + "mix.q.conv", (qk, mx.conv)),
                  WeightSpec(p + "mix.k", (qk, W)), WeightSpec(p + "mix.k.conv", (qk, mx.conv)),
                  WeightSpec(p + "mix.v", (v, W)), WeightSpec(p + "mix.v.conv", (v, mx.conv)),
                  WeightSpec(p + "mix.b", (mx.heads, W)), WeightSpec(p + "mix.a", (mx.heads, W)),
                  WeightSpec(p + "mix.A_log", (mx.heads,)), WeightSpec(p + "mix.dt_bias", (mx.heads,)),
                  WeightSpec(p + "mix.norm", (mx.vdim,)), WeightSpec(p + "mix.g", (v, W)), WeightSpec(p + "mix.o", (W, v))]
        if cfg.streams is not None:
            m += _hc_specs(p + "hc1.", cfg.streams)
        if layer.mlp is not None:
            m += [WeightSpec(p + "norm2", (W,)), WeightSpec(p + "mlp.up", (layer.mlp.ff, W)), WeightSpec(p + "mlp.down", (W, layer.mlp.ff))]
            if cfg.streams is not None:
                m += _hc_specs(p + "hc2.", cfg.streams)
    m += [WeightSpec("final.norm", (W,)), WeightSpec("head", (cfg.vocab, W))]
    return m


def _hc_specs(prefix: str, s: int) -> List[WeightSpec]:
    return [WeightSpec(prefix + "in", (s,)), WeightSpec(prefix + "out", (s,)), WeightSpec(prefix + "mix", (s, s))]


def is_norm_weight(name: str) -> bool:
    """Tensors that random initialisation makes 1 + noise instead of noise around 0 (True), or the identity + noise."""
    if name.endswith(("hc1.mix", "hc2.mix")):
        return "identity"
    last = name.rsplit(".", 1)[-1]
    return last in ("norm1", "norm2", "norm") or name.endswith(("hc1.in", "hc2.in", "hc1.out", "hc2.out"))


def build_lupanex(cfg: LupanexConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> DecoderModel:
    """Matrices go to the device in the compute dtype; norms, tables of biases and positions, the hyper-connections and the
    delta rule's per-head vectors and convolution weights are float32 in both paths."""
    dev = torch.device(device)
    W, s = cfg.width, cfg.streams

    def mat(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=dtype) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def vec(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=torch.float32) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def norm(name: str):
        return make_part("norm", "rmsnorm", width=W, eps=cfg.eps, weight=vec(name))

    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer.mixer
        if mx.kind == "attention":
            bias = None
            if mx.bias_max is not None:
                bias = bucketed_distance_bias(vec(p + "mix.rel"), mx.bias_max, cfg.max_positions)
            mixer = make_part("mixer", "attention", hidden=W, num_heads=mx.heads, num_kv_heads=mx.kv_heads, head_dim=mx.dim,
                              wqkv=mat(p + "mix.q", p + "mix.k", p + "mix.v"), wo=mat(p + "mix.o"), position=None, scale=mx.scale,
                              v_dim=mx.vdim, qk_norm_eps=cfg.eps, q_temp=mx.q_temp, dist_bias=bias)
        else:
            mixer = make_part("mixer", "gated_delta", hidden=W, num_heads=mx.heads, num_key_heads=mx.kv_heads, key_dim=mx.dim,
                              value_dim=mx.vdim, taps=mx.conv,
                              w_in=mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.b", p + "mix.a"),
                              conv=vec(p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv"), a_log=vec(p + "mix.A_log"),
                              dt_bias=vec(p + "mix.dt_bias"), norm_weight=vec(p + "mix.norm"), wo=mat(p + "mix.o"), eps=cfg.eps)
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = make_part("feed_forward", "dense", hidden=W, intermediate=layer.mlp.ff, w_up=mat(p + "mlp.up"), w_down=mat(p + "mlp.down"),
                            activation="gelu")
            ffn_norm = norm(p + "norm2")
        if s is None:
            blocks.append(make_part("block", "pre_norm", mixer_norm=norm(p + "norm1"), mixer=mixer, ffn_norm=ffn_norm, ffn=ffn))
        else:
            hc = lambda q: HyperConnection(s, vec(p + f"hc{q}.in"), vec(p + f"hc{q}.mix"), vec(p + f"hc{q}.out"))
            blocks.append(make_part("block", "hyper", streams=s, mixer_norm=norm(p + "norm1"), mixer_hc=hc(1), mixer=mixer,
                                    ffn_norm=ffn_norm, ffn_hc=hc(2) if ffn is not None else None, ffn=ffn))
    embedding = ScaledEmbedding(cfg.vocab, W, mat("embed"), cfg.embedding_scale, vec("pos"), copies=s or 1)
    # every run of a layer, a looped one each time, has a cache layer or state of its own
    schedule = [LayerRun(block=b, cache=r) for r, b in enumerate(cfg.runs())]
    return DecoderModel(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=norm("final.norm"),
                        lm_head=LMHead(cfg.vocab, W, mat("head")), position=None, dtype=dtype, vocab_size=cfg.vocab,
                        max_positions=cfg.max_positions, config=cfg, collect=StreamSum(s) if s is not None else None)
