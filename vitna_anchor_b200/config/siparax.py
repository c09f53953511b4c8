"""Typed configuration of the Siparax decoder, read from config.json.

config.json gives every size and every constant that differs between models of the design:

    architecture      "Siparax"
    vocab, width
    norm.eps          eps of every norm of the model (the layer norms and the RMS norms inside the mixers)
    logit_softcap     the logits become cap * tanh(logits / cap) (absent: they are left as they are)
    layers            a list; each entry has `type` (latent_attention | latent_attention_2 | channel_delta), `mixer` (its
                      sizes) and `mlp` (or null)

A latent attention mixer gives heads, dim (plain query/key values a head), rot_dim (rotated ones), vdim, kv_rank, q_rank,
scale and rot {base, dims, scaling {factor, original, fast, slow}}; the second form may give kv_from, the layer whose
cached rows it reads.  The two forms differ in how the rotation pairs its values (neighbours, or the two halves) and in
the second form's gate on every head's output.  A channel_delta mixer gives heads, kv_heads, dim, vdim and conv; the
ranks of its two low-rank projections are read from the tensors.  A feed-forward gives kind (dense) and ff.  There is no
limit on positions: nothing of the model is a table over them.  A key inside a layer that this reader does not know is
refused by name.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .lupanex import MlpSpec, _known, _number, _size

ARCHITECTURE = "Siparax"
LATENT_TYPES = ("latent_attention", "latent_attention_2")


@dataclass(frozen=True)
class RotationSpec:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # (factor, original, fast, slow)


@dataclass(frozen=True)
class LatentSpec:
    kind: str                       # latent_attention (neighbouring pairs) or latent_attention_2 (halves, gated)
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotationSpec
    kv_from: Optional[int] = None

    @property
    def interleaved(self) -> bool:
        return self.kind == "latent_attention"

    @property
    def gated(self) -> bool:
        return self.kind == "latent_attention_2"


@dataclass(frozen=True)
class ChannelDeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    kind = "channel_delta"


@dataclass(frozen=True)
class LayerSpec:
    mixer: Any                      # LatentSpec or ChannelDeltaSpec
    mlp: Optional[MlpSpec]


def _rotation(r: Mapping[str, Any], where: str) -> RotationSpec:
    _known(r, where, ("base", "dims", "scaling"))
    scaling = None
    if r.get("scaling") is not None:
        _known(r["scaling"], where + ".scaling", ("factor", "original", "fast", "slow"))
        scaling = tuple(_number(r["scaling"], k, where + ".scaling.") for k in ("factor", "original", "fast", "slow"))
        if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
            raise ConfigError(f"config.json: {where}.scaling has a number that is not positive")
    base, dims = _number(r, "base", where + "."), _size(r, "dims", where + ".", 0)
    if base <= 1 or dims % 2:
        raise ConfigError(f"config.json: {where} needs a base above 1 and an even number of dims")
    return RotationSpec(base, dims, scaling)


def _layer(i: int, entry: Mapping[str, Any]) -> LayerSpec:
    where = f"layers[{i}]."
    _known(entry, f"layers[{i}]", ("type", "mixer", "mlp"))
    kind, m = entry.get("type"), entry.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}mixer is missing")
    if kind in LATENT_TYPES:
        keys = ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot") + (("kv_from",) if kind == "latent_attention_2" else ())
        _known(m, where + "mixer", keys)
        s = lambda k, least=1: _size(m, k, where + "mixer.", least)
        if not isinstance(m.get("rot"), Mapping):
            raise ConfigError(f"config.json: {where}mixer.rot is missing")
        rot = _rotation(m["rot"], where + "mixer.rot")
        kv_from = s("kv_from", 0) if m.get("kv_from") is not None else None
        mixer = LatentSpec(kind, s("heads"), s("dim"), s("rot_dim", 0), s("vdim"), s("kv_rank"), s("q_rank"), _number(m, "scale", where + "mixer."),
                           rot, kv_from)
        if rot.dims > mixer.rot_dim:
            raise ConfigError(f"config.json: {where}mixer.rot.dims is larger than rot_dim")
    elif kind == "channel_delta":
        _known(m, where + "mixer", ("heads", "kv_heads", "dim", "vdim", "conv"))
        heads = _size(m, "heads", where + "mixer.")
        kv = _size(m, "kv_heads", where + "mixer.") if m.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}mixer.heads do not divide into kv_heads groups")
        dim = _size(m, "dim", where + "mixer.")
        mixer = ChannelDeltaSpec(heads, kv, dim, _size(m, "vdim", where + "mixer.") if m.get("vdim") is not None else dim,
                                 _size(m, "conv", where + "mixer."))
    else:
        raise ConfigError(f"config.json: {where}type is {kind!r}; the mixers are {', '.join(LATENT_TYPES)} and channel_delta")
    mlp = None
    if entry.get("mlp") is not None:
        _known(entry["mlp"], where + "mlp", ("kind", "ff"))
        if entry["mlp"].get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp.kind is {entry['mlp'].get('kind')!r}; the only kind is dense")
        mlp = MlpSpec("dense", _size(entry["mlp"], "ff", where + "mlp."))
    return LayerSpec(mixer, mlp)


@dataclass(frozen=True)
class SiparaxConfig:
    vocab: int
    width: int
    eps: float
    logit_softcap: Optional[float]
    layers: Tuple[LayerSpec, ...]

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "SiparaxConfig":
        top = ("architecture", "architectures", "vocab", "width", "norm", "logit_softcap", "layers")
        other = sorted(set(cfg) - set(top))
        if other:       # notes beside the model (a name, a seed) are no part of it; a key inside a layer is, and is refused
            warnings.warn(f"config.json: keys that are no part of the model are ignored: {', '.join(other)}", stacklevel=2)
        _known(cfg.get("norm"), "norm", ("eps",))
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers is not a list of layers")
        layers = tuple(_layer(i, e) for i, e in enumerate(entries))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, LatentSpec) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if m.kv_from < i else None
                if not isinstance(src, LatentSpec) or src.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from does not name an earlier latent attention layer with rows of its own")
                if (src.kv_rank, src.rot_dim) != (m.kv_rank, m.rot_dim):      # the rows are read as that layer wrote them; this layer's
                    raise ConfigError(f"config.json: layers[{i}] and the layer it reads rows from differ in kv_rank or rot_dim")     # own rotation turns its queries
        eps = _number(cfg["norm"], "eps", "norm.")
        if eps < 0:
            raise ConfigError("config.json: norm.eps is negative")
        cap = _number(cfg, "logit_softcap", "") if cfg.get("logit_softcap") is not None else None
        if cap is not None and cap <= 0:
            raise ConfigError("config.json: logit_softcap is not positive")
        return cls(vocab=_size(cfg, "vocab", ""), width=_size(cfg, "width", ""), eps=eps, logit_softcap=cap, layers=layers)

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        def mixer(m):
            if isinstance(m, ChannelDeltaSpec):
                return dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, conv=m.conv)
            rot = dict(base=m.rot.base, dims=m.rot.dims)
            if m.rot.scaling is not None:
                rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
            d = dict(heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale, rot=rot)
            if m.kv_from is not None:
                d["kv_from"] = m.kv_from
            return d

        d = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.eps),
                 layers=[dict(type=l.mixer.kind, mixer=mixer(l.mixer), mlp=None if l.mlp is None else dict(kind=l.mlp.kind, ff=l.mlp.ff))
                         for l in self.layers])
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
