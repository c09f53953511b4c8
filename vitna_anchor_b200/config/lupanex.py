"""Typed configuration of the Lupanex decoder, read from config.json.

config.json gives every size and every constant that differs between models of the design:

    architecture      "Lupanex"
    vocab, width, max_positions
    embedding.scale   the token rows are multiplied by it; a learned row per position is added unscaled
    norm.eps          eps of every RMS norm of the model (also of the weightless ones inside the mixers)
    streams           residual streams joined by hyper-connections (absent: one plain residual stream)
    layers            a list; each entry has `type` (attention | delta), `mixer` (its sizes) and `mlp` (or null)
    loop              {start, stop, times}: layers start..stop-1 run `times` times in a row with the same weights,
                      every pass with a cache or state of its own (absent: every layer runs once)

An attention mixer gives heads, kv_heads, dim, vdim and scale, and may give bias_max (with a table of distance
biases among the weights) and q_temp {coef, every}.  A delta mixer gives heads, kv_heads, dim, vdim and conv (taps of
the short convolution).  A feed-forward gives kind (dense) and ff.  What a configuration does not mention is not
there; a key inside a layer, the loop, the embedding or the norm that this reader does not know is refused by name, so
that a model that needs more than the engine has is never run as if it needed less.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .errors import ConfigError

ARCHITECTURE = "Lupanex"


def _known(obj: Mapping[str, Any], where: str, keys) -> None:
    if not isinstance(obj, Mapping):
        raise ConfigError(f"config.json: {where} is not an object")
    extra = sorted(set(obj) - set(keys))
    if extra:
        raise ConfigError(f"config.json: {where} has keys this engine does not know: {', '.join(extra)}")


def _size(obj: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    v = obj.get(key)
    if v is None:
        raise ConfigError(f"config.json: {where}{key} is missing")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != int(v) or v < least or v > 1e9:
        raise ConfigError(f"config.json: {where}{key} is not an integer of at least {least}")
    return int(v)


def _number(obj: Mapping[str, Any], key: str, where: str) -> float:
    v = obj.get(key)
    if v is None:
        raise ConfigError(f"config.json: {where}{key} is missing")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}{key} is not a number")
    return float(v)


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: Optional[int] = None                  # with it the layer has a table of distance biases
    q_temp: Optional[Tuple[float, int]] = None      # (coef, every)

    kind = "attention"


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    kind = "delta"


@dataclass(frozen=True)
class MlpSpec:
    kind: str
    ff: int


@dataclass(frozen=True)
class LayerSpec:
    mixer: Any                      # AttentionSpec or DeltaSpec
    mlp: Optional[MlpSpec]


def _heads(m: Mapping[str, Any], where: str):
    """heads, kv_heads (the heads, if not given), dim, vdim (dim, if not given)."""
    heads = _size(m, "heads", where)
    kv = _size(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads do not divide into kv_heads groups")
    dim = _size(m, "dim", where)
    return heads, kv, dim, _size(m, "vdim", where) if m.get("vdim") is not None else dim


def _layer(i: int, entry: Mapping[str, Any]) -> LayerSpec:
    where = f"layers[{i}]."
    _known(entry, f"layers[{i}]", ("type", "mixer", "mlp"))
    kind, m = entry.get("type"), entry.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}mixer is missing")
    if kind == "attention":
        _known(m, where + "mixer", ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max", "q_temp"))
        heads, kv, dim, vdim = _heads(m, where + "mixer.")
        q_temp = None
        if m.get("q_temp") is not None:
            _known(m["q_temp"], where + "mixer.q_temp", ("coef", "every"))
            q_temp = (_number(m["q_temp"], "coef", where + "mixer.q_temp."), _size(m["q_temp"], "every", where + "mixer.q_temp."))
        bias_max = _size(m, "bias_max", where + "mixer.", 2) if m.get("bias_max") is not None else None
        mixer = AttentionSpec(heads, kv, dim, vdim, _number(m, "scale", where + "mixer."), bias_max, q_temp)
    elif kind == "delta":
        _known(m, where + "mixer", ("heads", "kv_heads", "dim", "vdim", "conv"))
        heads, kv, dim, vdim = _heads(m, where + "mixer.")
        mixer = DeltaSpec(heads, kv, dim, vdim, _size(m, "conv", where + "mixer."))
    else:
        raise ConfigError(f"config.json: {where}type is {kind!r}; the mixers are attention and delta")
    mlp = None
    if entry.get("mlp") is not None:
        _known(entry["mlp"], where + "mlp", ("kind", "ff"))
        if entry["mlp"].get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp.kind is {entry['mlp'].get('kind')!r}; the only kind is dense")
        mlp = MlpSpec("dense", _size(entry["mlp"], "ff", where + "mlp."))
    return LayerSpec(mixer, mlp)


@dataclass(frozen=True)
class LupanexConfig:
    vocab: int
    width: int
    max_positions: int
    eps: float
    embedding_scale: float
    streams: Optional[int]
    layers: Tuple[LayerSpec, ...]
    loop: Optional[Tuple[int, int, int]]            # (start, stop, times)

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "LupanexConfig":
        top = ("architecture", "architectures", "vocab", "width", "max_positions", "embedding", "norm", "streams", "layers", "loop")
        other = sorted(set(cfg) - set(top))
        if other:       # notes beside the model (a name, a seed) are no part of it; a key inside a layer is, and is refused
            warnings.warn(f"config.json: keys that are no part of the model are ignored: {', '.join(other)}", stacklevel=2)
        _known(cfg.get("embedding"), "embedding", ("scale",))
        _known(cfg.get("norm"), "norm", ("eps",))
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers is not a list of layers")
        layers = tuple(_layer(i, e) for i, e in enumerate(entries))
        loop = None
        if cfg.get("loop") is not None:
            _known(cfg["loop"], "loop", ("start", "stop", "times"))
            start, stop = _size(cfg["loop"], "start", "loop.", 0), _size(cfg["loop"], "stop", "loop.", 0)
            times = _size(cfg["loop"], "times", "loop.", 1)
            if not (start <= stop <= len(layers)):
                raise ConfigError("config.json: loop.start .. loop.stop is not a range of the layers")
            loop = (start, stop, times)
        eps = _number(cfg["norm"], "eps", "norm.")
        if eps < 0:
            raise ConfigError("config.json: norm.eps is negative")
        return cls(vocab=_size(cfg, "vocab", ""), width=_size(cfg, "width", ""), max_positions=_size(cfg, "max_positions", ""),
                   eps=eps, embedding_scale=_number(cfg["embedding"], "scale", "embedding."),
                   streams=_size(cfg, "streams", "") if cfg.get("streams") is not None else None, layers=layers, loop=loop)

    def runs(self) -> List[int]:
        """The layers in the order they run, a looped one as often as it runs."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        def mixer(m):
            if m.kind == "delta":
                return dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, conv=m.conv)
            d = dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale)
            if m.bias_max is not None:
                d["bias_max"] = m.bias_max
            if m.q_temp is not None:
                d["q_temp"] = dict(coef=m.q_temp[0], every=m.q_temp[1])
            return d

        d = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, max_positions=self.max_positions,
                 embedding=dict(scale=self.embedding_scale), norm=dict(eps=self.eps),
                 layers=[dict(type=l.mixer.kind, mixer=mixer(l.mixer), mlp=None if l.mlp is None else dict(kind=l.mlp.kind, ff=l.mlp.ff))
                         for l in self.layers])
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = dict(start=self.loop[0], stop=self.loop[1], times=self.loop[2])
        return d
