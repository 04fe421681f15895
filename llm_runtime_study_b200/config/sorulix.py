"""Typed configuration of the Sorulix decoder.

``config.json`` gives the vocabulary, the width, the norms' epsilon, the list of layers (each with the
type of its mixer, the mixer's sizes and constants, and its feed-forward or ``null``) and, optionally, a
loop: layers ``start .. stop-1`` run ``times`` times in a row with the same weights.  Every size and
constant is read from there; nothing about a particular model is written in the code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..errors import ConfigError
from .fields import optional, required

NUMBER = (int, float)


@dataclass(frozen=True)
class SoftmaxHalf:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    q_temp: tuple[float, int] | None      # (coef, every)


@dataclass(frozen=True)
class LinearHalf:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxHalf
    right: LinearHalf


@dataclass(frozen=True)
class ChannelDeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float


@dataclass(frozen=True)
class SorulixLayer:
    type: str
    mixer: ParallelMixer | ChannelDeltaMixer
    mlp: DenseMlp | None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _positive(raw: Mapping[str, Any], name: str, where: str) -> int:
    value = required(raw, name, int)
    if value <= 0:
        raise ConfigError(f"{where}.{name} must be positive, got {value}")
    return value


def _object(raw: Mapping[str, Any], name: str, where: str) -> Mapping[str, Any]:
    value = required(raw, name, dict)
    return value


def _softmax_half(raw: Mapping[str, Any], where: str) -> SoftmaxHalf:
    heads, kv_heads = _positive(raw, "heads", where), _positive(raw, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    temp = optional(raw, "q_temp", (dict, type(None)), None)
    q_temp = None
    if temp is not None:
        q_temp = (float(required(temp, "coef", NUMBER)), _positive(temp, "every", f"{where}.q_temp"))
    softcap = optional(raw, "softcap", (*NUMBER, type(None)), None)
    if softcap is not None and softcap <= 0:
        raise ConfigError(f"{where}.softcap must be positive, got {softcap}")
    return SoftmaxHalf(heads, kv_heads, _positive(raw, "dim", where), _positive(raw, "vdim", where),
                       float(required(raw, "scale", NUMBER)), None if softcap is None else float(softcap), q_temp)


def _linear_half(raw: Mapping[str, Any], where: str) -> LinearHalf:
    heads = _positive(raw, "heads", where)
    decay = required(raw, "decay", list)
    if len(decay) != heads or not all(isinstance(d, NUMBER) and not isinstance(d, bool) for d in decay):
        raise ConfigError(f"{where}.decay must list one number per head ({heads})")
    return LinearHalf(heads, _positive(raw, "dim", where), _positive(raw, "vdim", where), tuple(float(d) for d in decay))


def _layer(raw: Any, index: int) -> SorulixLayer:
    where = f"layers[{index}]"
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be an object")
    kind = required(raw, "type", str)
    mixer = _object(raw, "mixer", where)
    if kind == "parallel":
        typed: Any = ParallelMixer(_softmax_half(_object(mixer, "left", f"{where}.mixer"), f"{where}.mixer.left"),
                                   _linear_half(_object(mixer, "right", f"{where}.mixer"), f"{where}.mixer.right"))
    elif kind == "channel_delta":
        m = f"{where}.mixer"
        heads, kv_heads = _positive(mixer, "heads", m), _positive(mixer, "kv_heads", m)
        if heads % kv_heads:
            raise ConfigError(f"{m}: heads {heads} is not a multiple of kv_heads {kv_heads}")
        typed = ChannelDeltaMixer(heads, kv_heads, _positive(mixer, "dim", m), _positive(mixer, "vdim", m), _positive(mixer, "conv", m))
    else:
        raise ConfigError(f"{where}.type {kind!r} is not a layer of this design; expected parallel or channel_delta")
    mlp_raw = optional(raw, "mlp", (dict, type(None)), None)
    mlp = None
    if mlp_raw is not None:
        mlp_kind = required(mlp_raw, "kind", str)
        if mlp_kind != "dense":
            raise ConfigError(f"{where}.mlp.kind {mlp_kind!r} is not a feed-forward of this design; expected dense")
        limit = float(required(mlp_raw, "limit", NUMBER))
        if limit <= 0:
            raise ConfigError(f"{where}.mlp.limit must be positive, got {limit}")
        mlp = DenseMlp(_positive(mlp_raw, "ff", f"{where}.mlp"), limit)
    return SorulixLayer(kind, typed, mlp)


@dataclass(frozen=True)
class SorulixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[SorulixLayer, ...]
    loop: Loop | None

    ARCHITECTURE = "Sorulix"
    MODEL_TYPE = "sorulix"
    # no table of positions exists in this design; the engine still wants a bound for its own bookkeeping
    MAX_POSITIONS = 1 << 24

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SorulixConfig":
        norm = _object(raw, "norm", "config")
        eps = float(required(norm, "eps", NUMBER))
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        layers_raw = required(raw, "layers", list)
        if not layers_raw:
            raise ConfigError("layers must not be empty")
        layers = tuple(_layer(item, i) for i, item in enumerate(layers_raw))
        loop_raw = optional(raw, "loop", (dict, type(None)), None)
        loop = None
        if loop_raw is not None:
            loop = Loop(required(loop_raw, "start", int), required(loop_raw, "stop", int), _positive(loop_raw, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"loop runs layers {loop.start} .. {loop.stop - 1}, but there are {len(layers)} layers")
        return cls(_positive(raw, "vocab", "config"), _positive(raw, "width", "config"), eps, layers, loop)

    def runs(self) -> list[tuple[int, int | None]]:
        """(layer, the number of the pass that starts with this run or ``None``) in execution order."""

        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        runs: list[tuple[int, int | None]] = [(i, None) for i in range(self.loop.start)]
        for t in range(self.loop.times):
            runs += [(i, t if i == self.loop.start else None) for i in range(self.loop.start, self.loop.stop)]
        return runs + [(i, None) for i in range(self.loop.stop, n)]

    def validate_context_length(self, max_seq_len: int) -> None:
        if max_seq_len <= 0:
            raise ConfigError(f"max_seq_len must be positive, got {max_seq_len}")
        if max_seq_len > self.MAX_POSITIONS:
            raise ConfigError(f"max_seq_len {max_seq_len} exceeds the engine's bound {self.MAX_POSITIONS}")
