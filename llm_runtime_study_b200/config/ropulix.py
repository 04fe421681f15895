"""Typed configuration of the Ropulix decoder.

``config.json`` gives the vocabulary, the width, the norms' epsilon and the list of layers; each layer names the type of
its mixer (``attention``, ``rglru`` or ``latent_attention``), the mixer's sizes and constants, and its feed-forward (a
mixture of experts, or ``null``).  Every size and constant is read from there; nothing about a particular model is
written in the code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..errors import ConfigError
from .fields import optional, required

NUMBER = (int, float)


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None


@dataclass(frozen=True)
class Recurrence:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int          # 0: not in config.json; the stored shape of ``dq`` gives it
    scale: float
    window: int | None
    rot_base: float
    rot_dims: int
    kv_from: int | None


@dataclass(frozen=True)
class Experts:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class RopulixLayer:
    type: str
    mixer: WindowAttention | Recurrence | LatentAttention
    mlp: Experts | None


def _positive(raw: Mapping[str, Any], name: str, where: str) -> int:
    value = required(raw, name, int)
    if value <= 0:
        raise ConfigError(f"{where}.{name} must be positive, got {value}")
    return value


def _window(mixer: Mapping[str, Any], where: str) -> int | None:
    mask = optional(mixer, "mask", (dict, type(None)), None)
    if mask is None:
        return None
    size = optional(mask, "size", (int, type(None)), None)
    if size is not None and size <= 0:
        raise ConfigError(f"{where}.mask.size must be positive, got {size}")
    return size


def _mixer(kind: str, mixer: Mapping[str, Any], where: str):
    if kind == "attention":
        heads = _positive(mixer, "heads", where)
        kv_heads = _positive(mixer, "kv_heads", where) if "kv_heads" in mixer else heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
        dim = _positive(mixer, "dim", where)
        vdim = _positive(mixer, "vdim", where) if "vdim" in mixer else dim
        return WindowAttention(heads, kv_heads, dim, vdim, float(required(mixer, "scale", NUMBER)), _window(mixer, where))
    if kind == "rglru":
        width, blocks = _positive(mixer, "width", where), _positive(mixer, "blocks", where)
        if width % blocks:
            raise ConfigError(f"{where}: width {width} is not a multiple of blocks {blocks}")
        return Recurrence(width, blocks, _positive(mixer, "conv", where))
    if kind == "latent_attention":
        rot_dim = required(mixer, "rot_dim", int)
        rot = optional(mixer, "rot", (dict, type(None)), None)
        if rot_dim < 0 or (rot_dim > 0 and rot is None):
            raise ConfigError(f"{where}: rot_dim {rot_dim} needs a rot entry with base and dims")
        rot_dims = required(rot, "dims", int) if rot else 0
        if rot_dims < 0 or rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"{where}.rot.dims must be even and at most rot_dim {rot_dim}, got {rot_dims}")
        base = float(required(rot, "base", NUMBER)) if rot else 1.0
        if base <= 0:
            raise ConfigError(f"{where}.rot.base must be positive, got {base}")
        kv_from = optional(mixer, "kv_from", (int, type(None)), None)
        dim = _positive(mixer, "dim", where)
        return LatentAttention(
            _positive(mixer, "heads", where), dim, rot_dim, _positive(mixer, "vdim", where) if "vdim" in mixer else dim,
            _positive(mixer, "kv_rank", where), _positive(mixer, "q_rank", where) if "q_rank" in mixer else 0,
            float(required(mixer, "scale", NUMBER)),
            _window(mixer, where), base, rot_dims, kv_from,
        )
    raise ConfigError(f"{where}: type {kind!r} is not a layer of this design; expected attention, rglru or latent_attention")


def _layer(raw: Any, index: int) -> RopulixLayer:
    where = f"layers[{index}]"
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} must be an object")
    kind = required(raw, "type", str)
    typed = _mixer(kind, required(raw, "mixer", dict), f"{where}.mixer")
    mlp_raw = optional(raw, "mlp", (dict, type(None)), None)
    mlp = None
    if mlp_raw is not None:
        mlp_kind = required(mlp_raw, "kind", str)
        if mlp_kind != "moe":
            raise ConfigError(f"{where}.mlp.kind {mlp_kind!r} is not a feed-forward of this design; expected moe")
        router, expert = required(mlp_raw, "router", dict), required(mlp_raw, "expert", dict)
        mlp = Experts(_positive(router, "experts", f"{where}.mlp.router"), _positive(router, "top", f"{where}.mlp.router"),
                      _positive(expert, "ff", f"{where}.mlp.expert"))
        if mlp.top > mlp.experts:
            raise ConfigError(f"{where}.mlp.router: top {mlp.top} exceeds experts {mlp.experts}")
    return RopulixLayer(kind, typed, mlp)


@dataclass(frozen=True)
class RopulixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[RopulixLayer, ...]

    ARCHITECTURE = "Ropulix"
    MODEL_TYPE = "ropulix"
    # positions enter through rotations and masks only; the engine still wants a bound for its own bookkeeping
    MAX_POSITIONS = 1 << 24

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "RopulixConfig":
        norm = required(raw, "norm", dict)
        eps = float(required(norm, "eps", NUMBER))
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        layers_raw = required(raw, "layers", list)
        if not layers_raw:
            raise ConfigError("layers must not be empty")
        layers = tuple(_layer(item, i) for i, item in enumerate(layers_raw))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, LatentAttention) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if 0 <= m.kv_from < i else None
                if not isinstance(src, LatentAttention) or src.kv_from is not None:
                    raise ConfigError(f"layers[{i}].mixer.kv_from {m.kv_from} must name an earlier latent_attention layer that keeps a latent of its own")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                    raise ConfigError(f"layers[{i}] borrows the latent of layers[{m.kv_from}], whose kv_rank, rot_dim and rotation differ")
        return cls(_positive(raw, "vocab", "config"), _positive(raw, "width", "config"), eps, layers)

    def validate_context_length(self, max_seq_len: int) -> None:
        if max_seq_len <= 0:
            raise ConfigError(f"max_seq_len must be positive, got {max_seq_len}")
        if max_seq_len > self.MAX_POSITIONS:
            raise ConfigError(f"max_seq_len {max_seq_len} exceeds the engine's bound {self.MAX_POSITIONS}")
