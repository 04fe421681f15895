"""Ropulix, described as parts.

A decoder whose norms sit on the sublayers' outputs (``x <- x + norm(sublayer(x))``) and whose layers carry one of three
mixers: ``attention`` (grouped-query softmax attention without rotation, unit-norm q and k, a sliding window, one sigmoid
gate per head), ``rglru`` (a gated linear recurrence per channel behind a short convolution) or ``latent_attention``
(attention over one low-rank latent per token with a rotated key part shared by the heads, a sliding window and an
element-wise sigmoid gate; a layer may read the latent another layer keeps).  The feed-forward is a mixture of experts
(squared relu, softmax over the chosen logits); the output head is the embedding table.

Tensor names: a layer's tensors start with ``l<i>.``; ``norm1``, ``norm2``, ``mix.*``, ``mlp.*``; a linear map's weight is
stored under the map's own name (no ``.weight``), its bias under ``<name>.b``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..errors import ConfigError
from ..config.ropulix import LatentAttention, Recurrence, RopulixConfig, RopulixLayer, WindowAttention
from .description import LayerDescription, ModelDescription
from .sorulix import stored_name

# Fixed by the design (not in config.json): the recurrence's decay is exp(-8 r softplus(lam)); experts square their relu.
DECAY_SCALE = 8.0
EXPERT_ACT = "relu2"


def _keep_window(index: int, config: RopulixConfig) -> int | None:
    """How far back the latent that layer ``index`` keeps is read: by itself and by every layer that borrows it."""

    windows = [config.layers[index].mixer.window]
    windows += [layer.mixer.window for layer in config.layers
                if isinstance(layer.mixer, LatentAttention) and layer.mixer.kv_from == index]
    return None if any(w is None for w in windows) else max(windows)


def _mixer(index: int, layer: RopulixLayer, config: RopulixConfig, q_ranks: dict[int, int]) -> dict:
    m = layer.mixer
    if isinstance(m, WindowAttention):
        return {"kind": "gated_attention", "hidden_size": config.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
                "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale, "unit_eps": config.eps, "window": m.window}
    if isinstance(m, Recurrence):
        return {"kind": "gated_linear_recurrence", "hidden_size": config.width, "width": m.width, "blocks": m.blocks,
                "taps": m.conv, "decay_scale": DECAY_SCALE}
    assert isinstance(m, LatentAttention)
    q_rank = m.q_rank or q_ranks.get(index, 0)
    if q_rank <= 0:
        raise ConfigError(f"layers[{index}].mixer.q_rank is neither in the configuration nor given by a stored tensor's shape")
    return {
        "kind": "latent_attention", "hidden_size": config.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
        "value_dim": m.vdim, "kv_rank": m.kv_rank, "q_rank": q_rank, "eps": config.eps, "scale": m.scale, "window": m.window,
        "position": {"kind": "rope", "head_dim": m.rot_dim, "theta": m.rot_base, "rotary_dim": m.rot_dims} if m.rot_dims else None,
        "shares_kv": m.kv_from is not None, "keep_window": None if m.kv_from is not None else _keep_window(index, config),
    }


def describe_ropulix(config: RopulixConfig, q_ranks: dict[int, int] | None = None) -> ModelDescription:
    """``q_ranks``: per latent attention layer whose configuration does not name it, the query latent's size (the stored
    shape of ``dq`` gives it: ``describe_for_checkpoint``)."""

    norm = {"kind": "rms_norm", "dim": config.width, "eps": config.eps}
    layers = []
    for i, layer in enumerate(config.layers):
        block = {
            "kind": "output_norm", "mixer_norm": norm, "mixer": _mixer(i, layer, config, q_ranks or {}),
            "ffn_norm": norm if layer.mlp else None,
            "feed_forward": {"kind": "routed_experts", "hidden_size": config.width, "intermediate_size": layer.mlp.ff,
                             "experts": layer.mlp.experts, "top": layer.mlp.top, "act": EXPERT_ACT} if layer.mlp else None,
            "names": {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "feed_forward": "mlp"},
        }
        layers.append(LayerDescription(block=block, prefix=f"l{i}"))
    cache_of = tuple(layer.mixer.kv_from if isinstance(layer.mixer, LatentAttention) else None for layer in config.layers)
    return ModelDescription(
        architecture=RopulixConfig.ARCHITECTURE, vocab_size=config.vocab, hidden_size=config.width,
        max_positions=RopulixConfig.MAX_POSITIONS, eos_token_ids=(),
        embedding={"prefix": "embed", "vocab_size": config.vocab, "hidden_size": config.width},
        layers=tuple(layers), order=tuple(range(len(layers))), cache_of=cache_of,
        final_norm={"prefix": "final.norm", **norm},
        head={"prefix": "head", "vocab_size": config.vocab, "hidden_size": config.width, "tied": True},
        stored_name=stored_name,
    )


def describe_for_checkpoint(config: RopulixConfig, shapes) -> ModelDescription:
    """The description with sizes that only the stored tensors give (``shapes``: name -> shape)."""

    q_ranks = {}
    for i, layer in enumerate(config.layers):
        dq = shapes.get(f"l{i}.mix.dq")
        if isinstance(layer.mixer, LatentAttention) and dq is not None and len(dq) == 2:
            q_ranks[i] = int(dq[0])
    return describe_ropulix(config, q_ranks)


ROPULIX = Architecture(
    name=RopulixConfig.ARCHITECTURE, model_type=RopulixConfig.MODEL_TYPE,
    config_from_dict=RopulixConfig.from_dict, describe=describe_ropulix, describe_for_checkpoint=describe_for_checkpoint,
)
register_architecture(ROPULIX, replace=True)
