"""Sorulix, described as parts.

A pre-norm decoder whose layers carry one of two mixers: ``parallel`` (softmax attention with a sink,
a soft cap, a bias by distance and a query temperature, beside linear attention with a constant decay
per head; the mean of their normalised outputs) or ``channel_delta`` (the delta rule with a decay per
key channel behind short convolutions).  Norm weights are kept as offsets from one (``1 + w``); the
feed-forward is a gated unit with limits and biases; the output head is the embedding table.  A run of
layers may be passed several times with the same weights: every pass has caches and states of its own,
and starts by adding the embedding's output (not in the first pass) and a row of ``loop.step``.

Tensor names: a layer's tensors start with ``l<i>.``; ``norm1``, ``norm2``, ``mix.*``, ``mlp.*``; a linear
map's weight is stored under the map's own name (no ``.weight``), its bias under ``<name>.b``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.sorulix import ChannelDeltaMixer, ParallelMixer, SorulixConfig, SorulixLayer
from .description import LayerDescription, ModelDescription

# Fixed by the design (not in config.json): the bias by distance falls as 2^(-8 (h+1) / H) over the heads;
# the low-rank maps of the delta rule's decay and gate are sized by their tensors, see ``_delta_ranks``.
SLOPE_EXPONENT = 8.0
GLU_ALPHA = 1.702
UNIT_EPS = 1e-6


def stored_name(name: str) -> str:
    """The parts of this package call a norm's or an embedding's tensor ``<part>.weight``; the checkpoint stores it
    under the part's own name."""

    return name[: -len(".weight")] if name.endswith(".weight") else name


def _mixer(layer: SorulixLayer, config: SorulixConfig, ranks: tuple[int, int]) -> dict:
    m = layer.mixer
    if isinstance(m, ParallelMixer):
        left, right = m.left, m.right
        return {
            "kind": "parallel", "hidden_size": config.width, "eps": config.eps,
            "branches": [
                {"name": "left", "mixer": {
                    "kind": "sink_attention", "hidden_size": config.width, "num_heads": left.heads, "num_kv_heads": left.kv_heads,
                    "head_dim": left.dim, "value_dim": left.vdim, "scale": left.scale, "qk_norm_eps": config.eps,
                    "temperature": left.q_temp, "softcap": left.softcap, "slope_exponent": SLOPE_EXPONENT, "sink": True,
                }},
                {"name": "right", "mixer": {
                    "kind": "decayed_linear_attention", "hidden_size": config.width, "num_heads": right.heads,
                    "head_dim": right.dim, "value_dim": right.vdim, "decay": right.decay, "eps": config.eps,
                }},
            ],
        }
    assert isinstance(m, ChannelDeltaMixer)
    return {
        "kind": "gated_delta_rule", "hidden_size": config.width, "num_heads": m.heads, "num_qk_heads": m.kv_heads,
        "head_dim": m.dim, "value_dim": m.vdim, "taps": m.conv, "decay_rank": ranks[0], "gate_rank": ranks[1],
        "eps": config.eps, "unit_eps": UNIT_EPS,
    }


def describe_sorulix(config: SorulixConfig, ranks: dict[int, tuple[int, int]] | None = None) -> ModelDescription:
    """``ranks``: per channel_delta layer, the inner sizes of its two low-rank maps (decay, gate).  config.json does
    not give them; a checkpoint's tensor shapes do (``describe_for_checkpoint``).  Without them a quarter of the
    key size is assumed for both, which is what random weights are drawn with."""

    norm = {"kind": "rms_norm", "dim": config.width, "eps": config.eps, "offset": 1.0}
    layers = []
    for i, layer in enumerate(config.layers):
        default = max(1, layer.mixer.dim // 4) if isinstance(layer.mixer, ChannelDeltaMixer) else 0
        block = {
            "kind": "pre_norm", "mixer_norm": norm, "mixer": _mixer(layer, config, (ranks or {}).get(i, (default, default))),
            "ffn_norm": norm if layer.mlp else None,
            "feed_forward": {"kind": "limited_glu", "hidden_size": config.width, "intermediate_size": layer.mlp.ff,
                             "limit": layer.mlp.limit, "alpha": GLU_ALPHA} if layer.mlp else None,
            "names": {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "feed_forward": "mlp"},
        }
        layers.append(LayerDescription(block=block, prefix=f"l{i}"))
    runs = config.runs()
    before_run = {
        run: {"kind": "pass_entry", "prefix": "loop", "hidden_size": config.width, "passes": config.loop.times,
              "index": starts_pass, "add_first": starts_pass > 0}
        for run, (_, starts_pass) in enumerate(runs) if starts_pass is not None
    }
    return ModelDescription(
        architecture=SorulixConfig.ARCHITECTURE, vocab_size=config.vocab, hidden_size=config.width,
        max_positions=SorulixConfig.MAX_POSITIONS, eos_token_ids=(),
        embedding={"prefix": "embed", "vocab_size": config.vocab, "hidden_size": config.width},
        layers=tuple(layers), order=tuple(layer for layer, _ in runs),
        final_norm={"prefix": "final.norm", **norm},
        head={"prefix": "head", "vocab_size": config.vocab, "hidden_size": config.width, "tied": True},
        before_run=before_run, stored_name=stored_name,
    )


def describe_for_checkpoint(config: SorulixConfig, shapes) -> ModelDescription:
    """The description with the low-rank sizes read from the checkpoint's tensor shapes (``shapes``: name -> shape)."""

    ranks = {}
    for i, layer in enumerate(config.layers):
        if isinstance(layer.mixer, ChannelDeltaMixer):
            a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
            if a1 is not None and g1 is not None and len(a1) == 2 and len(g1) == 2:
                ranks[i] = (int(a1[0]), int(g1[0]))
    return describe_sorulix(config, ranks)


SORULIX = Architecture(
    name=SorulixConfig.ARCHITECTURE, model_type=SorulixConfig.MODEL_TYPE,
    config_from_dict=SorulixConfig.from_dict, describe=describe_sorulix, describe_for_checkpoint=describe_for_checkpoint,
)
register_architecture(SORULIX, replace=True)
