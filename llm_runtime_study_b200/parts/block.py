"""Arrangement of norm, mixer and feed-forward in one layer."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..weights.checkpoint import TensorSpec
from ..weights.view import TensorView
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, ResidualStream, Runtime

_DEFAULT_NAMES = {
    "mixer_norm": "input_layernorm",
    "mixer": "self_attn",
    "ffn_norm": "post_attention_layernorm",
    "feed_forward": "mlp",
}


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h = h + mixer(norm_1(h)); h = h + ffn(norm_2(h))``
    (mini_llm/model/qwen.py:58-72).  The additions are carried out by the *next*
    norm, in float32, while it reads the rows anyway.  ``names`` gives the
    checkpoint's name of each sub-part below the layer's prefix.  A layer
    without a feed-forward (``feed_forward=None``) is its first half only."""

    def __init__(
        self, *, mixer: Mapping[str, Any], feed_forward: Mapping[str, Any] | None, mixer_norm: Mapping[str, Any],
        ffn_norm: Mapping[str, Any] | None = None, names: Mapping[str, str] | None = None,
    ) -> None:
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.mixer = MIXERS.build(mixer)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward else None
        self.ffn_norm = NORMS.build(ffn_norm) if feed_forward else None
        if feed_forward and not ffn_norm:
            raise ValueError("a pre_norm block with a feed-forward needs the norm before it (ffn_norm)")

    graph_safe = True

    def children(self):
        return tuple(part for _, part in self._parts())

    def _parts(self):
        parts = [(self.names["mixer_norm"], self.mixer_norm), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            parts += [(self.names["ffn_norm"], self.ffn_norm), (self.names["feed_forward"], self.feed_forward)]
        return tuple(parts)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {f"{prefix}.{n}": s for prefix, part in self._parts() for n, s in part.tensor_specs().items()}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        view = TensorView.of(tensors)
        for prefix, part in self._parts():
            part.load(view.sub(prefix), runtime)

    fuses_norms = True

    def first_norm(self):
        return self.mixer_norm

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any, next_norm: Any = None) -> None:
        x = stream.take_rows(self.mixer_norm, self.mixer)
        after_mixer = self.ffn_norm if self.feed_forward is not None else next_norm
        stream.put(self._run(self.mixer, (x, ctx, cache), stream.resid, after_mixer), after_mixer)
        if self.feed_forward is None:
            return
        x = stream.take_rows(self.ffn_norm, self.feed_forward)
        stream.put(self._run(self.feed_forward, (x, ctx), stream.resid, next_norm), next_norm)

    @staticmethod
    def _run(part: Any, args: tuple, resid: torch.Tensor, next_norm: Any):
        """Call a mixer or feed-forward with as much as it says it can take."""

        if not part.adds_to_residual:
            return part.forward(*args)
        if part.fuses_norms:
            return part.forward(*args, residual=resid, next_norm=next_norm)
        return part.forward(*args, residual=resid)


@BLOCKS.register("output_norm")
class OutputNormBlock(Block):
    """``h = h + norm_1(mixer(h)); h = h + norm_2(ffn(h))``: the sublayers read the residual rows themselves (rounded to
    the activation type where that is not float32) and the norm sits on their output only.  The kernel that normalises a
    sublayer's output adds it into the float32 rows and hands the next sublayer its rounded copy in the same pass.
    ``names`` as for ``pre_norm``; a layer without a feed-forward is its first half only."""

    graph_safe = True

    def __init__(
        self, *, mixer: Mapping[str, Any], feed_forward: Mapping[str, Any] | None, mixer_norm: Mapping[str, Any],
        ffn_norm: Mapping[str, Any] | None = None, names: Mapping[str, str] | None = None,
    ) -> None:
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.mixer = MIXERS.build(mixer)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward else None
        self.ffn_norm = NORMS.build(ffn_norm) if feed_forward else None
        if feed_forward and not ffn_norm:
            raise ValueError("an output_norm block with a feed-forward needs the norm behind it (ffn_norm)")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and norm.fusable() is None:
                raise ValueError("an output_norm block normalises with a norm of the form w * x * rsqrt(mean(x^2) + eps)")

    def children(self):
        return tuple(part for _, part in self._parts())

    _parts = PreNormBlock._parts
    tensor_specs = PreNormBlock.tensor_specs
    load = PreNormBlock.load

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any) -> None:
        from ..ops import mixer_steps as M

        resid = stream.resid
        if stream.delta is not None:
            resid += stream.delta
            stream.put(None, None)
        act = self.runtime.dtype
        rounds = act != torch.float32
        # what the block before this one left for its reader, if it was a block of this kind
        x = stream.rounded
        stream.put(None, None)
        if x is None:
            x = M.norm_accumulate_round(None, None, 0.0, resid, act) if rounds else resid
        out = self.mixer.forward(x, ctx, cache)
        weight, eps = self.mixer_norm.fusable()
        x = M.norm_accumulate_round(out, weight, eps, resid, act if rounds else None)
        if self.feed_forward is not None:
            # a feed-forward that can hand over its experts' rows unsummed does: the norm's kernel forms the sum
            pieces = {"pieces": True} if getattr(self.feed_forward, "returns_pieces", False) else {}
            out = self.feed_forward.forward(x if rounds else resid, ctx, **pieces)
            weight, eps = self.ffn_norm.fusable()
            x = M.norm_accumulate_round(out, weight, eps, resid, act if rounds else None)
        if rounds:
            stream.rounded = x
