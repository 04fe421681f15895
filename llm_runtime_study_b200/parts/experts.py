"""A feed-forward made of several small ones, of which a router picks a few per token."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import grouped as G
from ..ops.mixer_steps import PairedRows
from ..weights.checkpoint import TensorSpec
from .base import FEED_FORWARDS, FeedForward, Runtime


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """``experts`` feed-forward layers ``W_down act(W_up x)`` without biases (``act``: ``relu2``, the square of relu).  Router
    logits ``z = W_router x + b_router`` in float32; each token uses the ``top`` experts with the largest logits, weighted by
    the softmax over the chosen logits only; the output is the weighted sum.  Tensors: ``router``, ``router.b``,
    ``e<j>.up`` ``[ff, hidden]``, ``e<j>.down`` ``[hidden, ff]``.

    The (token, choice) pairs are sorted by expert on the device and every expert's rows are padded to whole tiles, so the
    two products run as one launch each over all experts, sized without the host knowing the counts."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, experts: int, top: int, act: str = "relu2",
                 router_bias: bool = True) -> None:
        if min(hidden_size, intermediate_size, experts, top) <= 0 or top > experts:
            raise ValueError("expert sizes must be positive and top at most the number of experts")
        if act != "relu2":
            raise ValueError(f"unknown expert activation {act!r}; expected relu2")
        self.hidden_size, self.intermediate_size, self.experts, self.top = hidden_size, intermediate_size, experts, top
        self.act, self.router_bias = act, bool(router_bias)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, f = self.hidden_size, self.intermediate_size
        specs = {"router": TensorSpec((self.experts, h), init="normal", std=h ** -0.5 * 2)}
        if self.router_bias:
            specs["router.b"] = TensorSpec((self.experts,), init="normal", std=0.5)
        for e in range(self.experts):
            specs[f"e{e}.up"] = TensorSpec((f, h))
            specs[f"e{e}.down"] = TensorSpec((h, f))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.router = tensors["router"].to(device=runtime.device).to(torch.float32).contiguous()
        self.router_b = runtime.place_vector_f32(tensors["router.b"]) if self.router_bias else None
        self.up = torch.stack([runtime.place_matrix(tensors[f"e{e}.up"]) for e in range(self.experts)])
        self.down = torch.stack([runtime.place_matrix(tensors[f"e{e}.down"]) for e in range(self.experts)])

    # the weighted sum over a token's experts may be left to the consumer (``PairedRows``): see ``forward``
    returns_pieces = True

    def forward(self, x: torch.Tensor, ctx: Any, *, pieces: bool = False) -> "torch.Tensor | PairedRows":
        """``pieces``: return the experts' rows with the pairing instead of their weighted sum, for a consumer that forms the
        sum while it reads the rows anyway (the norm behind this part does)."""

        wide = G.wide_tiles_pay(x.shape[0], self.top, x.dtype, self.hidden_size, self.intermediate_size)
        routing = G.route(x, self.router, self.router_b, top=self.top, wide_tiles=wide)
        hidden = G.expert_linear(x, self.up, routing, gather=True, act=self.act)
        rows = G.expert_linear(hidden, self.down, routing, gather=False, out_dtype=torch.float32)
        if pieces:
            return PairedRows(rows, routing.pair_row, routing.weights)
        return G.combine(rows, routing)
