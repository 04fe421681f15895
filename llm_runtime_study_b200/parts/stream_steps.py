"""Steps on the residual rows between two runs of layers."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from .base import STREAM_STEPS, ResidualStream, Runtime, StreamStep


@STREAM_STEPS.register("pass_entry")
class PassEntry(StreamStep):
    """The start of pass ``index`` (0-based) of ``passes`` over a run of shared layers: the embedding's
    output is added to the rows (``add_first``; a model leaves it out for the first pass), then row
    ``index`` of the table ``step`` ``[passes, hidden]``.  One launch."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, passes: int, index: int, add_first: bool) -> None:
        if not 0 <= index < passes:
            raise ValueError(f"pass {index} of {passes}")
        self.hidden_size, self.passes, self.index, self.add_first = hidden_size, passes, index, bool(add_first)

    @property
    def reads_first_rows(self) -> bool:
        return self.add_first

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"step": TensorSpec((self.passes, self.hidden_size), init="normal", std=0.1)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.vector = runtime.place_vector_f32(tensors["step"][self.index])

    def forward(self, stream: ResidualStream, ctx: Any, first_rows: torch.Tensor | None) -> None:
        F.add_rows(stream.resid, first_rows if self.add_first else None, None, self.vector)
