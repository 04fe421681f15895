"""Choice of the kernel for attention with rules on the scores (soft cap, bias by distance, sink)."""

from __future__ import annotations

from typing import Any

import torch

from . import functional as F


def paged_attention_rules(q: torch.Tensor, cache: Any, ctx: Any, table: torch.Tensor, *, scale: float, window: int = 0,
                          softcap: float = 0.0, slopes: torch.Tensor | None = None, sink: bool = False) -> torch.Tensor:
    """Causal attention of the batch's query tokens ``[N, heads, d]`` over their requests' pages with
    ``S <- cap * tanh(S / cap)``, ``S <- S - slope_h * distance`` and the sink's ``1 +`` in the denominator.

    Both run types: the CUDA-core kernel (one warp per token and head, float32 arithmetic, tiles of 32 keys
    from key 0, so the order of every sum depends on the token's position alone)."""

    return F.paged_attention_simt_rules(
        q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry, block_table=table,
        scale=scale, window=window, softcap=softcap, slopes=slopes, sink=sink,
    )
