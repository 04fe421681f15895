"""Choice of the kernel for attention over one shared row per token (latent attention with the up-projections moved
to the query's side)."""

from __future__ import annotations

import ctypes
import os
from typing import Any

import torch

from . import attention_bf16, native
from . import functional as F
from .native import c_float, c_int, c_void_p

# "mma": the tensor-core kernel wherever it takes the sizes; "simt": the CUDA-core kernel everywhere
BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_ATTENTION_LATENT", "mma")
ROWS_PER_TILE = 64
MAX_SHARED_BYTES = 227 * 1024

_TABLE = {
    "b200_attention_latent_rank": [],
    "b200_attention_latent_rot": [],
    "b200_attention_latent_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, ctypes.c_long, c_void_p],
}


def library_name(rank: int, rot: int) -> str:
    name = f"b200_attention_latent_r{rank}_t{rot}"
    if name not in native.library_specs():
        native.register_library(name, ("attention_latent.cu",), _TABLE, defines=(f"LATENT_RANK={rank}", f"LATENT_ROT={rot}"))
    return name


def supported(rank: int, rot: int) -> bool:
    """Both widths in steps of 16, values of at most 512 columns, and two key tiles beside the query tile in shared memory."""

    return (rank % 16 == 0 and rot % 16 == 0 and 16 <= rank <= 512 and rot >= 0
            and (ROWS_PER_TILE + 64) * (rank + rot + 8) * 2 <= MAX_SHARED_BYTES)


def build(rank: int, rot: int) -> None:
    from ..csrc.build import build_library

    name = library_name(rank, rot)
    build_library(name, ("attention_latent.cu",), native.library_defines(name))


def latent_attention(q: torch.Tensor, pool: torch.Tensor, ctx: Any, table: torch.Tensor, *, value_dim: int, scale: float,
                     window: int = 0) -> torch.Tensor:
    """Causal attention of the batch's query tokens ``[N, heads, d]`` over their requests' rows ``[pages, page_size, d]``,
    whose first ``value_dim`` columns are the values; result ``[N, heads, value_dim]``.

    bfloat16 with both widths in steps of 16: the mma.sync kernel (prompt portions and single tokens alike: a tile is up to
    ``64 // heads`` consecutive tokens of one request times the heads).  float32, and every other size: the CUDA-core kernel."""

    n, heads, d = q.shape
    rot = d - value_dim
    if BACKEND != "mma" or q.dtype != torch.bfloat16 or not supported(value_dim, rot):
        return F.paged_attention_simt_latent(q, pool, value_dim=value_dim, positions=ctx.positions, token_entry=ctx.token_entry,
                                             block_table=table, scale=scale, window=window)
    per_tile = max(1, ROWS_PER_TILE // heads)
    decode = ctx.all_decode and n == ctx.num_entries
    maps = ctx.__dict__.setdefault("_tile_maps", {})
    key = ("latent", per_tile)
    if key not in maps:
        if decode:
            maps[key] = (_single_token_tiles(n, q.device), n)      # one tile a request
        else:
            maps[key] = attention_bf16.tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
    tiles, count = maps[key]
    out = torch.empty((n, heads, value_dim), dtype=q.dtype, device=q.device)
    splits, scratch, floats = 1, None, 0
    if decode:
        splits = decode_splits(n, heads, min(window, ctx.max_kv_len) if window else ctx.max_kv_len)
        if splits > 1:
            floats = n * heads * splits * (value_dim + 2)
            scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    native.call("b200_attention_latent_bf16", q.data_ptr(), pool.data_ptr(), out.data_ptr(), ctx.positions.data_ptr(), table.data_ptr(),
                table.shape[1], pool.shape[1], heads, float(scale), int(window), tiles[0].data_ptr(), tiles[1].data_ptr(),
                tiles[2].data_ptr(), count, splits, native.ptr(scratch), floats, native.stream_ptr(),
                library=library_name(value_dim, rot), launches=2 if splits > 1 else 1)
    return out


_RAMPS: dict = {}


def _single_token_tiles(n: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(entry, first row, rows) of tiles that are token ``t`` alone: views of a ramp kept per device (made outside a graph
    capture; inside one, where nothing may outlive the graph's pool, a ramp of its own)."""

    if torch.cuda.is_current_stream_capturing():
        ramp = torch.arange(n, dtype=torch.int32, device=device)
        return ramp, ramp, torch.ones_like(ramp)
    kept = _RAMPS.get(device)
    if kept is None or kept[0].shape[0] < n:
        size = max(n, 256)
        kept = _RAMPS[device] = (torch.arange(size, dtype=torch.int32, device=device), torch.ones(size, dtype=torch.int32, device=device))
    return kept[0][:n], kept[0][:n], kept[1][:n]


def decode_splits(requests: int, heads: int, keys: int) -> int:
    """Into how many parts a single token's keys are cut: enough CTAs for two a multiprocessor, no part shorter than four
    tiles of 32 keys, at most 32 parts."""

    ctas = requests * -(-heads // ROWS_PER_TILE)
    wanted = -(-2 * native.sm_count() // max(ctas, 1))
    return max(1, min(wanted, keys // 128, 32))
