"""Kernels of mixers that keep a state of fixed size per request: the linear scan (plain or delta
rule, constant or per-row decay), the short convolution's bookkeeping, and the gated group norm of
the read-out.  The state and everything that enters the recurrence are float32."""

from __future__ import annotations

import torch

from ..errors import KernelError
from .native import call, ptr, require, stream_ptr, tag


def linear_scan(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, heads: int, qk_heads: int, dim: int, vdim: int,
    state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, gate: torch.Tensor | None = None,
    decay: torch.Tensor | None = None, beta: torch.Tensor | None = None, silu: bool = False, fixed_order: bool = False,
) -> torch.Tensor:
    """Per request (entry ``e`` owns rows ``q_start[e] .. q_start[e+1]-1`` and the state row ``slots[e]``) and head,
    token after token: ``S <- D S + k u^T``, ``o = S^T q`` with ``D`` the head's constant ``decay`` or the row's
    ``gate`` factors (one per key channel), and ``u = v`` or, with ``beta``, ``beta (v - (D S)^T k)``.  ``q`` and
    ``k`` are ``[N, qk_heads * dim]`` column blocks (a row stride of their own is fine), ``v`` ``[N, heads * vdim]``;
    head ``h`` reads q/k head ``h // (heads / qk_heads)``.  ``silu`` applies SiLU to q, k and v as they are read.
    ``state`` is ``[slots, heads, dim, vdim]`` float32 and is updated in place.  ``fixed_order``: every sum is formed in
    an order that does not depend on the shape of the batch (the kernel otherwise spreads a column over more lanes when few
    requests bring long portions), so a token's bits do not depend on the cut.  Returns float32 ``[N, heads * vdim]``."""

    n = q.shape[0]
    for t, name, width in ((q, "q", qk_heads * dim), (k, "k", qk_heads * dim), (v, "v", heads * vdim)):
        if t.device.type != "cuda" or t.dim() != 2 or t.shape != (n, width) or t.stride(1) != 1 or t.dtype != q.dtype:
            raise KernelError(f"{name} must be CUDA rows [{n}, {width}] of one type with unit column stride")
    require(state, "state", dtype=torch.float32, dims=4)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"state has shape {tuple(state.shape)}, expected [slots, {heads}, {dim}, {vdim}]")
    require(q_start, "q_start", dtype=torch.int32, dims=1)
    entries = q_start.shape[0] - 1
    require(slots, "slots", dtype=torch.int32, shape=(entries,))
    if (gate is None) == (decay is None):
        raise KernelError("linear_scan takes either per-row gate factors or one decay per head")
    if gate is not None:
        require(gate, "gate", dtype=torch.float32, shape=(n, heads * dim))
    else:
        require(decay, "decay", dtype=torch.float32, shape=(heads,))
    if beta is not None:
        require(beta, "beta", dtype=torch.float32, shape=(n, heads))
    out = torch.empty((n, heads * vdim), dtype=torch.float32, device=q.device)
    call("b200_linear_scan", ptr(q), ptr(k), ptr(v), q.stride(0), k.stride(0), v.stride(0), ptr(gate), heads * dim, ptr(decay),
         ptr(beta), heads, ptr(state), ptr(out), heads * vdim, ptr(q_start), ptr(slots), entries, n, heads, qk_heads, dim, vdim,
         1 if silu else 0, 1 if fixed_order else 0, tag(q.dtype), stream_ptr())
    return out


def delta_prepare(
    proj: torch.Tensor, *, heads: int, qk_heads: int, dim: int, vdim: int, beta_offset: int, low_offset: int, rank: int,
    taps: torch.Tensor, conv_state: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, a_up: torch.Tensor,
    q_start: torch.Tensor, slots: torch.Tensor, token_entry: torch.Tensor, unit_eps: float, q_scale: float,
):
    """From one stacked projection ``[N, q | k | v | ...]``: the short convolution over time and SiLU of every q, k
    and v channel (inputs before the step come from ``conv_state`` ``[slots, taps-1, channels]``), each q and k head
    divided by ``sqrt(sum of squares + unit_eps)`` (q times ``q_scale``), ``beta = sigmoid(proj[:, beta_offset + h])``
    and the decay factors ``exp(-exp(a_log[h]) * softplus(proj[:, low_offset : low_offset + rank] @ a_up + dt_bias))``
    (``a_up`` is ``[rank, heads * dim]``: the map's weight transposed, so that neighbouring threads read neighbouring outputs).
    Returns float32 ``(q, k, v, g, beta)``."""

    require(proj, "proj", dims=2)
    n, ld = proj.shape
    channels = 2 * qk_heads * dim + heads * vdim
    require(taps, "taps", dtype=torch.float32, dims=2)
    ntaps = taps.shape[1]
    if taps.shape[0] != channels:
        raise KernelError(f"taps has {taps.shape[0]} channels, expected {channels}")
    require(conv_state, "conv_state", dtype=torch.float32, dims=3)
    if tuple(conv_state.shape[1:]) != (ntaps - 1, channels):
        raise KernelError(f"conv_state has shape {tuple(conv_state.shape)}, expected [slots, {ntaps - 1}, {channels}]")
    require(a_log, "a_log", dtype=torch.float32, shape=(heads,))
    require(dt_bias, "dt_bias", dtype=torch.float32, shape=(heads * dim,))
    require(a_up, "a_up", dtype=proj.dtype, shape=(rank, heads * dim))
    if max(beta_offset + heads, low_offset + rank, channels) > ld:
        raise KernelError("delta_prepare: a column block lies outside the projection")
    dev = proj.device
    q = torch.empty((n, qk_heads * dim), dtype=torch.float32, device=dev)
    k = torch.empty_like(q)
    v = torch.empty((n, heads * vdim), dtype=torch.float32, device=dev)
    g = torch.empty((n, heads * dim), dtype=torch.float32, device=dev)
    beta = torch.empty((n, heads), dtype=torch.float32, device=dev)
    call("b200_delta_prepare", ptr(proj), ld, beta_offset, low_offset, rank, ptr(taps), ntaps, ptr(conv_state), ptr(a_log),
         ptr(dt_bias), ptr(a_up), ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(q_start), ptr(slots), ptr(token_entry),
         n, heads, qk_heads, dim, vdim, float(unit_eps), float(q_scale), tag(proj.dtype), stream_ptr())
    return q, k, v, g, beta


def conv_state_update(proj: torch.Tensor, conv_state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor) -> None:
    """After a step: every entry's slot keeps the last ``taps - 1`` inputs of its sequence (columns ``0 .. channels-1``
    of ``proj``), oldest first; a step shorter than that keeps the tail of what the slot held."""

    require(proj, "proj", dims=2)
    require(conv_state, "conv_state", dtype=torch.float32, dims=3)
    entries = q_start.shape[0] - 1
    call("b200_conv_state_update", ptr(proj), proj.shape[1], ptr(conv_state), conv_state.shape[2], conv_state.shape[1] + 1,
         ptr(q_start), ptr(slots), entries, tag(proj.dtype), stream_ptr())


def group_norm_gate(x: torch.Tensor, weight: torch.Tensor, eps: float, gate_in: torch.Tensor, *, gate_offset: int = 0,
                    gate_up: torch.Tensor | None = None, out_dtype: torch.dtype) -> torch.Tensor:
    """``x`` float32 ``[N, width]`` in groups of ``len(weight)`` columns: each group divided by its root mean square,
    times ``weight``, times ``sigmoid(logit)``; the logits are columns ``gate_offset ..`` of ``gate_in`` (``width`` of
    them), or, with ``gate_up`` ``[rank, width]`` (a low-rank map's weight transposed),
    ``gate_in[:, gate_offset : gate_offset + rank] @ gate_up``."""

    require(x, "x", dtype=torch.float32, dims=2)
    n, width = x.shape
    require(weight, "weight", dtype=torch.float32, dims=1)
    group = weight.shape[0]
    if width % group:
        raise KernelError(f"width {width} is not a multiple of the group size {group}")
    require(gate_in, "gate_in", dtype=out_dtype, dims=2)
    rank = 0
    if gate_up is not None:
        require(gate_up, "gate_up", dtype=out_dtype, dims=2)
        rank = gate_up.shape[0]
        if gate_up.shape[1] != width:
            raise KernelError(f"gate_up has {gate_up.shape[1]} columns, expected {width}")
    if gate_offset + (rank or width) > gate_in.shape[1]:
        raise KernelError("group_norm_gate: the gate's columns lie outside gate_in")
    out = torch.empty((n, width), dtype=out_dtype, device=x.device)
    gate_ptr = gate_in.data_ptr() + gate_offset * gate_in.element_size()
    call("b200_group_norm_gate", ptr(x), n, width, group, ptr(weight), float(eps), gate_ptr, gate_in.shape[1], rank,
         ptr(gate_up), ptr(out), tag(out_dtype), stream_ptr())
    return out
