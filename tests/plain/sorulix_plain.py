"""Plain, slow Sorulix forward pass: whole sequences, no cache, CPU.

One function per mechanism, elementary torch operations only, nothing shared with
the engine.  It takes a ``config.json`` dict and ``{tensor name: tensor}`` with the
checkpoint's own names.  ``dtype`` is the arithmetic type (float64 separates
rounding from faults).

``store`` (optional) is applied wherever a serving engine with 16-bit activations keeps a tensor in
memory between two operations: normalised rows, the results of projections, q and k as they enter the
attention, a mixer's gated read-out, the gated feed-forward rows.  With ``store=round_bfloat16`` the plain
model carries those roundings; the residual stream, the statistics, the states and the logits stay in
``dtype`` either way.

Notation: ``T`` tokens at positions ``0..T-1``; ``rms(x) = x / sqrt(mean(x^2) + eps)``
over the last axis; every linear map is ``x @ W.T`` with ``W`` stored ``[out, in]``.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch


# ----------------------------------------------------------------- elementary
def keep(x: torch.Tensor) -> torch.Tensor:
    return x


def round_bfloat16(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest bfloat16 and widen again."""

    return x.to(torch.bfloat16).to(x.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms keep their weight as an offset from one: ``rms(x) * (1 + w)``."""

    return rms(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


# ------------------------------------------------------------- softmax attention
def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """``1 + coef * ln(floor((p + 1) / every) + 1)``, one factor per position."""

    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def distance_slopes(heads: int) -> torch.Tensor:
    """``2^(-8 (h + 1) / H)`` for head ``h``."""

    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def sink_attention(q, k, v, *, scale: float, softcap: float | None, slopes: torch.Tensor | None) -> torch.Tensor:
    """q ``[T, H, d]``, k ``[T, G, d]``, v ``[T, G, dv]`` -> ``[T, H, dv]``.  Scores are scaled, squashed by
    ``cap * tanh(s / cap)``, lowered by ``slope_h * (i - j)``, masked causally, and turned into weights
    ``exp(s_j) / (1 + sum exp(s))``: a sink with score 0 that carries no value."""

    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    idx = torch.arange(T)
    dist = (idx[:, None] - idx[None, :]).to(q.dtype)
    visible = idx[None, :] <= idx[:, None]
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[h].to(q.dtype) * dist
        e = torch.where(visible, torch.exp(s), torch.zeros_like(s))
        out[:, h] = (e / (1.0 + e.sum(dim=-1, keepdim=True))) @ v[:, g]
    return out


def left_mixer(h, w: Mapping[str, torch.Tensor], p: str, c: Mapping, eps: float, store=keep) -> torch.Tensor:
    """The softmax half of a parallel mixer; ``p`` is the prefix of its tensors."""

    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = norm_plain(store(h @ w[f"{p}.q"].T), w[f"{p}.q.norm"], eps)       # over the whole projection, before the split
    k = store(norm_plain(store(h @ w[f"{p}.k"].T), w[f"{p}.k.norm"], eps))
    v = store(h @ w[f"{p}.v"].T)
    temp = c.get("q_temp")
    if temp:
        q = q * query_temperature(torch.arange(T), temp["coef"], temp["every"]).to(h.dtype)[:, None]
    q = store(q)
    o = sink_attention(q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv), scale=c["scale"],
                       softcap=c.get("softcap"), slopes=distance_slopes(H))
    return store(o).reshape(T, H * dv) @ w[f"{p}.o"].T


# ------------------------------------------------------------- linear attention
def decayed_outer_sum(q, k, v, decay: torch.Tensor) -> torch.Tensor:
    """q, k ``[T, H, d]``, v ``[T, H, dv]``: ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``."""

    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay.to(q.dtype)[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def right_mixer(h, w, p: str, c: Mapping, eps: float, store=keep) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = c["heads"], c["dim"], c["vdim"]
    q = silu(store(h @ w[f"{p}.q"].T)).view(T, H, d)
    k = silu(store(h @ w[f"{p}.k"].T)).view(T, H, d)
    v = silu(store(h @ w[f"{p}.v"].T)).view(T, H, dv)
    o = decayed_outer_sum(q, k, v, torch.tensor(c["decay"], dtype=torch.float64)).reshape(T, H * dv)
    o = store(norm_plain(o, w[f"{p}.norm"], eps) * sigmoid(store(h @ w[f"{p}.g"].T)))
    return o @ w[f"{p}.o"].T


def parallel_mixer(h, w, p: str, c: Mapping, eps: float, store=keep) -> torch.Tensor:
    """Both halves read the same rows; each output is normalised over the model width; the mean of the two."""

    left = norm_plain(left_mixer(h, w, f"{p}.left", c["left"], eps, store), w[f"{p}.left.out"], eps)
    right = norm_plain(right_mixer(h, w, f"{p}.right", c["right"], eps, store), w[f"{p}.right.out"], eps)
    return 0.5 * (left + right)


# ------------------------------------------------------------------ delta rule
def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x ``[T, C]``, taps ``[C, K]`` (the last column meets the current token), zeros before the start."""

    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat((torch.zeros(K - 1, C, dtype=x.dtype), x))
    out = torch.zeros_like(x)
    for j in range(K):
        out = out + padded[j : j + T] * taps[:, j]
    return out


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_scan(q, k, v, beta, g) -> torch.Tensor:
    """q, k, g ``[T, H, d]``, v ``[T, H, dv]``, beta ``[T, H]``.  Per head, in this order:
    ``S <- g * S`` (rows), ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``."""

    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def channel_delta_mixer(h, w, p: str, c: Mapping, eps: float, store=keep) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(short_convolution(store(h @ w[f"{p}.q"].T), w[f"{p}.q.conv"])).view(T, G, d)
    k = silu(short_convolution(store(h @ w[f"{p}.k"].T), w[f"{p}.k.conv"])).view(T, G, d)
    v = silu(short_convolution(store(h @ w[f"{p}.v"].T), w[f"{p}.v.conv"])).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = sigmoid(store(h @ w[f"{p}.b"].T))
    rate = torch.exp(w[f"{p}.A_log"])[None, :, None]
    step = softplus(store(h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.dt_bias"]).view(T, H, d)
    g = torch.exp(-rate * step)
    o = gated_delta_scan(q, k, v, beta, g)                      # [T, H, dv]
    o = norm_plain(o, w[f"{p}.norm"], eps)
    o = store(o * sigmoid(store(h @ w[f"{p}.g1"].T) @ w[f"{p}.g2"].T).view(T, H, dv))
    return o.reshape(T, H * dv) @ w[f"{p}.o"].T


# ---------------------------------------------------------------- feed-forward
def limited_glu(h, w, p: str, c: Mapping, store=keep) -> torch.Tensor:
    limit = c["limit"]
    g = torch.clamp(store(h @ w[f"{p}.gate"].T + w[f"{p}.gate.b"]), max=limit)
    u = torch.clamp(store(h @ w[f"{p}.up"].T + w[f"{p}.up.b"]), min=-limit, max=limit)
    y = store(g * sigmoid(1.702 * g) * (u + 1.0))
    return y @ w[f"{p}.down"].T + w[f"{p}.down.b"]


# ----------------------------------------------------------------------- model
def layer_runs(config: Mapping) -> list[tuple[int, int | None]]:
    """(layer, number of the pass that starts with this run or None), in execution order."""

    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(weights: Mapping[str, torch.Tensor], config: Mapping, token_ids, dtype: torch.dtype = torch.float64,
            *, layers_out: list | None = None, store=keep) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence."""

    w = {n: t.to(dtype) for n, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(token_ids, dtype=torch.long)]
    first = x.clone()
    for index, starts_pass in layer_runs(config):
        if starts_pass is not None:
            if starts_pass > 0:
                x = x + first
            x = x + w["loop.step"][starts_pass]
        layer, p = config["layers"][index], f"l{index}"
        h = store(norm_around_zero(x, w[f"{p}.norm1"], eps))
        if layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, f"{p}.mix", layer["mixer"], eps, store)
        elif layer["type"] == "channel_delta":
            x = x + channel_delta_mixer(h, w, f"{p}.mix", layer["mixer"], eps, store)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp"):
            x = x + limited_glu(store(norm_around_zero(x, w[f"{p}.norm2"], eps)), w, f"{p}.mlp", layer["mlp"], store)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = store(norm_around_zero(x, w["final.norm"], eps))
    return x @ w["embed"].T
