"""Plain, slow Ropulix forward pass: whole sequences, no cache, CPU.

One function per mechanism, elementary torch operations only, nothing shared with the engine.  It takes a
``config.json`` dict and ``{tensor name: tensor}`` with the checkpoint's own names.  ``dtype`` is the arithmetic
type (float64 separates rounding from faults).

``store`` (optional) is applied wherever a serving engine with 16-bit activations keeps a tensor in memory
between two operations: the rows a sublayer reads, the results of projections, q and k as they enter the
attention, the gated read-outs, the experts' hidden rows.  The residual stream, the statistics, the recurrent
state, the router and the logits stay in ``dtype`` either way.

Notation: ``T`` tokens at positions ``0..T-1``; ``unit(x) = x / sqrt(mean(x^2) + eps)`` over the last axis;
every linear map is ``x @ W.T`` with ``W`` stored ``[out, in]``.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch


# ----------------------------------------------------------------- elementary
def keep(x: torch.Tensor) -> torch.Tensor:
    return x


def round_bfloat16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit(x, eps) * w


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------ attention
def window_mask(T: int, window: int | None) -> torch.Tensor:
    """``[T, T]`` True where query i sees key j: ``0 <= i - j`` and, with a window, ``i - j < window``."""

    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def softmax_attention(q, k, v, *, scale: float, window: int | None) -> torch.Tensor:
    """q ``[T, H, d]``, k ``[T, G, d]``, v ``[T, G, dv]`` -> ``[T, H, dv]``; query head h reads key/value head
    ``h // (H / G)``; an ordinary softmax over the keys the mask lets through."""

    T, H, _ = q.shape
    G = k.shape[1]
    seen = window_mask(T, window)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def gated_attention_mixer(h, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, store=keep) -> torch.Tensor:
    """No rotation; q and k made unit vectors per head; a window; one sigmoid gate per head."""

    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ w["q"].T).view(T, H, d)
    k = store(h @ w["k"].T).view(T, G, d)
    v = store(h @ w["v"].T).view(T, G, dv)
    q, k = store(unit(q, eps)), store(unit(k, eps))
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, scale=m["scale"], window=window)
    gate = sigmoid(h @ w["g"].T)                   # [T, H]
    o = store(o * gate[:, :, None])
    return o.reshape(T, H * dv) @ w["o"].T


def rotate_half(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """The first ``dims`` columns of the last axis are rotated: column i pairs with column i + dims/2,
    ``(u, v) -> (u cos a - v sin a, v cos a + u sin a)`` with ``a = p * base^(-2i/dims)``."""

    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]          # [T, half]
    cos, sin = torch.cos(angle).to(x.dtype), torch.sin(angle).to(x.dtype)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = cos.view(shape), sin.view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def latent_kv(h, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, positions, store=keep):
    """What a latent attention layer keeps per token: the normed latent ``c`` and the rotated shared key part."""

    r = m["kv_rank"]
    down = store(h @ w["dkv"].T)
    c = store(rms_norm(down[:, :r], w["dkv.norm"], eps))
    k_rot = store(rotate_half(down[:, r:], positions, m["rot"]["base"], m["rot"]["dims"]))
    return c, k_rot


def latent_attention_mixer(h, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, kept, store=keep) -> torch.Tensor:
    """``kept`` is ``(c, k_rot)`` of this layer or of the layer it borrows them from."""

    T = h.shape[0]
    H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    positions = torch.arange(T)
    c, k_rot = kept
    cq = store(rms_norm(store(h @ w["dq"].T), w["dq.norm"], eps))
    q = store(cq @ w["uq"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], store(rotate_half(q[..., d:], positions, m["rot"]["base"], m["rot"]["dims"]))
    k_plain = store(c @ w["uk"].T).view(T, H, d)
    v = store(c @ w["uv"].T).view(T, H, dv)
    k = torch.cat([k_plain, k_rot[:, None, :].expand(T, H, dr)], dim=-1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(torch.cat([q_plain, q_rot], dim=-1), k, v, scale=m["scale"], window=window)
    gate = sigmoid(h @ w["g"].T)                   # [T, H * dv]
    o = store(o.reshape(T, H * dv) * gate)
    return o @ w["o"].T


# ------------------------------------------------------------------ recurrence
def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x`` ``[T, C]``, ``taps`` ``[C, K]``: the last tap multiplies the current token, zeros before the start."""

    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    out = bias[None, :].expand(T, C).clone()
    for j in range(K):
        out = out + padded[j : j + T] * taps[:, j][None, :]
    return out


def rglru_mixer(h, w: Mapping[str, torch.Tensor], m: Mapping, store=keep) -> torch.Tensor:
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = store(gelu_tanh(store(h @ w["y"].T + w["y.b"])))
    u = store(causal_conv(store(h @ w["x"].T + w["x.b"]), w["conv"], w["conv.b"]))
    ub = u.view(T, blocks, width // blocks)
    r = sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ra"]) + w["ra.b"]).reshape(T, width)
    i = sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ri"]) + w["ri.b"]).reshape(T, width)
    log_a = -8.0 * r * softplus(w["lam"])
    a = torch.exp(log_a)
    inp = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(width, dtype=h.dtype)
    states = []
    for t in range(T):
        S = a[t] * S + inp[t]
        states.append(S)
    return store(torch.stack(states) * y) @ w["o"].T


# ---------------------------------------------------------------- feed-forward
def moe(h, w: Mapping[str, torch.Tensor], m: Mapping, store=keep, margins=None) -> torch.Tensor:
    """``margins`` (a list) receives, per token, how far the last chosen logit lies above the first one left out."""

    experts, top = m["router"]["experts"], m["router"]["top"]
    z = h @ w["router"].T + w["router.b"]
    chosen = torch.topk(z, top, dim=-1)
    if margins is not None and top < experts:
        ranked = torch.sort(z, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top])
    weights = torch.softmax(chosen.values, dim=-1)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for e in range(experts):
        hidden = store(torch.relu(store(h @ w[f"e{e}.up"].T)) ** 2)
        y = hidden @ w[f"e{e}.down"].T
        share = (weights * (chosen.indices == e)).sum(dim=-1)
        out = out + share[:, None] * y
    return out


# ----------------------------------------------------------------------- model
def sub(weights: Mapping[str, torch.Tensor], prefix: str, dtype) -> dict:
    return {k[len(prefix):]: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items() if k.startswith(prefix)}


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, store=keep, layers_out=None,
            margins=None):
    """Logits ``[T, vocab]`` of one sequence.  ``layers_out`` (a list) receives the residual rows after every layer,
    ``margins`` (a list) every router's margins per token (see ``moe``)."""

    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    embed = weights["embed"].to(dtype)
    x = embed[tokens]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        w = sub(weights, f"l{i}.mix.", dtype)
        m = layer["mixer"]
        h = store(x)
        if layer["type"] == "attention":
            out = gated_attention_mixer(h, w, m, eps, store)
        elif layer["type"] == "rglru":
            out = rglru_mixer(h, w, m, store)
        elif layer["type"] == "latent_attention":
            source = m.get("kv_from")
            if source is None:
                kept[i] = latent_kv(h, w, m, eps, positions, store)
                source = i
            out = latent_attention_mixer(h, w, m, eps, kept[source], store)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(out, weights[f"l{i}.norm1"].to(dtype), eps)
        if layer.get("mlp"):
            out = moe(store(x), sub(weights, f"l{i}.mlp.", dtype), layer["mlp"], store, margins)
            x = x + rms_norm(out, weights[f"l{i}.norm2"].to(dtype), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = store(rms_norm(x, weights["final.norm"].to(dtype), eps))
    return x @ embed.T
