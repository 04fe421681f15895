"""Grouped-query causal self-attention over the paged cache."""

from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from ..ops import attention_bf16
from ..ops import attention_rules
from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from ..weights.view import TensorView
from .base import MIXERS, NORMS, POSITION_ENCODINGS, Mixer, PagedKV, PagedTensors, Runtime
from .linear import Projection
from .norm import RMSNorm


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    """q/k/v projections (one stacked product), optional per-head RMS norm of q and
    k *before* the rotation, rotary rotation, write of k and v into the request's
    pages, causal attention of ``num_heads`` query heads over ``num_kv_heads``
    key/value heads (query head j reads KV head ``j // (num_heads/num_kv_heads)``),
    output projection without bias (mini_llm/nn/attention.py:161-181, 250-254,
    291-302; scale ``1/sqrt(head_dim)`` unless given, :95-99).

    Every size is a parameter; the part does not know the model around it.
    """

    def __init__(
        self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
        scale: float | None = None, bias: bool = False, qk_norm: Mapping[str, Any] | None = None,
        position: Mapping[str, Any] | None = None, window: int | None = None, shares_kv: bool = False,
    ) -> None:
        if min(hidden_size, num_heads, num_kv_heads, head_dim) <= 0:
            raise ValueError("attention sizes must be positive")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim % 16:
            raise ValueError(f"head_dim {head_dim} is not a multiple of 16: no kernel takes it")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.bias = bool(bias)
        self.window = window
        # A layer that reads keys and values written by an earlier layer: it has a
        # query and an output projection only, and writes nothing into the cache.
        self.shares_kv = bool(shares_kv)
        self.q_norm = NORMS.build(qk_norm) if qk_norm else None
        self.k_norm = NORMS.build(qk_norm) if qk_norm else None
        if qk_norm and not isinstance(self.q_norm, RMSNorm):
            # the kernel that normalises, rotates and writes the cache in one pass computes an RMS norm
            raise ValueError(f"gqa_attention normalises q and k with an rms_norm only; got the norm kind {qk_norm.get('kind')!r}")
        self.position = POSITION_ENCODINGS.build(position) if position else None

    graph_safe = True

    def children(self):
        return tuple(p for p in (self.q_norm, self.k_norm, self.position) if p is not None)

    # ------------------------------------------------------------- weights
    def tensor_specs(self) -> dict[str, TensorSpec]:
        q_out, kv_out, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.hidden_size
        specs = {
            "q_proj.weight": TensorSpec((q_out, h)),
            "k_proj.weight": TensorSpec((kv_out, h)),
            "v_proj.weight": TensorSpec((kv_out, h)),
            "o_proj.weight": TensorSpec((h, q_out)),
        }
        if self.bias:
            specs.update({
                "q_proj.bias": TensorSpec((q_out,)),
                "k_proj.bias": TensorSpec((kv_out,)),
                "v_proj.bias": TensorSpec((kv_out,)),
            })
        if self.q_norm is not None:
            specs.update({f"q_norm.{n}": s for n, s in self.q_norm.tensor_specs().items()})
            specs.update({f"k_norm.{n}": s for n, s in self.k_norm.tensor_specs().items()})
        if self.shares_kv:
            specs = {n: s for n, s in specs.items() if not n.startswith(("k_", "v_"))}
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        names = ("q_proj",) if self.shares_kv else ("q_proj", "k_proj", "v_proj")
        self.qkv_proj = Projection(
            [tensors[f"{n}.weight"] for n in names],
            [tensors[f"{n}.bias"] for n in names] if self.bias else None,
            runtime,
        )
        self.o_proj = Projection([tensors["o_proj.weight"]], None, runtime)
        if self.q_norm is not None:
            view = TensorView.of(tensors)
            self.q_norm.load(view.sub("q_norm"), runtime)
            if not self.shares_kv:
                self.k_norm.load(view.sub("k_norm"), runtime)
        if self.position is not None:
            self.position.load({}, runtime)

    # --------------------------------------------------------------- cache
    def cache_requirement(self) -> PagedKV | None:
        return None if self.shares_kv else PagedKV(self.num_kv_heads, self.head_dim, self.window)

    # ------------------------------------------------------------- forward
    adds_to_residual = True
    fuses_norms = True

    def forward(self, x: Any, ctx: Any, cache: Any, residual: torch.Tensor | None = None, next_norm: Any = None):
        qkv = self.qkv_proj(x)
        rotary = self.position.rotary_parameters() if self.position is not None else None
        table = ctx.block_table(cache.group)
        written_kv_heads = 0 if self.shares_kv else self.num_kv_heads
        if (ctx.all_decode and qkv.dtype == torch.bfloat16 and qkv.shape[0] == ctx.num_entries and not self.shares_kv
                and (self.position is None or rotary is not None)
                and attention_bf16.fused_decode_supported(self.head_dim, cache.page_size, self.window or 0, rotary[1] if rotary else 0)):
            # one new token per request: the decode kernel normalises, rotates and stores q, k and v itself
            splits = attention_bf16.decode_parts(ctx, qkv.shape[0], self.num_heads, self.num_kv_heads, self.head_dim,
                                                 cache.page_size, 0)
            if splits <= attention_bf16.TMA_MAX_SPLITS:
                out = attention_bf16.decode_attention_fused(
                    qkv, cache.keys, cache.values, num_q_heads=self.num_heads,
                    q_weight=self.q_norm.weight if self.q_norm is not None else None,
                    k_weight=self.k_norm.weight if self.k_norm is not None else None,
                    eps=self.q_norm.eps if self.q_norm is not None else 1.0,
                    inv_freq=rotary[0] if rotary else None, kv_len=ctx.kv_len, block_table=table, scale=self.scale, splits=splits,
                    live=getattr(ctx, "live_parts", None))
                return self.o_proj(out.view(out.shape[0], -1), torch.float32, add_to=residual, next_norm=next_norm)
        if self.position is not None and rotary is None:
            nq, nkv, d = self.num_heads, written_kv_heads, self.head_dim
            q_view = qkv[:, : nq * d].unflatten(1, (nq, d))
            k_view = qkv[:, nq * d : (nq + nkv) * d].unflatten(1, (nkv, d)) if nkv else None
            self.position.apply(q_view, k_view, ctx)
        q = F.qk_norm_rope_write(
            qkv, num_q_heads=self.num_heads, num_kv_heads=written_kv_heads, head_dim=self.head_dim,
            q_weight=self.q_norm.weight if self.q_norm is not None else None,
            k_weight=self.k_norm.weight if self.k_norm is not None and not self.shares_kv else None,
            eps=self.q_norm.eps if self.q_norm is not None else 1.0,
            inv_freq=rotary[0] if rotary else None, rotary_dim=rotary[1] if rotary else 0,
            positions=ctx.positions, token_entry=ctx.token_entry,
            block_table=None if self.shares_kv else table, page_size=cache.page_size,
            k_pool=None if self.shares_kv else cache.keys, v_pool=None if self.shares_kv else cache.values,
        )
        out = ctx.attention(q, cache, scale=self.scale, window=self.window or 0)
        return self.o_proj(out.view(out.shape[0], -1), torch.float32, add_to=residual, next_norm=next_norm)


@MIXERS.register("sink_attention")
class SinkAttention(Mixer):
    """Grouped-query causal attention without rotation, with rules on the scores instead, every one a
    parameter:

    * q and k are RMS-normalised over the *whole* projection (all heads at once, a weight of that width),
      before they are split into heads (``qk_norm_eps``; ``None``: no norm);
    * q is multiplied by the position's temperature ``1 + coef * ln(floor((p + 1) / every) + 1)``
      (``temperature = (coef, every)``);
    * ``S = scale * q.k``; ``S <- softcap * tanh(S / softcap)``; ``S <- S - slope_h * (i - j)`` with
      ``slope_h = 2^(-slope_exponent * (h + 1) / heads)`` for head ``h`` (``slope_exponent = None``: no bias);
    * ``sink``: the weights are ``exp(S_j) / (1 + sum exp(S))``, a key of score 0 that has no value.

    Keys have ``head_dim`` columns, values ``value_dim``.  Tensors: ``q``, ``k``, ``v`` (one stacked product),
    ``q.norm``, ``k.norm``, ``o``.  Positions enter through the temperature and the distance only, so the
    cache holds k and v as they leave the norm.
    """

    graph_safe = True

    def __init__(
        self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int | None = None,
        scale: float | None = None, qk_norm_eps: float | None = None, temperature: tuple[float, int] | None = None,
        softcap: float | None = None, slope_exponent: float | None = None, sink: bool = False, window: int | None = None,
    ) -> None:
        value_dim = head_dim if value_dim is None else value_dim
        if min(hidden_size, num_heads, num_kv_heads, head_dim, value_dim) <= 0:
            raise ValueError("attention sizes must be positive")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim > 256 or value_dim > 256:
            raise ValueError(f"head sizes {head_dim} and {value_dim} must be at most 256: no kernel takes larger ones")
        if temperature is not None and int(temperature[1]) <= 0:
            raise ValueError("the temperature's period must be positive")
        if softcap is not None and softcap <= 0:
            raise ValueError("softcap must be positive")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.temperature = None if temperature is None else (float(temperature[0]), int(temperature[1]))
        self.softcap = None if softcap is None else float(softcap)
        self.slope_exponent = None if slope_exponent is None else float(slope_exponent)
        self.sink, self.window = bool(sink), window

    def tensor_specs(self) -> dict[str, TensorSpec]:
        q_out, k_out, v_out, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim, self.hidden_size
        specs = {
            "q": TensorSpec((q_out, h)), "k": TensorSpec((k_out, h)), "v": TensorSpec((v_out, h)),
            "o": TensorSpec((h, self.num_heads * self.value_dim)),
        }
        if self.qk_norm_eps is not None:
            specs["q.norm"] = TensorSpec((q_out,), init="one_plus_normal", std=0.05)
            specs["k.norm"] = TensorSpec((k_out,), init="one_plus_normal", std=0.05)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.qkv_proj = Projection([tensors["q"], tensors["k"], tensors["v"]], None, runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        self.q_weight = self.k_weight = None
        if self.qk_norm_eps is not None:
            self.q_weight = runtime.place_vector_f32(tensors["q.norm"])
            self.k_weight = runtime.place_vector_f32(tensors["k.norm"])
        self.slopes = None
        if self.slope_exponent is not None:
            # formed in float64, kept in float32
            slopes = [2.0 ** (-self.slope_exponent * (h + 1) / self.num_heads) for h in range(self.num_heads)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def cache_requirement(self) -> PagedTensors:
        return PagedTensors(
            tensors=(("keys", (self.num_kv_heads, self.head_dim)), ("values", (self.num_kv_heads, self.value_dim))),
            window=self.window,
        )

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        qkv = self.qkv_proj(x)
        table = ctx.block_table(cache.group)
        coef, every = self.temperature or (0.0, 0)
        q = F.qk_rownorm_write(
            qkv, num_q_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, value_dim=self.value_dim,
            q_weight=self.q_weight, k_weight=self.k_weight, eps=self.qk_norm_eps or 0.0, temp_coef=coef, temp_every=every,
            positions=ctx.positions, token_entry=ctx.token_entry, block_table=table, page_size=cache.page_size,
            k_pool=cache.keys, v_pool=cache.values,
        )
        out = attention_rules.paged_attention_rules(
            q, cache, ctx, table, scale=self.scale, window=self.window or 0, softcap=self.softcap or 0.0,
            slopes=self.slopes, sink=self.sink,
        )
        return self.o_proj(out.view(out.shape[0], -1), torch.float32)
