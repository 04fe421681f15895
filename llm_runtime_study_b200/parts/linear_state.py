"""Mixers that keep a state of fixed size per request, and mixers run side by side."""

from __future__ import annotations

from typing import Any, Mapping, Sequence

import torch

from ..ops import functional as F
from ..ops import sequence_state as S
from ..weights.checkpoint import TensorSpec
from ..weights.view import TensorView
from .base import MIXERS, FixedState, Mixer, PagedTensors, Runtime
from .linear import Projection


def _padded(weights: list[torch.Tensor], runtime: Runtime) -> Projection:
    """One stacked product; zero rows bring the number of outputs to a multiple of eight, so that every
    kernel's rows of results start on 16-byte boundaries whatever the sizes are."""

    rows = sum(w.shape[0] for w in weights)
    pad = -rows % 8
    if pad:
        weights = [*weights, torch.zeros((pad, weights[0].shape[1]), dtype=weights[0].dtype)]
    return Projection(weights, None, runtime)


@MIXERS.register("decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """Linear attention with one constant decay per head: ``q = silu(W_q x)``, ``k = silu(W_k x)``
    (``heads x dim``), ``v = silu(W_v x)`` (``heads x vdim``); per head ``S_t = decay_h S_(t-1) + k_t v_t^T``,
    ``o_t = S_t^T q_t``; the heads together are RMS-normalised with the weight ``norm``, multiplied by
    ``sigmoid(W_g x)`` and projected by ``W_o``.  The state ``[heads, dim, vdim]`` is float32, starts at
    zero and lives in the request's slot.  Tensors: ``q``, ``k``, ``v``, ``g`` (one stacked product), ``norm``, ``o``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: Sequence[float], eps: float) -> None:
        if min(hidden_size, num_heads, head_dim, value_dim) <= 0 or head_dim > 256:
            raise ValueError("linear attention sizes must be positive, the key size at most 256")
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.decay, self.eps = tuple(float(d) for d in decay), float(eps)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        qk, vw, h = self.num_heads * self.head_dim, self.num_heads * self.value_dim, self.hidden_size
        return {
            "q": TensorSpec((qk, h)), "k": TensorSpec((qk, h)), "v": TensorSpec((vw, h)), "g": TensorSpec((vw, h)),
            "norm": TensorSpec((vw,), init="one_plus_normal", std=0.05), "o": TensorSpec((h, vw)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.in_proj = _padded([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        self.norm_weight = runtime.place_vector_f32(tensors["norm"])
        self.decays = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def cache_requirement(self) -> FixedState:
        return FixedState((self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        proj = self.in_proj(x)
        qk, vw = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        out = S.linear_scan(
            proj[:, :qk], proj[:, qk : 2 * qk], proj[:, 2 * qk : 2 * qk + vw], heads=self.num_heads, qk_heads=self.num_heads,
            dim=self.head_dim, vdim=self.value_dim, state=cache.state, q_start=ctx.q_start, slots=ctx.slots, decay=self.decays,
            silu=True, fixed_order=self.runtime.dtype == torch.float32,
        )
        gated = S.group_norm_gate(out, self.norm_weight, self.eps, proj, gate_offset=2 * qk + vw, out_dtype=self.runtime.dtype)
        return self.o_proj(gated, torch.float32)


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """The delta rule with one decay per head and key channel.  ``q``, ``k`` (``qk_heads x dim``) and ``v``
    (``heads x vdim``) each pass a causal convolution over time per channel (``taps`` taps, the last one the
    current token's, zeros before the start) and SiLU; q and k become unit vectors per head
    (``x / sqrt(sum x^2 + unit_eps)``), q also times ``dim^(-1/2)``.  ``beta = sigmoid(W_b x)`` per head;
    ``g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 x) + dt_bias))`` per head and key channel.  Per head, in this
    order: ``S <- diag(g) S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``.  Each head's ``o`` is
    divided by its root mean square, times ``norm`` (``vdim``, shared by the heads), times
    ``sigmoid(W_g2 (W_g1 x))``, then ``W_o``.  Head ``h`` reads q/k head ``h // (heads / qk_heads)``.

    Per request: the float32 state ``[heads, dim, vdim]`` and the last ``taps - 1`` inputs of the convolutions.
    Tensors: ``q``, ``k``, ``v``, ``b``, ``a1``, ``g1`` (one stacked product), ``q.conv``, ``k.conv``, ``v.conv``,
    ``A_log``, ``dt_bias``, ``a2``, ``g2``, ``norm``, ``o``."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, value_dim: int, taps: int,
                 decay_rank: int, gate_rank: int, eps: float, unit_eps: float = 1e-6) -> None:
        if min(hidden_size, num_heads, num_qk_heads, head_dim, value_dim, taps, decay_rank, gate_rank) <= 0 or head_dim > 256:
            raise ValueError("delta rule sizes must be positive, the key size at most 256")
        if num_heads % num_qk_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_qk_heads {num_qk_heads}")
        self.hidden_size, self.num_heads, self.num_qk_heads = hidden_size, num_heads, num_qk_heads
        self.head_dim, self.value_dim, self.taps = head_dim, value_dim, taps
        self.decay_rank, self.gate_rank, self.eps, self.unit_eps = decay_rank, gate_rank, float(eps), float(unit_eps)
        self.channels = 2 * num_qk_heads * head_dim + num_heads * value_dim

    def tensor_specs(self) -> dict[str, TensorSpec]:
        qk, vw, hd, h = self.num_qk_heads * self.head_dim, self.num_heads * self.value_dim, self.num_heads * self.head_dim, self.hidden_size
        conv = dict(init="normal", std=0.5)
        return {
            "q": TensorSpec((qk, h)), "k": TensorSpec((qk, h)), "v": TensorSpec((vw, h)),
            "q.conv": TensorSpec((qk, self.taps), **conv), "k.conv": TensorSpec((qk, self.taps), **conv),
            "v.conv": TensorSpec((vw, self.taps), **conv),
            "b": TensorSpec((self.num_heads, h)), "A_log": TensorSpec((self.num_heads,), init="normal", std=0.5),
            "a1": TensorSpec((self.decay_rank, h)), "a2": TensorSpec((hd, self.decay_rank)),
            "dt_bias": TensorSpec((hd,), init="normal", std=0.5),
            "g1": TensorSpec((self.gate_rank, h)), "g2": TensorSpec((vw, self.gate_rank)),
            "norm": TensorSpec((self.value_dim,), init="one_plus_normal", std=0.05), "o": TensorSpec((h, vw)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.in_proj = _padded([tensors[n] for n in ("q", "k", "v", "b", "a1", "g1")], runtime)
        self.o_proj = Projection([tensors["o"]], None, runtime)
        self.conv_taps = torch.cat([runtime.place_vector_f32(tensors[f"{n}.conv"]) for n in ("q", "k", "v")], dim=0)
        self.a_log = runtime.place_vector_f32(tensors["A_log"])
        self.dt_bias = runtime.place_vector_f32(tensors["dt_bias"])
        # the second halves of the low-rank maps are applied inside the kernels, which read them transposed
        self.a_up = runtime.place_matrix(tensors["a2"]).t().contiguous()
        self.g_up = runtime.place_matrix(tensors["g2"]).t().contiguous()
        self.norm_weight = runtime.place_vector_f32(tensors["norm"])

    def cache_requirement(self):
        return (
            FixedState((self.num_heads, self.head_dim, self.value_dim), torch.float32, name="state"),
            FixedState((self.taps - 1, self.channels), torch.float32, name="conv"),
        )

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        proj = self.in_proj(x)
        beta_offset = self.channels
        low_offset = beta_offset + self.num_heads
        gate_offset = low_offset + self.decay_rank
        q, k, v, g, beta = S.delta_prepare(
            proj, heads=self.num_heads, qk_heads=self.num_qk_heads, dim=self.head_dim, vdim=self.value_dim,
            beta_offset=beta_offset, low_offset=low_offset, rank=self.decay_rank, taps=self.conv_taps,
            conv_state=cache.states["conv"], a_log=self.a_log, dt_bias=self.dt_bias, a_up=self.a_up, q_start=ctx.q_start,
            slots=ctx.slots, token_entry=ctx.token_entry, unit_eps=self.unit_eps, q_scale=self.head_dim ** -0.5,
        )
        if self.taps > 1:
            S.conv_state_update(proj, cache.states["conv"], ctx.q_start, ctx.slots)
        out = S.linear_scan(
            q, k, v, heads=self.num_heads, qk_heads=self.num_qk_heads, dim=self.head_dim, vdim=self.value_dim,
            state=cache.states["state"], q_start=ctx.q_start, slots=ctx.slots, gate=g, beta=beta,
            fixed_order=self.runtime.dtype == torch.float32,
        )
        gated = S.group_norm_gate(out, self.norm_weight, self.eps, proj, gate_offset=gate_offset, gate_up=self.g_up,
                                  out_dtype=self.runtime.dtype)
        return self.o_proj(gated, torch.float32)


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    """Several mixers side by side on the same rows.  Each branch's output is RMS-normalised over the model
    width with a weight of its own (``<name>.out``); the result is the mean of the normalised outputs.
    ``branches`` is a list of ``{"name": ..., "mixer": {...}}``; a branch's tensors live under its name.
    What the branches keep per request is asked for together: pages from at most one of them, arrays of
    fixed size under ``<name>.<array>``."""

    def __init__(self, *, hidden_size: int, eps: float, branches: Sequence[Mapping[str, Any]]) -> None:
        if not branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.branches = [(str(b["name"]), MIXERS.build(b["mixer"])) for b in branches]
        if len({name for name, _ in self.branches}) != len(self.branches):
            raise ValueError("two branches of a parallel mixer share a name")

    graph_safe = True

    def children(self):
        return tuple(mixer for _, mixer in self.branches)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for name, mixer in self.branches:
            specs.update({f"{name}.{n}": s for n, s in mixer.tensor_specs().items()})
            specs[f"{name}.out"] = TensorSpec((self.hidden_size,), init="one_plus_normal", std=0.05)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        view = TensorView.of(tensors)
        self.out_weights = []
        for name, mixer in self.branches:
            mixer.load(view.sub(name), runtime)
            self.out_weights.append(runtime.place_vector_f32(view[f"{name}.out"]))

    @staticmethod
    def _needs(mixer: Mixer) -> tuple:
        need = mixer.cache_requirement()
        return tuple(need) if isinstance(need, (tuple, list)) else (() if need is None else (need,))

    def cache_requirement(self):
        needs = []
        for name, mixer in self.branches:
            for need in self._needs(mixer):
                needs.append(FixedState(need.shape, need.dtype, name=f"{name}.{need.name}") if isinstance(need, FixedState) else need)
        return tuple(needs)

    def _branch_cache(self, name: str, mixer: Mixer, cache: Any) -> Any:
        from ..cache.manager import LayerCache

        needs = self._needs(mixer)
        states = {need.name: cache.states[f"{name}.{need.name}"] for need in needs if isinstance(need, FixedState)}
        if any(isinstance(need, PagedTensors) for need in needs):
            return LayerCache(group=cache.group, tensors=cache.tensors, page_size=cache.page_size, states=states)
        return LayerCache(states=states)

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        total = None
        for (name, mixer), weight in zip(self.branches, self.out_weights):
            out = mixer.forward(x, ctx, self._branch_cache(name, mixer, cache))
            total = F.rmsnorm_accumulate(out, weight, self.eps, 1.0 / len(self.branches), total)
        return total
