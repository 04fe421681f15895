"""Ropulix without a GPU: configuration, description, tensor names, cache layout, and the plain implementation's own
mechanisms against closed forms."""

import copy
import math

import pytest
import torch

from llm_runtime_study_b200.cache.manager import CacheLayout
from llm_runtime_study_b200.config import RopulixConfig, architecture_for
from llm_runtime_study_b200.errors import ConfigError
from llm_runtime_study_b200.models.description import tensor_schema
from llm_runtime_study_b200.models.model import DecoderModel
from llm_runtime_study_b200.models.ropulix import describe_ropulix
from llm_runtime_study_b200.parts import FixedState, PagedTensors
from tests import helpers
from tests.plain import ropulix_plain as plain


def test_the_registry_finds_the_design_by_its_architecture_key():
    assert architecture_for(helpers.ROPULIX_A).name == "Ropulix"


def test_every_size_and_constant_is_read_from_the_dict():
    cfg = RopulixConfig.from_dict(helpers.ROPULIX_A)
    assert (cfg.vocab, cfg.width, cfg.eps, len(cfg.layers)) == (211, 64, 1e-5, 5)
    latent, attention, recurrence, borrower, last = (layer.mixer for layer in cfg.layers)
    assert (latent.heads, latent.dim, latent.rot_dim, latent.vdim, latent.kv_rank, latent.q_rank) == (3, 16, 8, 24, 40, 48)
    assert (latent.window, latent.rot_base, latent.rot_dims, latent.scale, latent.kv_from) == (9, 1000.0, 8, 0.35, None)
    assert (attention.heads, attention.kv_heads, attention.dim, attention.vdim, attention.window, attention.scale) == (4, 1, 16, 16, 5, 0.3)
    assert (recurrence.width, recurrence.blocks, recurrence.conv) == (96, 3, 4)
    assert (borrower.kv_from, borrower.window) == (0, 13) and last.window is None
    assert cfg.layers[1].mlp is None
    assert (cfg.layers[3].mlp.experts, cfg.layers[3].mlp.top, cfg.layers[3].mlp.ff) == (4, 1, 32)


@pytest.mark.parametrize("patch,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.__setitem__("width", True), "width must be int, got bool"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "not a layer of this design"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("blocks", 5), "multiple of blocks"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "not a feed-forward of this design"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "exceeds experts"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_rank", 24), "borrows the latent"),
    (lambda c: c.__setitem__("layers", []), "layers must not be empty"),
])
def test_a_bad_config_is_refused_with_the_key_named(patch, match):
    raw = copy.deepcopy(helpers.ROPULIX_A)
    patch(raw)
    with pytest.raises(ConfigError, match=match):
        RopulixConfig.from_dict(raw)


def test_tensor_names_and_shapes():
    schema = tensor_schema(describe_ropulix(RopulixConfig.from_dict(helpers.ROPULIX_A)))
    shapes = {name: tuple(spec.shape) for name, spec in schema.items() if not spec.optional}
    assert shapes["embed"] == (211, 64) and shapes["final.norm"] == (64,) and shapes["l0.norm1"] == (64,)
    assert shapes["l0.mix.dq"] == (48, 64) and shapes["l0.mix.dq.norm"] == (48,) and shapes["l0.mix.uq"] == (3 * 24, 48)
    assert shapes["l0.mix.dkv"] == (48, 64) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (48, 40) and shapes["l0.mix.uv"] == (72, 40) and shapes["l0.mix.g"] == (72, 64) and shapes["l0.mix.o"] == (64, 72)
    assert "l3.mix.dkv" not in shapes and "l3.mix.dkv.norm" not in shapes and shapes["l3.mix.uk"] == (16, 40)
    assert shapes["l1.mix.q"] == (64, 64) and shapes["l1.mix.k"] == (16, 64) and shapes["l1.mix.g"] == (4, 64) and "l1.norm2" not in shapes
    assert shapes["l4.mix.v"] == (16, 64) and shapes["l4.mix.o"] == (64, 16)
    assert shapes["l2.mix.x"] == (96, 64) and shapes["l2.mix.y.b"] == (96,) and shapes["l2.mix.conv"] == (96, 4) and shapes["l2.mix.conv.b"] == (96,)
    assert shapes["l2.mix.ra"] == (3, 32, 32) and shapes["l2.mix.ri.b"] == (3, 32) and shapes["l2.mix.lam"] == (96,)
    assert shapes["l2.mlp.router"] == (3, 64) and shapes["l2.mlp.router.b"] == (3,) and shapes["l2.mlp.e2.up"] == (24, 64) and shapes["l2.mlp.e0.down"] == (64, 24)
    assert "l2.mlp.e3.up" not in shapes


def test_cache_layout_follows_the_mixers():
    """The latent layer keeps one row per token, read as far back as the widest window among its readers; the borrowing
    layer keeps nothing; attention layers with different masks have pages of their own; the recurrence keeps a state row
    and the convolution's last inputs (none where the convolution has a single tap)."""

    model = DecoderModel(describe_ropulix(RopulixConfig.from_dict(helpers.ROPULIX_A)))
    assert model.description.cache_of == (None, None, None, 0, None)
    layout = model.cache_layout()
    by_layers = {group.layers: group.requirement for group in layout.groups}
    assert by_layers[(0,)] == PagedTensors(tensors=(("latent", (48,)),), window=13)
    assert by_layers[(1,)] == PagedTensors(tensors=(("keys", (1, 16)), ("values", (1, 16))), window=5)
    assert by_layers[(4,)] == PagedTensors(tensors=(("keys", (2, 24)), ("values", (2, 8))), window=None)
    states = {(s.layer, s.requirement.name): s.requirement for s in layout.states}
    assert states == {(2, "state"): FixedState((96,), torch.float32, "state"), (2, "conv"): FixedState((3, 96), torch.float32, "conv")}
    other = DecoderModel(describe_ropulix(RopulixConfig.from_dict(helpers.ROPULIX_B))).cache_layout()
    assert {(s.layer, s.requirement.name) for s in other.states} == {(0, "state"), (3, "state"), (3, "conv")}
    assert [g.requirement.window for g in other.groups] == [33, None]
    assert isinstance(layout, CacheLayout)


# ------------------------------------------------------------- the plain implementation against closed forms
def test_plain_window_and_softmax():
    seen = plain.window_mask(6, 3)
    assert seen.tolist()[4] == [False, False, True, True, True, False] and seen.tolist()[0] == [True] + [False] * 5
    assert plain.window_mask(4, None).tolist()[3] == [True] * 4
    q = torch.zeros(5, 1, 2, dtype=torch.float64)
    v = torch.arange(5, dtype=torch.float64).view(5, 1, 1)
    out = plain.softmax_attention(q, q, v, scale=1.0, window=2)       # equal scores: the mean of the visible values
    assert torch.allclose(out.flatten(), torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5], dtype=torch.float64))


def test_plain_rotation_and_norms():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0]], dtype=torch.float64)
    out = plain.rotate_half(x, torch.tensor([3]), 100.0, 4)
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0),
            4 * math.cos(a1) + 2 * math.sin(a1), 5.0]
    assert torch.allclose(out[0], torch.tensor(want, dtype=torch.float64))
    assert torch.allclose(plain.rotate_half(x, torch.tensor([0]), 100.0, 4), x)
    u = plain.unit(torch.tensor([[3.0, 4.0]], dtype=torch.float64), 0.0)
    assert torch.allclose(u, torch.tensor([[3.0, 4.0]], dtype=torch.float64) / math.sqrt(12.5))


def test_plain_convolution_recurrence_and_experts():
    x = torch.arange(1.0, 5.0, dtype=torch.float64).view(4, 1)
    out = plain.causal_conv(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert out.flatten().tolist() == [1.5, 12.5, 123.5, 234.5]
    # a recurrence whose gates are shut (r -> 0) keeps a = 1 and lets nothing in; with r -> 1 and a large lam nothing is kept
    w = {"y": torch.zeros(2, 2), "y.b": torch.full((2,), 3.0), "x": torch.eye(2), "x.b": torch.zeros(2), "conv": torch.ones(2, 1),
         "conv.b": torch.zeros(2), "ra": torch.zeros(1, 2, 2), "ra.b": torch.tensor([[-40.0, 40.0]]), "ri": torch.zeros(1, 2, 2),
         "ri.b": torch.full((1, 2), 40.0), "lam": torch.full((2,), 5.0), "o": torch.eye(2)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.tensor([[1.0, 1.0], [2.0, 2.0]], dtype=torch.float64)
    out = plain.rglru_mixer(h, w, {"width": 2, "blocks": 1})
    y = float(plain.gelu_tanh(torch.tensor(3.0, dtype=torch.float64)))
    assert torch.allclose(out[:, 0], torch.zeros(2, dtype=torch.float64), atol=1e-6)
    assert torch.allclose(out[:, 1], torch.tensor([1.0, 2.0], dtype=torch.float64) * y, atol=1e-6)
    # experts: two of three chosen, weights from the chosen logits only
    m = {"router": {"experts": 3, "top": 2}}
    w = {"router": torch.tensor([[1.0], [3.0], [2.0]]), "router.b": torch.zeros(3)}
    for e in range(3):
        w[f"e{e}.up"], w[f"e{e}.down"] = torch.tensor([[float(e + 1)]]), torch.tensor([[1.0]])
    w = {k: v.double() for k, v in w.items()}
    out = plain.moe(torch.tensor([[1.0]], dtype=torch.float64), w, m)
    p = math.exp(3) / (math.exp(3) + math.exp(2))
    assert abs(float(out) - (p * 4.0 + (1 - p) * 9.0)) < 1e-12
    assert float(plain.moe(torch.tensor([[-1.0]], dtype=torch.float64), w, m)) == 0.0       # relu shuts every expert


def test_a_size_the_configuration_leaves_out_comes_from_the_stored_shapes():
    from llm_runtime_study_b200.models.ropulix import describe_for_checkpoint

    raw = copy.deepcopy(helpers.ROPULIX_B)
    del raw["layers"][2]["mixer"]["q_rank"]
    config = RopulixConfig.from_dict(raw)
    with pytest.raises(ConfigError, match="q_rank"):
        describe_ropulix(config)
    schema = tensor_schema(describe_for_checkpoint(config, {"l2.mix.dq": (20, 48)}))
    assert tuple(schema["l2.mix.dq"].shape) == (20, 48) and tuple(schema["l2.mix.uq"].shape) == (40, 20)
