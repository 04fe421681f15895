"""Sorulix without a GPU: configuration, description, tensor names, cache layout, the order of runs, and the
plain implementation's own mechanisms against closed forms."""

import copy
import json

import pytest
import torch

from llm_runtime_study_b200.cache import CacheManager
from llm_runtime_study_b200.cache.manager import CacheLayout
from llm_runtime_study_b200.config import SorulixConfig, architecture_for, load_config
from llm_runtime_study_b200.errors import ConfigError, KVCacheError
from llm_runtime_study_b200.models.description import tensor_schema
from llm_runtime_study_b200.models.model import DecoderModel
from llm_runtime_study_b200.models.sorulix import describe_for_checkpoint, describe_sorulix, stored_name
from llm_runtime_study_b200.parts import FixedState, PagedTensors
from llm_runtime_study_b200.weights import Checkpoint
from llm_runtime_study_b200.weights.view import TensorView
from tests import helpers
from tests.plain import sorulix_plain as plain


def test_the_registry_finds_the_design_by_its_architecture_key():
    arch = architecture_for(helpers.SORULIX_A)
    assert arch.name == "Sorulix" and arch.describe_for_checkpoint is not None
    with pytest.raises(ConfigError, match="unsupported architecture"):
        architecture_for({"architecture": "Nobody"})


def test_every_size_and_constant_is_read_from_the_dict():
    cfg = SorulixConfig.from_dict(helpers.SORULIX_A)
    assert (cfg.vocab, cfg.width, cfg.eps, len(cfg.layers)) == (97, 64, 1e-5, 4)
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 3, 3)
    delta, parallel = cfg.layers[0], cfg.layers[1]
    assert (delta.type, delta.mixer.heads, delta.mixer.kv_heads, delta.mixer.dim, delta.mixer.vdim, delta.mixer.conv) == ("channel_delta", 4, 2, 24, 16, 3)
    assert (parallel.mixer.left.heads, parallel.mixer.left.kv_heads, parallel.mixer.left.dim, parallel.mixer.left.vdim) == (4, 2, 16, 24)
    assert (parallel.mixer.left.scale, parallel.mixer.left.softcap, parallel.mixer.left.q_temp) == (0.9, 1.0, (0.5, 3))
    assert parallel.mixer.right.decay == (0.9, 0.5) and (parallel.mixer.right.dim, parallel.mixer.right.vdim) == (8, 40)
    assert cfg.layers[2].mlp is None and (cfg.layers[3].mlp.ff, cfg.layers[3].mlp.limit) == (48, 0.7)
    other = SorulixConfig.from_dict(helpers.SORULIX_B)
    assert other.loop is None and other.layers[0].mixer.left.softcap is None and other.layers[0].mixer.left.q_temp is None


@pytest.mark.parametrize("patch,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.__setitem__("width", True), "width must be int, got bool"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "not a layer of this design"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("softcap", -1.0), "softcap"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"), "not a feed-forward of this design"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop runs layers"),
    (lambda c: c["loop"].__setitem__("times", 0), "times"),
    (lambda c: c.__setitem__("layers", []), "layers must not be empty"),
])
def test_a_bad_config_is_refused_with_the_key_named(patch, match):
    raw = copy.deepcopy(helpers.SORULIX_A)
    patch(raw)
    with pytest.raises(ConfigError, match=match):
        SorulixConfig.from_dict(raw)


def test_the_order_of_runs_and_where_a_pass_starts():
    cfg = SorulixConfig.from_dict(helpers.SORULIX_A)
    assert cfg.runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert cfg.runs() == plain.layer_runs(helpers.SORULIX_A)
    description = describe_sorulix(cfg, helpers.SORULIX_A_RANKS)
    assert description.order == (0, 1, 2, 1, 2, 1, 2, 3)
    assert sorted(description.before_run) == [1, 3, 5]
    assert [description.before_run[r]["add_first"] for r in (1, 3, 5)] == [False, True, True]
    assert [description.before_run[r]["index"] for r in (1, 3, 5)] == [0, 1, 2]
    assert describe_sorulix(SorulixConfig.from_dict(helpers.SORULIX_B)).before_run == {}
    whole = copy.deepcopy(helpers.SORULIX_A)
    whole["loop"] = {"start": 0, "stop": 4, "times": 2}
    assert sorted(describe_sorulix(SorulixConfig.from_dict(whole)).before_run) == [0, 4]


def test_tensor_names_shapes_and_the_sizes_that_only_the_checkpoint_gives(tmp_path):
    cfg = SorulixConfig.from_dict(helpers.SORULIX_A)
    schema = tensor_schema(describe_sorulix(cfg, helpers.SORULIX_A_RANKS))
    assert schema["embed"].shape == (97, 64) and schema["final.norm"].shape == (64,) and schema["loop.step"].shape == (3, 64)
    assert schema["l0.norm1"].shape == (64,) and "l2.norm2" not in schema and "l2.mlp.gate" not in schema
    assert schema["l0.mix.q"].shape == (48, 64) and schema["l0.mix.v"].shape == (64, 64) and schema["l0.mix.q.conv"].shape == (48, 3)
    assert schema["l0.mix.a1"].shape == (5, 64) and schema["l0.mix.a2"].shape == (96, 5) and schema["l0.mix.g2"].shape == (64, 7)
    assert schema["l0.mix.b"].shape == (4, 64) and schema["l0.mix.A_log"].shape == (4,) and schema["l0.mix.norm"].shape == (16,)
    assert schema["l1.mix.left.q"].shape == (64, 64) and schema["l1.mix.left.v"].shape == (48, 64) and schema["l1.mix.left.o"].shape == (64, 96)
    assert schema["l1.mix.left.q.norm"].shape == (64,) and schema["l1.mix.left.k.norm"].shape == (32,)
    assert schema["l1.mix.right.v"].shape == (80, 64) and schema["l1.mix.right.norm"].shape == (80,) and schema["l1.mix.left.out"].shape == (64,)
    assert schema["l1.mlp.gate.b"].shape == (80,) and schema["l1.mlp.down.b"].shape == (64,)
    assert schema["head"].optional and not any(name.endswith(".weight") for name in schema)
    assert stored_name("l3.norm2.weight") == "l3.norm2" and stored_name("l1.mix.left.q") == "l1.mix.left.q"
    # a folder's own shapes decide the inner sizes of the low-rank maps
    path, state = helpers.make_sorulix_dir(tmp_path / "m", helpers.SORULIX_A, helpers.SORULIX_A_RANKS, 3)
    arch, typed = load_config(path)
    checkpoint = Checkpoint.from_model_dir(path)
    described = arch.describe_for_checkpoint(typed, {info.name: info.shape for info in checkpoint.manifest})
    assert set(tensor_schema(described)) - {"head"} == set(state)
    mixer = described.layers[2].block["mixer"]
    assert (mixer["decay_rank"], mixer["gate_rank"]) == (8, 3)
    assert json.loads((path / "config.json").read_text())["architecture"] == "Sorulix"


def test_a_view_under_other_names():
    store = {"a.norm": torch.ones(2), "a.mix.q": torch.zeros(3)}
    view = TensorView.of(store).renamed(stored_name)
    assert "a.norm.weight" in view and "a.norm" in view and "a.mix.q" in view and "a.mix.k" not in view
    sub = view.sub("a").sub("norm")
    assert "weight" in sub and torch.equal(sub["weight"], store["a.norm"])
    with pytest.raises(KeyError):
        view["a.mix.k"]


def test_a_layer_may_ask_for_pages_and_several_arrays():
    model = DecoderModel(describe_sorulix(SorulixConfig.from_dict(helpers.SORULIX_A), helpers.SORULIX_A_RANKS))
    layout = model.cache_layout()
    # runs 1, 3, 5 are layer 1 (keys 16 wide, values 24), run 7 is layer 3 (32 and 32): two groups of pages
    assert [g.layers for g in layout.groups] == [(1, 3, 5), (7,)]
    assert layout.groups[0].requirement.tensors == (("keys", (2, 16)), ("values", (2, 24)))
    names = sorted((s.layer, s.requirement.name, s.requirement.shape) for s in layout.states)
    assert (0, "conv", (2, 160)) in names and (0, "state", (4, 24, 16)) in names and (1, "right.state", (2, 8, 40)) in names
    assert len(names) == 4 * 2 + 4 * 1        # four runs of a delta layer (two arrays each), four of a parallel layer
    manager = CacheManager(layout, max_tokens=64, page_size=4, max_requests=2, dtype=torch.float32, device="cpu")
    cache = manager.layer_cache(1)
    assert cache.group == 0 and cache.keys.shape == (16, 2, 4, 16) and cache.values.shape == (16, 2, 4, 24)
    assert cache.states["right.state"].shape == (3, 2, 8, 40)
    delta = manager.layer_cache(0)
    assert delta.group is None and delta.states["state"].shape == (3, 4, 24, 16) and delta.states["conv"].shape == (3, 2, 160)
    assert delta.state is delta.states["state"]
    # a slot that is taken again starts from zero in every array
    first = manager.admit()
    for array in manager.state_arrays.values():
        array[first.slot] += 1.0
    manager.release(first)
    again = manager.admit()
    assert again.slot == first.slot and all(float(a[again.slot].abs().sum()) == 0.0 for a in manager.state_arrays.values())
    with pytest.raises(KVCacheError, match="pages twice"):
        CacheLayout.from_requirements([(PagedTensors((("a", (1,)),)), PagedTensors((("b", (2,)),)))])
    with pytest.raises(KVCacheError, match="under one name"):
        CacheLayout.from_requirements([(FixedState((1,)), FixedState((2,)))])


# ----------------------------------------------------------- the plain implementation against closed forms
def test_plain_sink_attention_first_token_and_uniform_keys():
    """One key of score 0 beside the sink: half the value.  n equal keys of score s: n e^s / (1 + n e^s)."""

    q, k, v = torch.zeros(1, 1, 4, dtype=torch.float64), torch.zeros(1, 1, 4, dtype=torch.float64), torch.ones(1, 1, 3, dtype=torch.float64)
    assert torch.allclose(plain.sink_attention(q, k, v, scale=1.0, softcap=None, slopes=None), torch.full((1, 1, 3), 0.5, dtype=torch.float64))
    n = 5
    q = torch.ones(n, 1, 2, dtype=torch.float64)
    k = torch.ones(n, 1, 2, dtype=torch.float64)
    v = torch.ones(n, 1, 1, dtype=torch.float64)
    out = plain.sink_attention(q, k, v, scale=0.25, softcap=None, slopes=None)
    e = torch.exp(torch.tensor(0.5, dtype=torch.float64))
    assert torch.allclose(out[:, 0, 0], torch.tensor([(i + 1) * e / (1 + (i + 1) * e) for i in range(n)], dtype=torch.float64))
    capped = plain.sink_attention(100 * q, k, v, scale=1.0, softcap=2.0, slopes=None)       # every score is the cap
    e = torch.exp(torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(capped[-1, 0, 0], n * e / (1 + n * e))


def test_plain_slopes_temperature_and_runs():
    assert torch.allclose(plain.distance_slopes(4), torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    temp = plain.query_temperature(torch.arange(7), 0.5, 3)
    assert torch.allclose(temp[:2], torch.ones(2, dtype=torch.float64)) and torch.allclose(temp[2:5], 1 + 0.5 * torch.log(torch.tensor(2.0, dtype=torch.float64)))


def test_plain_scans_against_closed_forms():
    """Constant decay with k = q = 1, v = 1: a geometric sum.  Delta rule with beta = 1, g = 1 and a repeated unit
    key: the state stores the value exactly, and a second write of the same pair changes nothing."""

    T = 6
    one = torch.ones(T, 1, 1, dtype=torch.float64)
    out = plain.decayed_outer_sum(one, one, one, torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(out[:, 0, 0], torch.tensor([2 - 0.5 ** t for t in range(T)], dtype=torch.float64))
    k = torch.zeros(3, 1, 4, dtype=torch.float64)
    k[:, 0, 1] = 1.0
    v = torch.tensor([[[1.0, 2.0]], [[1.0, 2.0]], [[5.0, -1.0]]], dtype=torch.float64)
    out = plain.gated_delta_scan(k, k, v, torch.ones(3, 1, dtype=torch.float64), torch.ones(3, 1, 4, dtype=torch.float64))
    assert torch.allclose(out[:, 0], v[:, 0])            # each read-out is the value just written for that key
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    x = torch.arange(10, dtype=torch.float64).view(5, 2)
    conv = plain.short_convolution(x, taps)
    assert torch.equal(conv[:, 0], x[:, 0]) and torch.equal(conv[:, 1], torch.tensor([0.0, 0.0, 1.0, 3.0, 5.0], dtype=torch.float64))


def test_plain_feed_forward_limits():
    w = {"m.gate": torch.eye(2, dtype=torch.float64), "m.gate.b": torch.zeros(2, dtype=torch.float64),
         "m.up": torch.eye(2, dtype=torch.float64), "m.up.b": torch.zeros(2, dtype=torch.float64),
         "m.down": torch.eye(2, dtype=torch.float64), "m.down.b": torch.tensor([1.0, 0.0], dtype=torch.float64)}
    out = plain.limited_glu(torch.tensor([[10.0, -10.0]], dtype=torch.float64), w, "m", {"limit": 2.0})
    g = torch.tensor([2.0, -10.0], dtype=torch.float64)
    want = g * plain.sigmoid(1.702 * g) * (torch.tensor([2.0, -2.0], dtype=torch.float64) + 1) + torch.tensor([1.0, 0.0], dtype=torch.float64)
    assert torch.allclose(out[0], want)
