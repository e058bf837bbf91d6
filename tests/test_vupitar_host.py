"""Vupitar on the CPU: the configuration reader, the tensor names, the run order with its passes, the
caches (pages that chunks give back, one state slot a request), and the whole model stepped through
the engine's replay session with the stand-in kernels, against the plain implementation: whole, in
portions down to two tokens, and mixed on a tight pool."""

import copy

import numpy as np
import pytest
import torch

import shrike_b200.models  # noqa: F401
from shrike_b200.cache.manager import CacheManager, KVGroupSpec
from shrike_b200.config import ConfigError, parse_config
from shrike_b200.config.model_config import GatedHeadAttentionSpec, GatedMLPSpec, MatrixMemorySpec, RoutedExpertsSpec
from shrike_b200.replay import TraceSession
from shrike_b200.weights.expected import expected_tensors
from tests.emulated_ops import EmulatedOps
from tests.helpers import collect, mixed_trace, portions_trace, random_tokens, read_weights, whole_trace
from tests.plain import plain_vupitar as pv
from tests.vupitar_configs import VUPITAR, VUPITAR_A, VUPITAR_B, VUPITAR_C, VUPITAR_D, make_vupitar_folder


def test_config_gives_each_layer_its_parts_and_every_run_its_cache():
    config = parse_config(VUPITAR_A)
    assert config.architecture == "Vupitar" and config.num_layers == 3
    assert [(run.layer, run.cache, run.enter) for run in config.order] == [
        (0, 0, None), (1, 1, 0), (2, 2, None), (1, 3, 1), (2, 4, None)]
    assert config.pass_entry.passes == 2 and config.embedding.scale == 1.7
    left, right = (branch for _, branch, _ in config.layers[0].mixer.branches)
    assert isinstance(left, GatedHeadAttentionSpec) and isinstance(right, MatrixMemorySpec)
    assert (left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim, left.chunk, left.rotary) == (4, 2, 32, 16, 20, (16, 10000.0))
    assert (right.num_heads, right.head_dim, right.value_dim, right.gate_cap) == (3, 16, 24, 8.0)
    assert [scale for _, _, scale in config.layers[2].mixer.branches] == [1.2, 0.6]
    kinds = [type(layer.feed_forward) for layer in config.layers]
    assert kinds == [RoutedExpertsSpec, GatedMLPSpec, type(None)] and config.layers[2].feed_forward_norm is None
    assert (config.layers[1].feed_forward.activation, config.layers[1].feed_forward.limit) == ("clamped_swish", 0.8)
    routed = config.layers[0].feed_forward
    assert (routed.experts, routed.top, routed.intermediate, routed.shared_intermediate) == (5, 2, 40, 24)
    plain = parse_config(VUPITAR_B)
    assert plain.pass_entry is None and [run.enter for run in plain.order] == [None] * 3
    assert plain.layers[1].feed_forward.shared_intermediate is None
    once = parse_config(VUPITAR_C)
    assert [(run.layer, run.enter) for run in once.order] == [(0, 0), (1, None)]
    assert parse_config(VUPITAR_D).layers[0].mixer.branches[0][1].chunk is None
    assert [(run.layer, run.cache, run.enter) for run in parse_config(VUPITAR_D).order] == [(0, 0, 0), (0, 1, 1), (0, 2, 2), (1, 3, None)]


def test_tensor_names_follow_the_layers():
    names = expected_tensors(parse_config(VUPITAR_A))
    assert {"embed", "loop.step", "head", "final.norm", "final.norm.b", "final.norm.alpha", "l0.norm1", "l0.norm1.b",
            "l0.norm1.alpha", "l0.norm2.alpha", "l0.mix.left.q", "l0.mix.left.q.b", "l0.mix.left.q.norm", "l0.mix.left.g",
            "l0.mix.left.o.b", "l0.mix.right.i", "l0.mix.right.i.b", "l0.mix.right.f.b", "l0.mix.right.norm",
            "l0.mlp.router", "l0.mlp.e4.down", "l0.mlp.shared.gate", "l0.mlp.shared.sg", "l1.mlp.gate", "l1.mlp.down"} <= set(names)
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names and "l0.mlp.e5.gate" not in names and "l1.mlp.router" not in names
    assert names["loop.step"].shape == (2, 96) and names["l0.norm1.alpha"].shape == ()
    assert names["l0.mix.left.q"].shape == (4 * 32, 96) and names["l0.mix.left.v"].shape == (2 * 16, 96)
    assert names["l0.mix.left.q.norm"].shape == (32,) and names["l0.mix.left.g"].shape == (4, 96)
    assert names["l0.mix.left.o"].shape == (96, 4 * 16) and names["l0.mix.right.g"].shape == (3 * 24, 96)
    assert names["l0.mix.right.k"].shape == (3 * 16, 96) and names["l0.mix.right.f"].shape == (3, 96)
    assert names["l0.mlp.shared.sg"].shape == (1, 96) and names["l0.mlp.e0.gate"].shape == (40, 96)
    assert "loop.step" not in expected_tensors(parse_config(VUPITAR_B))


@pytest.mark.parametrize("change,text", [
    (lambda raw: raw["layers"][0].update(type="serial"), "known: parallel"),
    (lambda raw: raw["layers"][0]["mixer"]["left"].pop("kv_heads"), "kv_heads"),
    (lambda raw: raw["layers"][0]["mixer"]["left"]["rot"].update(dims=34), "rotary dims"),
    (lambda raw: raw["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda raw: raw["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda raw: raw["layers"][0]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda raw: raw["layers"][0]["mlp"]["router"].update(top=6), "top=6"),
    (lambda raw: raw["layers"][1]["mlp"].update(kind="sparse"), "known: dense, moe"),
    (lambda raw: raw["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda raw: raw["loop"].update(stop=4), "loop runs layers"),
    (lambda raw: raw.pop("norm"), "norm"),
])
def test_config_errors_name_the_key(change, text):
    raw = copy.deepcopy(VUPITAR_A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_chunked_groups_give_back_the_pages_of_earlier_chunks():
    manager = CacheManager([KVGroupSpec((0,), 1, 16, chunk=20), KVGroupSpec((1,), 1, 16)], page_size=4, num_pages=[64, 64], max_slots=2)
    assert manager.groups[0].span == 20 and manager.groups[1].span is None
    assert [manager.groups[0].first_needed(p) for p in (0, 19, 20, 39, 40, 41)] == [0, 0, 20, 20, 40, 40]
    cache = manager.open()
    manager.append(cache, 0, 50)
    manager.advance(cache, 50)        # the next query, at 50, sees keys from 40 on: pages 0 .. 9 are behind it
    chunked, kept = cache.tables
    assert list(chunked.view() < 0) == [True] * 10 + [False] * 3 and (kept.view() >= 0).all()
    assert manager.num_free == [64 - 3, 64 - 13]
    manager.append(cache, 50, 31)     # through 80: the chunk from 80 on starts a page
    manager.advance(cache, 81)
    assert int((cache.tables[0].view() < 0).sum()) == 20
    manager.free(cache)
    assert manager.whole()


def run(folder, steps, **options):
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), **options)
    outputs = {}
    for record in steps:
        result = session.step(record)
        if result is not None:
            outputs[record["step"]] = result.copy()
    return collect(steps, outputs), session


LENGTHS = [5, 47, 1, 83, 2, 30]


@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_engine_with_stand_in_kernels_matches_plain(tmp_path, key):
    folder = make_vupitar_folder(tmp_path, key)
    weights = read_weights(folder)
    requests = {f"r{i}": random_tokens(VUPITAR[key]["vocab"], n, 200 + i) for i, n in enumerate(LENGTHS)}
    want = {ident: pv.forward(VUPITAR[key], weights, tokens).numpy() for ident, tokens in requests.items()}
    spread = float(np.sqrt(np.mean([np.var(w, axis=-1).mean() for w in want.values()])))
    for steps in (whole_trace(requests), portions_trace(requests, [7, 2, 5, 3, 16, 17, 2]), mixed_trace(requests, seed=4)):
        got, session = run(folder, steps, page_size=8, num_pages=40, max_live=4)
        assert session.runner.cache.whole()
        for ident in requests:
            assert np.abs(got[ident] - want[ident]).max() < 2e-4 * max(1.0, spread), ident   # float32 stand-ins against float64


def test_a_request_holds_one_state_slot_and_the_pages_of_its_chunk(tmp_path):
    folder = make_vupitar_folder(tmp_path, "A")
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), page_size=4, num_pages=64, max_live=2)
    groups = session.runner.groups
    assert sorted((g.chunk, g.head_dim, g.num_kv_heads, g.cache_ids) for g in groups) == [(20, 32, 2, (0, 1, 3)), (33, 16, 3, (2, 4))]
    state = session.runner.storage.state
    assert sorted(state) == [0, 1, 2, 3, 4]
    assert tuple(state[0].shape) == (2, 3, 16 * 24 + 16 + 4) and tuple(state[2].shape) == (2, 2, 24 * 8 + 24 + 4)
    tokens = random_tokens(211, 70, 5)
    session.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": []}], "end": []})
    tables = session.live["a"][0].tables
    for group, table in zip(groups, tables):
        assert int((table.view() < 0).sum()) == (70 // group.chunk * group.chunk) // 4
    slot = session.live["a"][0].slot
    assert float(state[0][slot].abs().sum()) > 0 and float(state[0][1 - slot].abs().sum()) == 0
    session.step({"step": 1, "entries": [], "end": ["a"]})
    assert session.runner.cache.whole()
    # the slot's next owner starts from zero state although the kernels left the old one's behind
    session.step({"step": 2, "entries": [{"id": "b", "tokens": tokens[:3], "want": []}], "end": []})
    session.step({"step": 3, "entries": [{"id": "c", "tokens": tokens[:3], "want": []}], "end": []})
    b, c = session.live["b"][0].slot, session.live["c"][0].slot
    assert b != c and torch.equal(state[0][b], state[0][c]) and torch.equal(state[4][b], state[4][c])
