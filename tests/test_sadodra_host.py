"""Sadodra on the CPU: the configuration reader, the tensor names, the run order and the caches,
and the whole model stepped through the engine's replay session with the stand-in kernels, against
the plain implementation: whole, in portions down to two tokens, and mixed on a tight pool."""

import numpy as np
import pytest
import torch

import shrike_b200.models  # noqa: F401
from shrike_b200.config import ConfigError, parse_config
from shrike_b200.config.model_config import LatentAttentionSpec, SharedKeyValueAttentionSpec
from shrike_b200.replay import TraceSession
from shrike_b200.weights.expected import expected_tensors
from tests.emulated_ops import EmulatedOps
from tests.helpers import collect, mixed_trace, portions_trace, random_tokens, read_weights, whole_trace
from tests.plain import plain_sadodra as ps
from tests.sadodra_configs import SADODRA, SADODRA_A, SADODRA_B, make_sadodra_folder


def test_config_gives_each_layer_its_parts_and_caches():
    config = parse_config(SADODRA_A)
    assert config.architecture == "Sadodra" and config.num_layers == 4
    kinds = [type(layer.mixer) for layer in config.layers]
    assert kinds == [LatentAttentionSpec, SharedKeyValueAttentionSpec, LatentAttentionSpec, SharedKeyValueAttentionSpec]
    assert config.layers[2].feed_forward is None and config.layers[2].feed_forward_norm is None
    assert not config.layers[2].mixer.own_latent and config.layers[0].mixer.own_latent
    assert [(run.cache, run.writes_cache) for run in config.order] == [(0, True), (1, True), (0, False), (3, True)]
    first = config.layers[1].mixer
    assert (first.window, first.q_temperature, first.softcap, first.num_kv_heads) == (20, (0.3, 16), 12.0, 2)
    assert config.layers[3].mixer.window == 37 and config.layers[0].feed_forward.activation == "gelu_tanh"
    plain = parse_config(SADODRA_B).layers[2].mixer
    assert plain.window is None and plain.softcap is None and plain.q_temperature == (0.25, 1)
    assert parse_config(SADODRA_B).layers[0].mixer.q_temperature is None


def test_tensor_names_follow_the_layers():
    names = expected_tensors(parse_config(SADODRA_A))
    assert {"embed", "pos", "head", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.mix.dkv", "l0.mix.dkv.norm",
            "l0.mix.uk", "l0.mix.uv", "l0.mix.g", "l1.mix.q.norm", "l1.mix.k", "l3.mlp.down"} <= set(names)
    assert "l2.mix.dkv" not in names and "l2.norm2" not in names and "l2.mlp.gate" not in names and "l1.mix.v" not in names
    assert names["l0.mix.uv"].shape == (4 * 24, 40) and names["l2.mix.uk"].shape == (6 * 16, 40)
    assert names["l1.mix.k"].shape == (2 * 32, 96) and names["l1.mix.q.norm"].shape == (4 * 32,) and names["pos"].shape == (512, 96)


@pytest.mark.parametrize("change,text", [
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=1), "caches no latent"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_rank=24), "kv_rank differs"),
    (lambda raw: raw["layers"][1]["mixer"].update(vdim=16), "vdim must equal dim"),
    (lambda raw: raw["layers"][1].update(type="recurrent"), "known: attention"),
    (lambda raw: raw["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda raw: raw.pop("norm"), "norm"),
])
def test_config_errors_name_the_key(change, text):
    import copy

    raw = copy.deepcopy(SADODRA_A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def run(folder, steps, **options):
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), **options)
    outputs = {}
    for record in steps:
        result = session.step(record)
        if result is not None:
            outputs[record["step"]] = result.copy()
    return collect(steps, outputs), session


LENGTHS = [5, 47, 1, 83, 2, 30]


@pytest.mark.parametrize("key", ["A", "B"])
def test_engine_with_stand_in_kernels_matches_plain(tmp_path, key):
    folder = make_sadodra_folder(tmp_path, key)
    weights = read_weights(folder)
    requests = {f"r{i}": random_tokens(SADODRA[key]["vocab"], n, 200 + i) for i, n in enumerate(LENGTHS)}
    want = {ident: ps.forward(SADODRA[key], weights, tokens).numpy() for ident, tokens in requests.items()}
    for steps in (whole_trace(requests), portions_trace(requests, [7, 2, 5, 3, 16, 17, 2]), mixed_trace(requests, seed=4)):
        got, session = run(folder, steps, page_size=8, num_pages=40, max_live=4)
        assert session.runner.cache.whole()
        for ident in requests:
            assert np.abs(got[ident] - want[ident]).max() < 1e-4, ident   # float32 kernels against float64


def test_windowed_groups_give_pages_back_and_latent_pages_have_one_plane(tmp_path):
    folder = make_sadodra_folder(tmp_path, "A")
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), page_size=4, num_pages=64, max_live=2)
    groups = session.runner.groups
    assert sorted((g.window or 0, g.planes, g.head_dim, g.cache_ids) for g in groups) == [
        (0, 1, 48, (0,)), (20, 2, 32, (1,)), (37, 2, 32, (3,))]
    latent = [i for i, g in enumerate(groups) if g.planes == 1][0]
    assert session.runner.storage.kv[latent].shape[1] == 1
    tokens = random_tokens(211, 120, 5)
    session.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": []}], "end": []})
    tables = session.live["a"][0].tables
    for group, table in zip(groups, tables):
        released = int((table.view() < 0).sum())
        assert released == (0 if group.window is None else (120 - group.window + 1) // 4)
