"""The Vupitar decoder on the GPU through the engine's own step function, cache manager and
scheduler, against the plain implementation in float64: every way of cutting (whole; most in one
step and the last tokens one by one; portions of changing size down to two tokens; mixed batches of
unequal requests on a poisoned pool), tight pools whose pages and state slots have several owners,
long decoding past many chunks, the first tokens, other page sizes, a request against itself in
other company, captured against eager steps, greedy generation through `LLMEngine` with a
preemption, and the replay program."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.gpu_common import replay
from tests.helpers import mixed_trace, portions_trace, random_tokens, read_weights, tail_decode_trace, whole_trace
from tests.plain import plain_vupitar as pv
from tests.vupitar_configs import VUPITAR, make_vupitar_folder

pytestmark = pytest.mark.gpu
LENGTHS = {"A": [5, 47, 1, 130, 2, 64, 33], "B": [5, 17, 150, 70, 1, 90, 2], "C": [40, 3, 25, 1, 18], "D": [30, 2, 300, 140]}
_cache = {}


def setup(tmp_path_factory, key):
    if key not in _cache:
        folder = make_vupitar_folder(tmp_path_factory.mktemp(f"vupitar_{key}"), key)
        weights = read_weights(folder)
        requests = {f"r{i}": random_tokens(VUPITAR[key]["vocab"], n, 300 + i) for i, n in enumerate(LENGTHS[key])}
        want = {ident: pv.forward(VUPITAR[key], weights, tokens).numpy() for ident, tokens in requests.items()}
        scale = float(np.sqrt(np.mean([np.var(w, axis=-1).mean() for w in want.values()])))
        _cache[key] = (folder, requests, want, scale)
    return _cache[key]


def distance(got, want, scale):
    """Per position: the root mean square over the vocabulary of the difference of the logits, each
    with its mean taken off, in units of the logits' own spread."""
    d = got.astype(np.float64) - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / scale


# float32 kernels against float64: rounding alone stays far below this, a key wrongly seen or missed does not.
# bfloat16: three times what rounding alone causes in that request, measured with the plain implementation
# rounding its products' outputs to bfloat16 (both sides see the weights rounded to bfloat16).
LIMIT_FLOAT32 = 3e-5


CLOSE_CALL = 0.15   # a margin of the router's logits below this may fall the other way once its input is rounded to bfloat16


def check(got, want, scale, limit, what):
    """`limit`: a number, or (number, every position's smallest router margin) from the bfloat16 oracle: which
    expert runs may then hang on the rounding of the router's input, and a token whose expert changed shows in
    every later position of its request.  So the first position over the limit must be such a close call."""
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    err = distance(got, want, scale)
    if isinstance(limit, tuple):
        limit, margin = limit
        if (err > limit).any() and margin[int(np.argmax(err > limit))] < CLOSE_CALL:
            return
    assert err.max() <= limit, f"{what}: position {int(np.argmax(err > limit))} is off by {err.max():.3e} (limit {limit:.1e})"


def rounded_weights(weights):
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 else v) for k, v in weights.items()}


def oracle(key, weights, tokens, dtype, scale=None):
    """(logits, limit) for one request."""
    if dtype == "float32":
        return pv.forward(VUPITAR[key], weights, tokens).numpy(), LIMIT_FLOAT32
    weights = rounded_weights(weights)
    gaps = []
    want = pv.forward(VUPITAR[key], weights, tokens, gaps=gaps).numpy()
    rough = pv.forward(VUPITAR[key], weights, tokens, rounding=True, gaps=gaps).numpy()
    scale = scale or float(np.sqrt(np.var(want, axis=-1).mean()))
    margin = np.full(len(tokens), np.inf) if not gaps else torch.stack(gaps).min(0).values.numpy()
    sure = np.cumsum(margin < CLOSE_CALL) == 0          # the positions before the request's first close call
    return want, (max(2e-2, 3.0 * float(np.where(sure, distance(rough, want, scale), 0.0).max())), margin)


def reference(key, dtype, tmp_path_factory):
    """folder, requests, {id: logits}, scale, {id: limit}"""
    folder, requests, want, scale = setup(tmp_path_factory, key)
    if dtype == "float32":
        return folder, requests, want, scale, {ident: LIMIT_FLOAT32 for ident in requests}
    if key + "/bf16" not in _cache:
        weights = read_weights(folder)
        both = {ident: oracle(key, weights, tokens, dtype, scale) for ident, tokens in requests.items()}
        _cache[key + "/bf16"] = ({i: b[0] for i, b in both.items()}, {i: b[1] for i, b in both.items()})
    want, limits = _cache[key + "/bf16"]
    return folder, requests, want, scale, limits


WAYS = {
    "whole": lambda reqs: whole_trace(reqs),
    "tail": lambda reqs: tail_decode_trace(reqs, 45),
    "portions": lambda reqs: portions_trace(reqs, [7, 2, 5, 3, 2, 15, 16, 17, 2, 31, 33]),
    "mixed": lambda reqs: mixed_trace(reqs, seed=3),
    "mixed_other_order": lambda reqs: mixed_trace(dict(reversed(list(reqs.items()))), seed=11),
}


@pytest.mark.parametrize("way", list(WAYS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("A", 16), ("B", 16), ("A", 8), ("B", 24), ("C", 4), ("C", 32), ("D", 16), ("D", 64)])
def test_replay_matches_plain(tmp_path_factory, key, page, dtype, way):
    folder, requests, want, scale, limits = reference(key, dtype, tmp_path_factory)
    steps = WAYS[way](requests)
    got, session = replay(folder, dtype, steps, poison=way.startswith("mixed"), page_size=page, max_live=4)
    assert session.runner.cache.whole(), "pages or slots were not given back"
    for ident in requests:
        check(got[ident], want[ident], scale, limits[ident], f"{key} page {page} {dtype} {way} {ident}")


def pages_needed(steps, page):
    held, worst = {}, 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-n // page) for n in held.values()))
        for ident in record["end"]:
            held.pop(ident, None)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("A", 8), ("B", 16)])
def test_pages_and_slots_have_several_owners_on_a_tight_pool(tmp_path_factory, key, page, dtype):
    folder, requests, want, scale, limits = reference(key, dtype, tmp_path_factory)
    steps = mixed_trace(requests, seed=5, max_live=3)
    num_pages = pages_needed(steps, page)
    assert num_pages < sum(-(-len(t) // page) for t in requests.values())
    got, session = replay(folder, dtype, steps, num_pages=num_pages, page_size=page, max_live=3, poison=True)
    shared = {pid: owners for pid, owners in session.page_owners.items() if len(owners) > 1}
    assert len({owner for owners in shared.values() for owner in owners}) >= 4
    assert session.runner.cache.whole()
    for ident in requests:
        check(got[ident], want[ident], scale, limits[ident], f"reuse {key} {dtype} {ident}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_long_decoding_token_by_token_past_many_chunks(tmp_path_factory, key, dtype):
    folder, _, _, scale, _ = reference(key, dtype, tmp_path_factory)
    tokens = random_tokens(VUPITAR[key]["vocab"], 260, 9)
    want, limit = oracle(key, read_weights(folder), tokens, dtype, scale)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == 259 else []}
             for i, t in enumerate(tokens)]
    got, session = replay(folder, dtype, steps, page_size=16)
    check(got["x"], want, scale, limit, f"long decode {key} {dtype}")
    assert session.runner.cache.whole()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_first_tokens_of_a_sequence(tmp_path_factory, key, dtype):
    folder, _, _, scale, _ = reference(key, dtype, tmp_path_factory)
    tokens = random_tokens(VUPITAR[key]["vocab"], 4, 77)
    want, limit = oracle(key, read_weights(folder), tokens, dtype, scale)
    one_by_one = [{"step": i, "entries": [{"id": "f", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(tokens)]
    got, _ = replay(folder, dtype, one_by_one, max_tokens=64)
    check(got["f"], want, scale, limit, "first tokens one by one")
    two_two = [{"step": 0, "entries": [{"id": "f", "tokens": tokens[:2], "want": [0, 1]}], "end": []},
               {"step": 1, "entries": [{"id": "f", "tokens": tokens[2:], "want": [0, 1]}], "end": ["f"]}]
    got, _ = replay(folder, dtype, two_two, max_tokens=64)
    check(got["f"], want, scale, limit, "first tokens two and two")


def test_a_request_in_company_equals_itself_alone(tmp_path_factory):
    """float32: the logits of a position change by rounding at most with the cutting and the company."""
    folder, requests, _, scale, _ = reference("B", "float32", tmp_path_factory)
    whole, _ = replay(folder, "float32", whole_trace(requests))
    mixed, _ = replay(folder, "float32", mixed_trace(requests, seed=3), poison=True)
    cut, _ = replay(folder, "float32", portions_trace(requests, [2, 9, 2, 33]))
    for ident in requests:
        assert distance(mixed[ident], whole[ident], scale).max() < 1e-5
        assert distance(cut[ident], whole[ident], scale).max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_captured_decode_steps_equal_eager_ones(tmp_path_factory, key, dtype):
    """Decode steps are replayed from CUDA graphs; the same trace with graphs off gives the same bits."""
    from shrike_b200.replay import TraceSession

    folder, requests, _, _, _ = reference(key, dtype, tmp_path_factory)
    steps = tail_decode_trace({k: v for k, v in list(requests.items())[:3]}, 20)
    results = []
    for graphs in (True, False):
        session = TraceSession(folder, dtype, 512, page_size=16, max_live=4)
        session.runner.use_graphs = graphs
        results.append([session.step(record).copy() for record in steps])
        if graphs:
            assert session.runner.capture_safe and session.runner._graphs, "no decode step was captured"
    for a, b in zip(*results):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_with_portions_equal_eager_ones(tmp_path_factory, dtype):
    """A batch shape with portions is recorded when it has come several times; ten requests fed in two equal
    portions each make one shape come twenty times."""
    from shrike_b200.replay import TraceSession

    folder, _, _, _, _ = reference("A", dtype, tmp_path_factory)
    steps = []
    for index in range(10):
        tokens = random_tokens(VUPITAR["A"]["vocab"], 48, 900 + index)
        for half in (0, 1):
            steps.append({"step": len(steps), "entries": [{"id": f"p{index}", "tokens": tokens[24 * half: 24 * half + 24],
                                                           "want": list(range(24))}], "end": [f"p{index}"] if half else []})
    results = []
    for graphs in (True, False):
        session = TraceSession(folder, dtype, 256, page_size=16, max_live=4)
        session.runner.use_graphs = graphs
        results.append([session.step(record).copy() for record in steps])
        if graphs:
            assert any(not isinstance(key[0], int) for key in session.runner._graphs), "no step with a portion was captured"
    for a, b in zip(*results):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,lengths,new", [("A", (5, 17, 33), 8), ("B", (3, 40, 75), 8)])
def test_greedy_generation_through_the_engine(tmp_path_factory, key, lengths, new, dtype):
    from shrike_b200 import SamplingParams
    from shrike_b200.engine.llm_engine import LLMEngine

    folder, _, _, scale, _ = reference(key, dtype, tmp_path_factory)
    weights = read_weights(folder)
    if dtype == "bfloat16":
        weights = rounded_weights(weights)
    engine = LLMEngine(str(folder), block_size=8, num_blocks=40, max_tokens_per_step=32, dtype=dtype)
    prompts = [random_tokens(VUPITAR[key]["vocab"], n, 30 + n) for n in lengths]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    assert engine.block_manager.whole()
    tie = 12 * scale * (LIMIT_FLOAT32 if dtype == "float32" else 4e-2)   # a top-2 gap within the logits' tolerance is a tie
    for prompt, out in zip(prompts, outs):
        want, margins = pv.greedy_continue(VUPITAR[key], weights, prompt, new)
        for position, (a, b, margin) in enumerate(zip(out, want, margins)):
            if a != b:
                assert margin < tie, f"token {position}: engine {a}, plain {b}, gap {margin}"
                break   # after a tie went the other way the continuations differ


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_survives_preemption_with_state(tmp_path_factory, dtype):
    """A pool too small for three requests at once: one is preempted (pages and state slot returned) and
    computed again later from zero state; every continuation still equals the plain implementation's."""
    from shrike_b200 import SamplingParams
    from shrike_b200.engine.llm_engine import LLMEngine

    folder, _, _, scale, _ = reference("B", dtype, tmp_path_factory)
    weights = read_weights(folder)
    if dtype == "bfloat16":
        weights = rounded_weights(weights)
    engine = LLMEngine(str(folder), block_size=8, num_blocks=15, max_tokens_per_step=32, dtype=dtype)
    prompts = [random_tokens(VUPITAR["B"]["vocab"], n, 60 + n) for n in (30, 31, 29)]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=24, ignore_eos=True))
    assert engine.block_manager.whole() and engine.scheduler.num_preemptions >= 1
    tie = 12 * scale * (LIMIT_FLOAT32 if dtype == "float32" else 4e-2)
    for prompt, out in zip(prompts, outs):
        want, margins = pv.greedy_continue(VUPITAR["B"], weights, prompt, 24)
        for position, (a, b, margin) in enumerate(zip(out, want, margins)):
            if a != b:
                assert margin < tie, f"token {position}: engine {a}, plain {b}, gap {margin}"
                break


def test_trace_run_program_serves_the_design(tmp_path):
    folder = make_vupitar_folder(tmp_path, "A")
    requests = {"a": random_tokens(211, 41, 1), "b": random_tokens(211, 9, 2)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": requests["a"][:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": requests["a"][30:31], "want": []},
                                {"id": "b", "tokens": requests["b"], "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": requests["a"][31:], "want": [9]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    program = Path(__file__).resolve().parents[1] / "bin" / "trace_run"
    run = subprocess.run(
        [sys.executable, str(program), "--model", str(folder), "--dtype", "bfloat16", "--out", str(out), "--max-tokens", "128"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900,
    )
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    weights = read_weights(folder)
    (ref_a, limit_a), (ref_b, limit_b) = oracle("A", weights, requests["a"], "bfloat16"), oracle("A", weights, requests["b"], "bfloat16")
    scale = float(np.sqrt(np.var(ref_a, axis=-1).mean()))
    check(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, 211), ref_a[[0, 29]], scale, limit_a[0], "step 0")
    check(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, 211), ref_b[[8]], scale, limit_b[0], "step 1")
    check(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, 211), ref_a[[40]], scale, limit_a[0], "step 2")


def test_command_line_programs_serve_the_design(tmp_path):
    """The interactive program from a shape without a folder, and the one-prompt program on a folder."""
    import os

    bin_dir = Path(__file__).resolve().parents[1] / "bin"

    def run(program, arguments, text=""):
        done = subprocess.run([sys.executable, str(bin_dir / program), *arguments], input=text, capture_output=True,
                              text=True, timeout=900, env=dict(os.environ, PYTHONUNBUFFERED="1"))
        assert done.returncode == 0, done.stderr[-3000:]
        return done

    done = run("shrike_b200", ["--random", "vupitar-tiny", "--seed", "1", "--num-blocks", "32"], "/temp 0\n/max 4\n1 2 3\n/exit\n")
    assert "shape vupitar-tiny" in done.stdout and "[4 tok |" in done.stdout
    folder = make_vupitar_folder(tmp_path, "A")
    prompt = [7, 200, 41, 41, 2]
    want, margins = pv.greedy_continue(VUPITAR["A"], read_weights(folder), prompt, 6)
    assert min(margins) > 1e-4
    done = run("shrike_b200_complete", [" ".join(map(str, prompt)), "--model", str(folder), "--max-tokens", "6",
                                         "--dtype", "float32", "--num-blocks", "8", "--block-size", "8"])
    assert [int(t) for t in done.stdout.split()] == want
