"""Tiny Vupitar configurations for tests, and model folders with weights that make faults show.

The configurations differ from one another in every size and option: width, vocabulary, head counts
and groups (kv heads fewer than heads, one kv head, as many as heads), key size against value size,
rotated dimensions fewer than the head's or all of it or none, chunks that are no multiple of a
page, smaller than a page, of one position, or absent, memory heads whose sizes are no multiple of
16 or differ between keys and values, dense and routed feed-forwards in either order or none, experts
of which all, one or some are chosen, with and without a shared expert, and the repeated layers at
the start, in the middle, at the end, once, or not at all.
"""

from __future__ import annotations

from pathlib import Path

import torch


def _layer(left, right, scales, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]},
            "mlp": mlp}


def _left(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None):
    spec = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        spec["mask"] = {"size": chunk}
    if rot is not None:
        spec["rot"] = {"dims": rot[0], "base": rot[1]}
    return spec


def _right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff, shared=None):
    spec = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        spec["shared"] = {"ff": shared}
    return spec


# the repeated layers in the middle and at the end; values narrower than keys; a rotation of half a head; a chunk that
# no page size divides; a layer without a feed-forward; experts first, dense second
VUPITAR_A = {
    "architecture": "Vupitar", "width": 96, "vocab": 211, "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(_left(4, 2, 32, 16, 0.2, chunk=20, rot=(16, 10000.0)), _right(3, 16, 24, 8.0), (0.7, 1.3), _moe(5, 2, 40, shared=24)),
        _layer(_left(4, 2, 32, 16, 0.2, chunk=20, rot=(16, 10000.0)), _right(3, 16, 24, 8.0), (0.7, 1.3), _dense(80, 0.8)),
        _layer(_left(6, 3, 16, 16, 0.3, chunk=33, rot=(8, 500.0)), _right(2, 24, 8, 3.0), (1.2, 0.6), None),
    ],
}

# heads of 64 with one kv head (the sizes the tensor-core kernels take); the whole head rotates; no repeated layers;
# every expert chosen and no shared expert; a limit that never clamps
VUPITAR_B = {
    "architecture": "Vupitar", "width": 128, "vocab": 300, "embedding": {"scale": 0.25}, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_left(2, 1, 64, 64, 0.12, chunk=37, rot=(64, 1000000.0)), _right(1, 64, 64, 15.0), (1.0, 1.0), _dense(192, 7.0)),
        _layer(_left(2, 1, 64, 64, 0.12, chunk=37, rot=(64, 1000000.0)), _right(1, 64, 64, 15.0), (1.0, 1.0), _moe(3, 3, 32)),
        _layer(_left(4, 4, 64, 32, 0.1, chunk=64, rot=(32, 100.0)), _right(2, 32, 64, 15.0), (0.5, 2.0), _moe(4, 1, 48, shared=16)),
    ],
}

# chunks of one position and of fewer positions than a page; one pass "repeated" once; as many kv heads as heads; one
# expert chosen; two rotated dimensions; memory heads of 40 by 8 and 8 by 40; a gate cap near 1
VUPITAR_C = {
    "architecture": "Vupitar", "width": 72, "vocab": 97, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
    "loop": {"start": 0, "stop": 1, "times": 1},
    "layers": [
        _layer(_left(3, 3, 16, 48, 0.3, chunk=1, rot=(2, 10.0)), _right(2, 40, 8, 1.5), (0.9, 1.1), _moe(6, 1, 24, shared=8)),
        _layer(_left(2, 1, 48, 16, 0.25, chunk=5), _right(3, 8, 40, 2.5), (1.1, 0.9), _dense(40, 0.3)),
    ],
}

# heads of 128, no chunk at all (every earlier key is seen), the repeated layers at the very start, three passes
VUPITAR_D = {
    "architecture": "Vupitar", "width": 64, "vocab": 151, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 1, "times": 3},
    "layers": [
        _layer(_left(2, 1, 128, 128, 0.09, rot=(64, 10000.0)), _right(2, 16, 16, 10.0), (1.0, 0.8), _dense(96, 1.0)),
        _layer(_left(1, 1, 128, 128, 0.09, chunk=130, rot=(128, 10000.0)), _right(1, 48, 48, 10.0), (0.8, 1.0), _moe(8, 3, 16, shared=32)),
    ],
}

VUPITAR = {"A": VUPITAR_A, "B": VUPITAR_B, "C": VUPITAR_C, "D": VUPITAR_D}
VUPITAR_SEEDS = {"A": 21, "B": 22, "C": 23, "D": 24}


def sharpened(tensors: dict) -> dict:
    """Random weights leave every attention nearly uniform, every gate at a half and every router undecided, which
    hides a key that is wrongly seen, a state that was lost or an expert that was mistaken.  This scales what sets
    the size of the scores (the query norm's weight), of the memory's gates and of the router, and gives the pass
    vectors and the norms' biases a size that matters."""
    out = {}
    for name, tensor in tensors.items():
        t = tensor.clone()
        if name.endswith(".left.q.norm"):
            t *= 4.0
        elif name.endswith((".right.i", ".right.f")):
            t *= 40.0
        elif name.endswith((".right.i.b", ".right.f.b")):
            t *= 50.0
        elif name.endswith(".router"):
            t *= 60.0
        elif name.endswith((".left.g", ".shared.sg")):
            t *= 30.0
        elif name == "loop.step" or name.endswith((".norm1.b", ".norm2.b", ".q.b", ".k.b", ".v.b", ".o.b")):
            t *= 10.0
        elif name.endswith((".gate", ".up")):
            t *= 8.0       # so that the dense feed-forward's clamp is met
        out[name] = t
    return out


def make_vupitar_folder(tmp_path, key: str, dtype: str = "float32", raw: dict | None = None, seed: int | None = None) -> Path:
    """A model folder (config.json, model.safetensors) of a tiny configuration with sharpened weights."""
    import json

    from shrike_b200 import models  # noqa: F401
    from shrike_b200.config.registry import parse_config
    from shrike_b200.weights.random_init import random_tensors
    from shrike_b200.weights.safetensors_io import write_safetensors

    raw = dict(raw if raw is not None else VUPITAR[key])
    seed = VUPITAR_SEEDS.get(key, 0) if seed is None else seed
    out = Path(tmp_path) / f"vupitar_{key}_{dtype}"
    out.mkdir(parents=True, exist_ok=True)
    config = parse_config(raw)
    tensors = sharpened(random_tensors(config, seed, "cpu", torch.float32))
    tensors = {name: t.to(getattr(torch, dtype)) for name, t in tensors.items()}
    (out / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(out / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return out
