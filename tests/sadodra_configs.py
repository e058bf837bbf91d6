"""Tiny Sadodra configurations for tests, and model folders with weights that make faults show.

The configurations differ from one another in every size and option: width, vocabulary, head
counts and groups (kv heads fewer than heads, one kv head), key size against value size, latent
ranks that are no multiple of 16, head sizes that are no multiple of 16, windows that differ
from layer to layer or are absent, query temperature with several periods or absent, soft cap
present or absent, a layer without a feed-forward, layers that read another layer's latent, and
the order of the two mixers.
"""

from __future__ import annotations

from pathlib import Path

import torch


def _attention(heads, kv_heads, dim, scale, window=None, temp=None, softcap=None, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if temp is not None:
        mixer["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if softcap is not None:
        mixer["softcap"] = softcap
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _latent(heads, dim, vdim, rank, scale, kv_from=None, ff=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# latent first; a latent rank and a head size that the kernels pad (40 -> 48, 24 -> 32); grouped heads;
# two windows; a layer without feed-forward that reads layer 0's latent with other head counts
SADODRA_A = {
    "architecture": "Sadodra", "width": 96, "vocab": 211, "max_positions": 512, "norm": {"eps": 1e-5},
    "layers": [
        _latent(4, 16, 24, 40, 0.25, ff=160),
        _attention(4, 2, 32, 0.18, window=20, temp=(0.3, 16), softcap=12.0, ff=128),
        _latent(6, 16, 16, 40, 0.3, kv_from=0),
        _attention(3, 3, 24, 0.2, window=37, temp=(0.7, 5), softcap=50.0, ff=64),
    ],
}

# heads of 64 and a rank of 64 (the sizes the page-wise single-token kernel takes); one kv head; an
# attention layer without window, cap and temperature; a period of 1; two readers of one latent
SADODRA_B = {
    "architecture": "Sadodra", "width": 128, "vocab": 300, "max_positions": 640, "norm": {"eps": 1e-6},
    "layers": [
        _attention(4, 1, 64, 0.11, window=70, ff=192),
        _latent(2, 64, 32, 64, 0.15, ff=96),
        _attention(2, 2, 64, 0.09, temp=(0.25, 1), ff=96),
        _latent(3, 32, 48, 64, 0.2, kv_from=1, ff=64),
        _latent(2, 16, 16, 64, 0.35, kv_from=1),
    ],
}

# a single attention layer with a short window, and a single latent layer: each mixer alone
SADODRA_ATTENTION_ONLY = {
    "architecture": "Sadodra", "width": 80, "vocab": 97, "max_positions": 400, "norm": {"eps": 1e-5},
    "layers": [_attention(5, 5, 16, 0.3, window=9, temp=(0.5, 7), softcap=8.0, ff=48)],
}
SADODRA_LATENT_ONLY = {
    "architecture": "Sadodra", "width": 72, "vocab": 101, "max_positions": 400, "norm": {"eps": 1e-5},
    "layers": [_latent(3, 16, 8, 24, 0.4, ff=40)],
}

# a latent wider than the tensor-core attention kernels' heads (300 -> 304 > 256): the CUDA-core kernel serves it
SADODRA_WIDE_LATENT = {
    "architecture": "Sadodra", "width": 64, "vocab": 89, "max_positions": 300, "norm": {"eps": 1e-5},
    "layers": [_latent(2, 16, 16, 300, 0.3, ff=48), _attention(2, 1, 16, 0.3, window=11, ff=32), _latent(3, 8, 8, 300, 0.3, kv_from=0)],
}

SADODRA = {"wide": SADODRA_WIDE_LATENT, "A": SADODRA_A, "B": SADODRA_B, "attention": SADODRA_ATTENTION_ONLY, "latent": SADODRA_LATENT_ONLY}
SADODRA_SEEDS = {"wide": 15, "A": 11, "B": 12, "attention": 13, "latent": 14}


def sharpened(tensors: dict) -> dict:
    """Random weights leave every attention nearly uniform, which hides a key that is wrongly seen or
    missed.  This scales what sets the size of the scores (the query norm's weight, the latent's key
    projection, the query projection of latent layers) so that a softmax row has a few large
    entries (scores a few units apart: more would make the logits hang on single roundings), and gives the position vectors and the norm biases a size that matters."""
    out = {}
    for name, tensor in tensors.items():
        t = tensor.clone()
        if name.endswith(".mix.q.norm"):
            t *= 1.5
        elif name.endswith(".mix.uk"):
            t *= 8.0
        elif name.endswith(".mix.q") and name.replace(".mix.q", ".mix.uk") in tensors:
            t *= 4.0
        elif name == "pos":
            t *= 2.0
        out[name] = t
    return out


def make_sadodra_folder(tmp_path, key: str, dtype: str = "float32", raw: dict | None = None, seed: int | None = None) -> Path:
    """A model folder (config.json, model.safetensors) of a tiny configuration with sharpened weights."""
    import json

    from shrike_b200 import models  # noqa: F401
    from shrike_b200.config.registry import parse_config
    from shrike_b200.weights.random_init import random_tensors
    from shrike_b200.weights.safetensors_io import write_safetensors

    raw = dict(raw if raw is not None else SADODRA[key])
    seed = SADODRA_SEEDS.get(key, 0) if seed is None else seed
    out = Path(tmp_path) / f"sadodra_{key}_{dtype}"
    out.mkdir(parents=True, exist_ok=True)
    config = parse_config(raw)
    tensors = sharpened(random_tensors(config, seed, "cpu", torch.float32))
    tensors = {name: t.to(getattr(torch, dtype)) for name, t in tensors.items()}
    (out / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(out / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return out
