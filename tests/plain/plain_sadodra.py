"""Plain, slow, whole-sequence implementation of the Sadodra decoder.

One function per mechanism, written from the design's equations; no cache, no
batching, no code shared with the `shrike_b200` package.  It reads the raw
`config.json` dictionary and a name -> tensor dictionary itself.

The design in this file's notation (x: residual stream [n, W], p: position from 0):

  x0          = embed[token] + pos[p]
  layer       : x <- x + LN1(mixer(x)); x <- x + LN2(ff(x))      (the norm sits on the branch's
                output; both branches read x itself)
  LN(y)       = (y - mean y) / sqrt(var y + eps) * w + b
  ff(h)       = Wd (gelu_tanh(Wg h) * (Wu h))
  attention   : q = Wq h, k = Wk h, v = k (as projected, before its norm)
                q, k <- RMS over the WHOLE projection (all heads at once) * weight
                q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))
                s_ij = cap * tanh(scale * q_i.k_j / cap) - slope_h * (i - j),
                slope_h = 2^(-8 (h + 1) / H); i sees j with 0 <= i - j < window; softmax
  latent attn : c = RMS(Wdkv h) * weight (or the latent of the layer `kv_from` names)
                k_h = Wuk_h c, v_h = Wuv_h c, s_ij = scale * q_i.k_j, causal softmax,
                head h's output times sigmoid(Wg h)_h, then Wo
  logits      = head LN_final(x)

`rounding=True` rounds to bfloat16 where a bfloat16 engine may (products' outputs and
activations); norms, scores, softmax, the residual sum and positions stay in the working
precision, as the design asks.
"""

from __future__ import annotations

import math

import torch


def _r(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype) if on else x


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def layer_norm(y: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mean = y.mean(-1, keepdim=True)
    var = (y - mean).pow(2).mean(-1, keepdim=True)
    return (y - mean) / torch.sqrt(var + eps) * w + b


def embed(tokens, weights, dtype) -> torch.Tensor:
    ids = torch.as_tensor(tokens, dtype=torch.long)
    return weights["embed"].to(dtype)[ids] + weights["pos"].to(dtype)[torch.arange(len(ids))]


def query_temperature(n: int, coef: float, every: int, dtype) -> torch.Tensor:
    p = torch.arange(n)
    return (1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype)))


def distance_slopes(heads: int, dtype) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def attend(q, k, v, scale, window=None, softcap=None, slopes=None, first_position=0) -> torch.Tensor:
    """Softmax attention of queries q [m, H, D] at positions first_position .. over keys k [n, G, D]
    and values v [n, G, Dv] at positions 0 .. n - 1 (n = first_position + m): head h uses key/value
    head h // (H / G); score = scale q.k, soft-capped, less slope_h * distance; query i sees key j
    with 0 <= i - j (< window)."""
    m, H, _ = q.shape
    n, G = k.shape[0], k.shape[1]
    i = torch.arange(first_position, first_position + m)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    out = torch.empty(m, H, v.shape[-1], dtype=q.dtype)
    for head in range(H):
        s = (q[:, head] @ k[:, head // (H // G)].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[head] * (i - j).to(q.dtype)
        s = s.masked_fill(~seen, float("-inf"))
        out[:, head] = s.softmax(-1) @ v[:, head // (H // G)]
    return out


def normed_queries_keys(q, k, q_weight, k_weight, eps, temperature, positions):
    """q and k [n, all heads * D], each divided by its root mean square over the whole row and scaled;
    the query then times its temperature at its position."""
    q = rms_unit(q, eps) * q_weight
    k = rms_unit(k, eps) * k_weight
    if temperature is not None:
        coef, every = temperature
        steps = torch.div(positions + 1, every, rounding_mode="floor") + 1
        q = q * (1.0 + coef * torch.log(steps.to(q.dtype)))[:, None]
    return q, k


def windowed_attention(h, weights, prefix, mixer, eps, rounding) -> torch.Tensor:
    """The `attention` mixer on a whole sequence h [n, W] -> [n, W]."""
    n, dtype = h.shape[0], h.dtype
    H, G, D = mixer["heads"], mixer["kv_heads"], mixer["dim"]
    q = _r(h @ weights[prefix + "q"].to(dtype).T, rounding)
    k = _r(h @ weights[prefix + "k"].to(dtype).T, rounding)
    v = k.view(n, G, D)                                    # the values are the keys as projected
    temp = mixer.get("q_temp")
    q, k = normed_queries_keys(q, k, weights[prefix + "q.norm"].to(dtype), weights[prefix + "k.norm"].to(dtype), eps,
                               None if temp is None else (temp["coef"], temp["every"]), torch.arange(n))
    q, k = _r(q, rounding).view(n, H, D), _r(k, rounding).view(n, G, D)
    mask = mixer.get("mask")
    out = attend(q, k, v, mixer["scale"], None if mask is None else mask["size"], mixer.get("softcap"),
                 distance_slopes(H, dtype))
    out = _r(out.reshape(n, H * D), rounding)
    return out @ weights[prefix + "o"].to(dtype).T


def latent_of(h, weights, prefix, eps, rounding) -> torch.Tensor:
    """The cached latent of a latent-attention layer: c = RMS(Wdkv h) * weight, [n, rank]."""
    dtype = h.dtype
    c = _r(h @ weights[prefix + "dkv"].to(dtype).T, rounding)
    return _r(rms_unit(c, eps) * weights[prefix + "dkv.norm"].to(dtype), rounding)


def latent_attention(h, c, weights, prefix, mixer, rounding) -> torch.Tensor:
    """The `latent_attention` mixer on a whole sequence, given the latent c it attends over."""
    n, dtype = h.shape[0], h.dtype
    H, D, V = mixer["heads"], mixer["dim"], mixer["vdim"]
    q = _r(h @ weights[prefix + "q"].to(dtype).T, rounding).view(n, H, D)
    k = _r(c @ weights[prefix + "uk"].to(dtype).T, rounding).view(n, H, D)
    v = _r(c @ weights[prefix + "uv"].to(dtype).T, rounding).view(n, H, V)
    gate = torch.sigmoid(h @ weights[prefix + "g"].to(dtype).T)          # [n, H]
    out = attend(q, k, v, mixer["scale"]) * gate[:, :, None]
    out = _r(out.reshape(n, H * V), rounding)
    return out @ weights[prefix + "o"].to(dtype).T


def feed_forward(h, weights, prefix, rounding) -> torch.Tensor:
    dtype = h.dtype
    gate = _r(h @ weights[prefix + "gate"].to(dtype).T, rounding)
    up = _r(h @ weights[prefix + "up"].to(dtype).T, rounding)
    act = _r(gelu_tanh(gate) * up, rounding)
    return act @ weights[prefix + "down"].to(dtype).T


def forward(raw: dict, weights: dict, tokens, dtype=torch.float64, rounding: bool = False, return_layers: bool = False):
    """Logits [n, vocab] of a whole sequence (and the residual after every layer, if asked)."""
    eps = raw["norm"]["eps"]
    x = embed(tokens, weights, dtype)
    latents: dict[int, torch.Tensor] = {}
    after = []
    for index, layer in enumerate(raw["layers"]):
        name = f"l{index}."
        mixer = layer["mixer"]
        h = _r(x, rounding)
        if layer["type"] == "attention":
            y = windowed_attention(h, weights, name + "mix.", mixer, eps, rounding)
        elif layer["type"] == "latent_attention":
            source = mixer.get("kv_from")
            if source is None:
                latents[index] = latent_of(h, weights, name + "mix.", eps, rounding)
                source = index
            y = latent_attention(h, latents[source], weights, name + "mix.", mixer, rounding)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + layer_norm(y, weights[name + "norm1"].to(dtype), weights[name + "norm1.b"].to(dtype), eps)
        if layer.get("mlp") is not None:
            y = feed_forward(_r(x, rounding), weights, name + "mlp.", rounding)
            x = x + layer_norm(y, weights[name + "norm2"].to(dtype), weights[name + "norm2.b"].to(dtype), eps)
        after.append(x)
    x = _r(layer_norm(x, weights["final.norm"].to(dtype), weights["final.norm.b"].to(dtype), eps), rounding)
    logits = x @ weights["head"].to(dtype).T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy_continue(raw: dict, weights: dict, prompt, count: int, dtype=torch.float64):
    """`count` greedy tokens after `prompt`, each from a whole-sequence pass, and the gap between
    the two largest logits at each step."""
    tokens, margins = list(prompt), []
    for _ in range(count):
        logits = forward(raw, weights, tokens, dtype=dtype)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(torch.argmax(logits)))
    return tokens[len(prompt):], margins
