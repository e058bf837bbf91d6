"""Plain, slow, whole-sequence implementation of the Vupitar decoder.

One function per mechanism, written from the design's equations; no cache, no batching, no
code shared with the `shrike_b200` package.  It reads the raw `config.json` dictionary and a
name -> tensor dictionary itself.

The design in this file's notation (x: residual stream [n, W], p: position from 0):

  e           = embed[token] * embedding.scale
  passes      : layers start .. stop - 1 run `times` times (same weights, fresh memory each pass),
                then the rest once.  Entering pass t: x <- x + e (t > 0 only), x <- x + step[t].
  layer       : x <- x + mixer(N1(x)) + ff(N2(x))                  (both branches read the same x)
  N(x)        = tanh(alpha x) * w + b                               (no statistics at all)
  mixer       = left_scale * attention(h) + right_scale * memory(h)
  attention   : q, k, v = W h + b; q, k <- per-head RMS * weight (one weight of size D for all heads);
                the first R dimensions of each head rotate by p * base^(-2i/R), i paired with i + R/2;
                s_ij = scale q_i.k_j; i sees j <= i with floor(i / C) = floor(j / C); softmax;
                head h's output times sigmoid(Wg h)_h; Wo (.) + bo
  memory      : q = Wq h / sqrt(D), k = Wk h, v = Wv h, per head
                a = cap tanh((Wi h + bi) / cap), f = logsigmoid(cap tanh((Wf h + bf) / cap))
                m_t = max(f + m_(t-1), a), m_0 = 0, S_0 = 0, z_0 = 0
                S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(a - m_t) k v^T,  z_t likewise with k
                o_t = S_t^T q / (max(|z_t.q|, exp(-m_t)) + 1e-6)
                each head's o over its root mean square; all heads * weight * sigmoid(Wg h); Wo
  ff dense    : g = min(Wg h, L), u = clamp(Wu h, -L, L); Wd (g sigmoid(1.702 g) (u + 1))
  ff experts  : p = softmax(Wr h) over all experts (32-bit); the `top` largest, their p over the sum of
                those (+ 1e-20); sum of weight * Wd_e (silu(Wg_e h) * (Wu_e h)); plus the shared expert
                (same form) times sigmoid(Wsg h)
  logits      = head N_final(x)

`rounding=True` rounds to bfloat16 where a bfloat16 engine may (products' outputs and
activations); norms, scores, softmax, gates of the memory, its state, routers, the residual sum
and positions stay in the working precision.
"""

from __future__ import annotations

import math

import torch


def _r(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype) if on else x


def tanh_norm(x, weights, name):
    """tanh(alpha x) * w + b with the scalar alpha stored beside the weight."""
    dtype = x.dtype
    return torch.tanh(weights[name + ".alpha"].to(dtype) * x) * weights[name].to(dtype) + weights[name + ".b"].to(dtype)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rotate_partial(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, H, D]: the first `dims` dimensions of every head rotate, dimension i with i + dims/2."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def chunk_mask(n: int, size: int) -> torch.Tensor:
    """[n, n] True where query i sees key j: j <= i and both in the same run of `size` positions."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def attend(q, k, v, scale, chunk=None, first_position=0) -> torch.Tensor:
    """Softmax attention of queries q [m, H, D] at positions first_position .. over keys k [n, G, D] and
    values v [n, G, Dv] at positions 0 .. n - 1 (n = first_position + m): head h uses key/value head
    h // (H / G); query i sees key j <= i, and with `chunk` only if floor(i / chunk) = floor(j / chunk)."""
    m, H, _ = q.shape
    n, G = k.shape[0], k.shape[1]
    seen = chunk_mask(n, chunk) if chunk else (torch.arange(n)[None, :] <= torch.arange(n)[:, None])
    seen = seen[first_position:]
    out = torch.empty(m, H, v.shape[-1], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        out[:, head] = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1) @ v[:, g]
    return out


def chunked_attention(h, weights, prefix, spec, eps, rounding) -> torch.Tensor:
    n, dtype = h.shape[0], h.dtype
    H, G, D, Dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)
    q = _r(h @ w("q").T + w("q.b"), rounding).view(n, H, D)
    k = _r(h @ w("k").T + w("k.b"), rounding).view(n, G, D)
    v = _r(h @ w("v").T + w("v.b"), rounding).view(n, G, Dv)
    q = rms_unit(q, eps) * w("q.norm")
    k = rms_unit(k, eps) * w("k.norm")
    positions = torch.arange(n)
    rot = spec.get("rot")
    if rot is not None:
        q = rotate_partial(q, positions, rot["dims"], rot["base"])
        k = rotate_partial(k, positions, rot["dims"], rot["base"])
    q, k = _r(q, rounding), _r(k, rounding)
    out = attend(q, k, v, spec["scale"], spec["mask"]["size"] if spec.get("mask") else None)
    gate = torch.sigmoid(h @ w("g").T)                          # [n, H]
    out = _r(out * gate[:, :, None], rounding).reshape(n, H * Dv)
    return out @ w("o").T + w("o.b")


def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def matrix_memory(h, weights, prefix, spec, eps, rounding, trace=None) -> torch.Tensor:
    """The recurrence, token by token.  `trace`, a list, receives (m, S, z) after the last token."""
    n, dtype = h.shape[0], h.dtype
    H, D, Dv, cap = spec["heads"], spec["dim"], spec["vdim"], spec["gate_cap"]
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)
    q = _r(h @ w("q").T, rounding).view(n, H, D) * D ** -0.5
    k = _r(h @ w("k").T, rounding).view(n, H, D)
    v = _r(h @ w("v").T, rounding).view(n, H, Dv)
    a = capped(h @ w("i").T + w("i.b"), cap)                                     # [n, H] log input gate
    f = torch.nn.functional.logsigmoid(capped(h @ w("f").T + w("f.b"), cap))     # [n, H] log forget gate
    S = torch.zeros(H, D, Dv, dtype=dtype)
    z = torch.zeros(H, D, dtype=dtype)
    m = torch.zeros(H, dtype=dtype)
    out = torch.empty(n, H, Dv, dtype=dtype)
    for t in range(n):
        m_new = torch.maximum(f[t] + m, a[t])
        keep = torch.exp(f[t] + m - m_new)
        take = torch.exp(a[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        z = keep[:, None] * z + take[:, None] * k[t]
        m = m_new
        top = torch.einsum("hdv,hd->hv", S, q[t])
        bottom = torch.maximum((z * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = top / bottom[:, None]
    if trace is not None:
        trace.append((m, S, z))
    out = rms_unit(out, eps).reshape(n, H * Dv) * w("norm") * torch.sigmoid(h @ w("g").T)
    return _r(out, rounding) @ w("o").T


def parallel_mixer(h, weights, prefix, spec, eps, rounding) -> torch.Tensor:
    left = chunked_attention(h, weights, prefix + ".left", spec["left"], eps, rounding)
    right = matrix_memory(h, weights, prefix + ".right", spec["right"], eps, rounding)
    return spec["left_scale"] * left + spec["right_scale"] * right


def dense_ff(h, weights, prefix, spec, rounding) -> torch.Tensor:
    dtype, limit = h.dtype, spec["limit"]
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)
    g = torch.clamp(_r(h @ w("gate").T, rounding), max=limit)
    u = torch.clamp(_r(h @ w("up").T, rounding), -limit, limit)
    return _r(g * torch.sigmoid(1.702 * g) * (u + 1.0), rounding) @ w("down").T


def expert(h, weights, prefix, rounding) -> torch.Tensor:
    dtype = h.dtype
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)
    g = _r(h @ w("gate").T, rounding)
    u = _r(h @ w("up").T, rounding)
    return _r(g * torch.sigmoid(g) * u, rounding) @ w("down").T


def route(h, weights, prefix, experts: int, top: int, gaps=None):
    """(chosen [n, top], weights [n, top]): softmax over all experts, the largest `top`, renormalised.
    `gaps`, a list, receives per token the gap of the logarithms of the scores (that is, of the router's logits)
    between the last expert chosen and the first one left out."""
    scores = torch.softmax(h @ weights[f"{prefix}.router"].to(h.dtype).T, dim=-1)
    best, chosen = torch.topk(scores, top, dim=-1)
    if gaps is not None and top < experts:
        ranked = torch.sort(scores, dim=-1, descending=True).values
        gaps.append(torch.log(ranked[:, top - 1]) - torch.log(ranked[:, top]))
    return chosen, best / (best.sum(-1, keepdim=True) + 1e-20)


def expert_ff(h, weights, prefix, spec, rounding, gaps=None) -> torch.Tensor:
    n = h.shape[0]
    chosen, share = route(h, weights, prefix, spec["router"]["experts"], spec["router"]["top"], gaps)
    out = torch.zeros(n, weights[f"{prefix}.e0.down"].shape[0], dtype=h.dtype)
    for e in range(spec["router"]["experts"]):
        rows, place = (chosen == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += share[rows, place][:, None] * expert(h[rows], weights, f"{prefix}.e{e}", rounding)
    if spec.get("shared") is not None:
        gate = torch.sigmoid(h @ weights[f"{prefix}.shared.sg"].to(h.dtype).T)        # [n, 1]
        out = out + gate * expert(h, weights, f"{prefix}.shared", rounding)
    return out


def feed_forward(h, weights, prefix, spec, rounding, gaps=None) -> torch.Tensor:
    if spec["kind"] == "dense":
        return dense_ff(h, weights, prefix, spec, rounding)
    if spec["kind"] == "moe":
        return expert_ff(h, weights, prefix, spec, rounding, gaps)
    raise ValueError(spec["kind"])


def layer(x, weights, index: int, spec, eps, rounding, gaps=None) -> torch.Tensor:
    name = f"l{index}"
    if spec["type"] != "parallel":
        raise ValueError(spec["type"])
    branch = parallel_mixer(_r(tanh_norm(x, weights, name + ".norm1"), rounding), weights, name + ".mix", spec["mixer"], eps, rounding)
    if spec.get("mlp") is not None:
        branch = branch + feed_forward(_r(tanh_norm(x, weights, name + ".norm2"), rounding), weights, name + ".mlp", spec["mlp"], rounding, gaps)
    return x + branch


def run_order(raw: dict):
    """(layer, pass number or None when the layer's run does not open a pass)."""
    count = len(raw["layers"])
    loop = raw.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t if i == loop["start"] else None))
    return order + [(i, None) for i in range(loop["stop"], count)]


def forward(raw: dict, weights: dict, tokens, dtype=torch.float64, rounding: bool = False, layers_out=None, gaps=None) -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence.  `layers_out`, a list, receives the residual after every run;
    `gaps`, a list, per routed layer run the router's margin at every token (see `route`)."""
    eps = raw["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    e = weights["embed"].to(dtype)[ids] * raw["embedding"]["scale"]
    x = e.clone()
    for index, opens in run_order(raw):
        if opens is not None:
            if opens > 0:
                x = x + e
            x = x + weights["loop.step"].to(dtype)[opens]
        x = layer(x, weights, index, raw["layers"][index], eps, rounding, gaps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return _r(tanh_norm(x, weights, "final.norm"), rounding) @ weights["head"].to(dtype).T


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
