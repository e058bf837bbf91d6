"""Each mechanism of the Sadodra parts alone on the GPU, against the plain functions of
`tests/plain/plain_sadodra.py` in float64: the norm on a branch's output, the position embedding,
the GELU gate (alone and in the tensor-core product's epilogue), queries and keys normed over the
whole projection with the query temperature, the latent with its gate, and
paged attention with soft cap, distance bias and window, with inputs crafted so that one key just
inside or just outside a window, at a page's border or far back decides the result."""

import math

import pytest
import torch

from tests.gpu_common import cuda_ops
from tests.plain import plain_sadodra as ps

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def close(got, want, atol, what=""):
    """|got - want| <= atol, plus 2^-7 of |want| where the tolerance is a bfloat16 one (a bfloat16
    result is rounded to 8 bits of mantissa whatever its size)."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    bound = atol + (2.0 ** -7 if atol >= 1e-2 else 0.0) * want.abs()
    worst = ((got - want).abs() - bound).max().item()
    assert worst <= 0, f"{what}: exceeds the tolerance {atol:.1e} by {worst:.3e}"


# ------------------------------------------------------------------ norm on a branch's output
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,partials", [(3, 96, 1), (5, 70, 3), (300, 320, 1), (2, 4096, 8), (260, 1030, 2), (1, 8192, 1)])
def test_norm_add_sums_normed_branch_into_residual(dtype, n, width, partials):
    ops = cuda_ops(dtype)
    resid = rnd(n, width, seed=1, scale=3.0)
    branch = rnd(partials, n, width, seed=2) + 0.7          # a mean far from zero: the norm must take it off
    w, b = 1.0 + 0.1 * rnd(width, seed=3), 0.2 * rnd(width, seed=4)
    want = resid.double() + ps.layer_norm(branch.double().sum(0), w.double(), b.double(), 1e-5)
    x = resid.to(DEV)
    out = torch.empty(n, width, dtype=dtype, device=DEV)
    stack = branch.to(DEV) if partials > 1 else branch[0].contiguous().to(DEV)
    ops.norm_add(x, stack, w.to(DEV), b.to(DEV), 1e-5, out)
    close(x, want, 2e-5, "residual")
    close(out, want, 2e-5 if dtype == torch.float32 else 4e-2, "residual in the activation type")
    # the RMS form without a bias, and the plain cast
    x2 = resid.to(DEV)
    ops.norm_add(x2, branch[0].contiguous().to(DEV), w.to(DEV), None, 1e-5, None, layer_norm=False)
    close(x2, resid.double() + ps.rms_unit(branch[0].double(), 1e-5) * w.double(), 2e-5, "rms form")
    ops.norm_add(x2, None, None, None, 0.0, out)
    close(out, x2, 0 if dtype == torch.float32 else 4e-2, "cast only")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_norm_norms_only_the_wanted_rows(dtype):
    ops = cuda_ops(dtype)
    resid = rnd(40, 150, seed=5, scale=2.0) - 0.4
    w, b = 1.0 + 0.1 * rnd(150, seed=6), 0.3 * rnd(150, seed=7)
    rows = torch.tensor([39, 0, 7, 7, 20], dtype=torch.int32)
    x = resid.to(DEV)
    out = torch.empty(5, 150, dtype=dtype, device=DEV)
    ops.gather_norm(x, rows.to(DEV), w.to(DEV), b.to(DEV), 1e-6, out)
    close(out, ps.layer_norm(resid.double()[rows.long()], w.double(), b.double(), 1e-6), TOL[dtype], "gathered rows")
    assert torch.equal(x.cpu(), resid), "the residual was written"


# ------------------------------------------------------------------ embedding with positions
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_adds_the_position_vector(dtype):
    ops = cuda_ops(dtype)
    table, pos = rnd(50, 72, seed=1).to(dtype), rnd(30, 72, seed=2).to(dtype)
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32)
    positions = torch.tensor([0, 29, 5, 6, 1], dtype=torch.int32)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    ops.embed(ids.to(DEV), table.to(DEV), out, None, position_table=pos.to(DEV), positions=positions.to(DEV))
    want = table.double()[ids.long()] + pos.double()[positions.long()]
    close(out, want, 1e-6, "token + position")


# ------------------------------------------------------------------ GELU gate
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,inter", [(5, 179), (3, 176), (300, 320)])
def test_gelu_gate(dtype, n, inter):
    ops = cuda_ops(dtype)
    gate_up = (rnd(n, 2 * inter, seed=8, scale=2.5)).to(dtype)
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops.act_mul(gate_up.to(DEV), out, 0, "gelu_tanh")
    g, u = gate_up.double()[:, :inter], gate_up.double()[:, inter:]
    close(out, ps.gelu_tanh(g) * u, 1e-5 if dtype == torch.float32 else 6e-2, "gelu_tanh(gate) * up")


@pytest.mark.parametrize("tokens,inter,k", [(1, 64, 64), (8, 176, 192), (33, 320, 240)])
def test_gelu_gate_in_the_product_epilogue_equals_the_separate_kernel(tokens, inter, k):
    ops = cuda_ops(torch.bfloat16)
    run = ops.gated_rows
    gate, up = rnd(inter, k, seed=1, scale=0.2).bfloat16(), rnd(inter, k, seed=2, scale=0.2).bfloat16()
    x = rnd(tokens, k, seed=3).bfloat16().to(DEV)
    mixed = torch.stack([gate.view(inter // run, run, k), up.view(inter // run, run, k)], dim=1).reshape(2 * inter, k).contiguous().to(DEV)
    fused = torch.empty(tokens, inter, dtype=torch.bfloat16, device=DEV)
    assert ops.linear_gated(x, mixed, fused, "gelu_tanh")
    both = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops.linear(x, mixed, both)
    stepwise = torch.empty_like(fused)
    ops.act_mul(both, stepwise, run, "gelu_tanh")
    ops.check_status()
    assert torch.equal(fused, stepwise)
    want = ps.gelu_tanh(x.double().cpu() @ gate.double().T) * (x.double().cpu() @ up.double().T)
    close(fused, want, 5e-2, "against float64")


# ------------------------------------------------------------------ queries and keys
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,temperature,partials", [(4, 2, 32, (0.3, 16), 1), (3, 3, 24, (0.7, 5), 3),
                                                                     (5, 1, 64, None, 2), (2, 2, 16, (0.25, 1), 1), (3, 1, 10, (0.5, 3), 2)])
def test_queries_and_keys_are_normed_over_the_whole_projection(dtype, heads, kv_heads, dim, temperature, partials):
    ops = cuda_ops(dtype)
    padded = -(-dim // 16) * 16
    every = temperature[1] if temperature else 4
    positions = [0, 1, every - 2, every - 1, every, 2 * every - 1, 2 * every, 300, 7 * every - 1]
    positions = [p for p in positions if p >= 0]
    n = len(positions)
    qw, kw = heads * dim, kv_heads * dim
    qk = rnd(partials, n, qw + kw, seed=3, scale=0.5)
    q_weight, k_weight = 1.0 + 0.2 * rnd(qw, seed=4), 1.0 + 0.2 * rnd(kw, seed=5)
    page, pages = 4, 6
    keys = torch.full((pages, page, kv_heads, padded), float("nan"), dtype=dtype, device=DEV)
    values = torch.full_like(keys, float("nan"))
    slots = torch.tensor([5, 0, 9, 23, 11, 2, 7, 8, -1][:n], dtype=torch.int32)
    q_out = torch.full((n, heads * padded), float("nan"), dtype=dtype, device=DEV)
    stack = qk.to(DEV) if partials > 1 else qk[0].contiguous().to(DEV)
    ops.qk_norm_store(stack, q_weight.to(DEV), k_weight.to(DEV), 1e-5, torch.tensor(positions, dtype=torch.int32, device=DEV),
                      temperature, q_out, keys, values, slots.to(DEV), heads, kv_heads, dim, padded)
    total = qk.double().sum(0)
    q, k = ps.normed_queries_keys(total[:, :qw], total[:, qw:], q_weight.double(), k_weight.double(), 1e-5, temperature,
                                  torch.tensor(positions))
    tol = 2e-5 if dtype == torch.float32 else 5e-2
    got_q = q_out.view(n, heads, padded)
    close(got_q[:, :, :dim], q.view(n, heads, dim), tol, "queries")
    assert (got_q[:, :, dim:] == 0).all(), "query padding is not zero"
    flat_k, flat_v = keys.view(-1, kv_heads, padded), values.view(-1, kv_heads, padded)
    for row, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        close(flat_k[slot, :, :dim], k.view(n, kv_heads, dim)[row], tol, f"key of token {row}")
        close(flat_v[slot, :, :dim], total[row, qw:].view(kv_heads, dim), tol, f"value of token {row}: the key as projected")
        assert (flat_k[slot, :, dim:] == 0).all() and (flat_v[slot, :, dim:] == 0).all()
    untouched = sorted(set(range(pages * page)) - set(s for s in slots.tolist() if s >= 0))
    assert torch.isnan(flat_k[untouched].float()).all(), "a slot that no token names was written"


# ------------------------------------------------------------------ latent, gate, per-head products
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_width,rank,gates,partials", [(64, 40, 4, 1), (96, 24, 6, 3), (48, 0, 3, 1), (32, 64, 0, 2)])
def test_latent_is_normed_into_its_pages_and_the_gate_is_a_sigmoid(dtype, q_width, rank, gates, partials):
    ops = cuda_ops(dtype)
    padded = -(-max(rank, 1) // 16) * 16
    n = 7
    fused = rnd(partials, n, q_width + rank + gates, seed=6, scale=1.5)
    weight = 1.0 + 0.2 * rnd(max(rank, 1), seed=7)
    pages = torch.full((5, 4, 1, padded), float("nan"), dtype=dtype, device=DEV)
    slots = torch.tensor([3, 19, 0, -1, 8, 9, 10], dtype=torch.int32)
    q_out = torch.empty(n, q_width, dtype=dtype, device=DEV)
    gate_out = torch.full((n, max(gates, 1)), float("nan"), dtype=torch.float32, device=DEV)
    stack = fused.to(DEV) if partials > 1 else fused[0].contiguous().to(DEV)
    ops.latent_store(stack, weight.to(DEV) if rank else None, 1e-5, q_out, pages if rank else None, slots.to(DEV),
                     gate_out if gates else None, q_width, rank, padded, gates)
    total = fused.double().sum(0)
    tol = 2e-5 if dtype == torch.float32 else 5e-2
    close(q_out, total[:, :q_width], tol, "queries")
    if gates:
        close(gate_out, torch.sigmoid(total[:, q_width + rank:]), 2e-6, "gate")
    if rank:
        want = ps.rms_unit(total[:, q_width: q_width + rank], 1e-5) * weight.double()
        flat = pages.view(-1, padded)
        for row, slot in enumerate(slots.tolist()):
            if slot >= 0:
                close(flat[slot, :rank], want[row], tol, f"latent of token {row}")
                assert (flat[slot, rank:] == 0).all()
        assert torch.isnan(flat[1].float()).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,heads,dim", [(1, 4, 48), (70, 3, 16), (2100, 12, 256)])
def test_head_scale(dtype, n, heads, dim):
    ops = cuda_ops(dtype)
    x = rnd(n, heads * dim, seed=1).to(dtype)
    gate = torch.rand(n, heads, generator=torch.Generator().manual_seed(3))
    scaled = x.clone().to(DEV)
    ops.head_scale(scaled, gate.to(DEV), heads, dim)
    close(scaled.view(n, heads, dim), x.double().view(n, heads, dim) * gate.double()[:, :, None],
          1e-6 if dtype == torch.float32 else 3e-2, "head scale")


# ------------------------------------------------------------------ paged attention with changed scores
def paged(dtype, sequences, page, kv_heads, dim, shared_plane=False, seed=0):
    """Puts sequences (q [ctx, H, D], k [ctx, G, D], v [ctx, G, D], q_len) on shuffled pages; the rest of
    the pool is NaN.  `shared_plane`: keys and values are one tensor (v must be k)."""
    g = torch.Generator().manual_seed(seed)
    total = sum(-(-len(k) // page) for _, k, _, _ in sequences) + 2
    order = torch.randperm(total, generator=g).tolist()
    keys = torch.full((total, page, kv_heads, dim), float("nan"), dtype=dtype)
    values = keys if shared_plane else torch.full_like(keys, float("nan"))
    width = max(-(-len(k) // page) for _, k, _, _ in sequences)
    table = torch.full((len(sequences), width), -1, dtype=torch.int32)
    q_rows, seq_of, q_start, ctx_lens, q_lens = [], [], [0], [], []
    for s, (q, k, v, q_len) in enumerate(sequences):
        ctx = len(k)
        for b in range(-(-ctx // page)):
            pid = order.pop()
            table[s, b] = pid
            rows = slice(b * page, min(ctx, (b + 1) * page))
            keys[pid, : rows.stop - rows.start] = k[rows].to(dtype)
            values[pid, : rows.stop - rows.start] = v[rows].to(dtype)
        q_rows.append(q[ctx - q_len:].to(dtype))
        seq_of += [s] * q_len
        q_start.append(q_start[-1] + q_len)
        ctx_lens.append(ctx)
        q_lens.append(q_len)
    keys_dev = keys.to(DEV)
    return dict(keys=keys_dev, values=keys_dev if shared_plane else values.to(DEV), table=table.to(DEV),
                q=torch.cat(q_rows).reshape(sum(q_lens), -1).contiguous().to(DEV),
                q_start=torch.tensor(q_start, dtype=torch.int32, device=DEV),
                ctx_len=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
                seq_of=torch.tensor(seq_of, dtype=torch.int32, device=DEV), q_lens=q_lens, ctx_lens=ctx_lens)


def attend_both(ops, dtype, sequences, page, heads, kv_heads, dim, scale, window, softcap, slopes, shared_plane=False):
    case = paged(dtype, sequences, page, kv_heads, dim, shared_plane)
    out = torch.empty_like(case["q"])
    ops.paged_attention(case["q"], case["keys"], case["values"], case["table"], case["q_start"], case["ctx_len"], case["seq_of"],
                        heads, kv_heads, dim, scale, window, out, max_q_len=max(case["q_lens"]), max_ctx_len=max(case["ctx_lens"]),
                        min_q_len=min(case["q_lens"]), q_lens=case["q_lens"], softcap=softcap,
                        slopes=None if slopes is None else slopes.float().to(DEV))
    want = []
    for q, k, v, q_len in sequences:
        ctx = len(k)
        r = lambda t: t.to(dtype).double()   # noqa: E731  the oracle sees the stored values
        want.append(ps.attend(r(q[ctx - q_len:]), r(k), r(v), scale, window, softcap,
                              None if slopes is None else slopes.float().double(), first_position=ctx - q_len))
    return out, torch.cat(want).reshape(out.shape)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,page,window,softcap", [(4, 2, 32, 8, 20, 12.0), (3, 3, 32, 5, 37, 50.0), (8, 1, 64, 16, 70, None),
                                                                    (6, 2, 48, 16, None, 5.0), (20, 1, 16, 4, 9, 8.0)])
def test_capped_and_biased_scores_in_single_tokens_and_portions(dtype, heads, kv_heads, dim, page, window, softcap):
    ops = cuda_ops(dtype)
    slopes = ps.distance_slopes(heads, torch.float64)
    sequences = []
    for s, (ctx, q_len) in enumerate([(1, 1), (40, 1), (130, 1), (21, 2), (100, 37), (300, 129), (64, 64), (33, 1), (200, 3)]):
        g = torch.Generator().manual_seed(50 + s)
        sequences.append((torch.randn(ctx, heads, dim, generator=g) * 1.5, torch.randn(ctx, kv_heads, dim, generator=g),
                          torch.randn(ctx, kv_heads, dim, generator=g), q_len))
    got, want = attend_both(ops, dtype, sequences, page, heads, kv_heads, dim, dim ** -0.5 * 2, window, softcap, slopes)
    close(got, want, TOL[dtype], "attention with cap, bias and window")
    singles = [(q, k, v, 1) for q, k, v, _ in sequences]     # the single-token kernel alone (other split and cluster shapes)
    got, want = attend_both(ops, dtype, singles, page, heads, kv_heads, dim, dim ** -0.5 * 2, window, softcap, slopes)
    close(got, want, TOL[dtype], "single tokens only")


@pytest.mark.parametrize("tensor_core,splits", [(True, 0), (True, 3), (False, 0)])
@pytest.mark.parametrize("heads,kv_heads,dim,page,window,softcap", [(6, 2, 64, 16, 150, 20.0), (4, 1, 128, 16, None, 9.0), (2, 2, 128, 8, 300, None),
                                                                    (3, 3, 64, 32, 64, 4.0)])
def test_capped_and_biased_scores_on_the_tensor_core_portions_kernel(heads, kv_heads, dim, page, window, softcap, tensor_core, splits):
    """Head sizes 64 and 128 take the tcgen05 kernel for portions: with and without it, and with a
    query tile's keys shared by several CTAs, the same scores."""
    ops = cuda_ops(torch.bfloat16)
    ops.tensor_core_attention, ops.portion_splits = tensor_core, splits
    slopes = ps.distance_slopes(heads, torch.float64)
    sequences = []
    for s, (ctx, q_len) in enumerate([(700, 700), (130, 1), (500, 129), (300, 300), (64, 2), (1000, 37)]):
        g = torch.Generator().manual_seed(70 + s)
        sequences.append((torch.randn(ctx, heads, dim, generator=g), torch.randn(ctx, kv_heads, dim, generator=g),
                          torch.randn(ctx, kv_heads, dim, generator=g), q_len))
    got, want = attend_both(ops, torch.bfloat16, sequences, page, heads, kv_heads, dim, dim ** -0.5 * 3, window, softcap, slopes)
    ops.check_status()
    close(got, want, TOL[torch.bfloat16], "portions on the tensor cores")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_len", [1, 2, 50])
@pytest.mark.parametrize("page,window", [(16, 48), (8, 20), (5, 37), (16, 16)])
def test_a_key_at_the_windows_edge_decides(dtype, q_len, page, window):
    """The last query's direction is planted in one key: at distance window - 1 (seen, and the output
    is that key's value) or at distance window (not seen: the output must not hold a trace of it)."""
    ops = cuda_ops(dtype)
    heads = kv_heads = 2
    dim, ctx = 32, 3 * window + 11
    for distance, seen in ((window - 1, True), (window, False), (0, True)):
        g = torch.Generator().manual_seed(distance)
        q, k, v = (torch.randn(ctx, heads, dim, generator=g) * 0.3 for _ in range(3))
        direction = torch.nn.functional.normalize(torch.randn(dim, generator=g), dim=0)
        q[ctx - 1] = direction * 12.0
        k[ctx - 1 - distance] = direction * 12.0
        v[ctx - 1 - distance] = 100.0
        slopes = torch.tensor([0.01, 0.002], dtype=torch.float64)
        got, want = attend_both(ops, dtype, [(q, k, v, q_len)], page, heads, kv_heads, dim, 1.0, window, None, slopes)
        close(got, want, TOL[dtype] * 100, f"distance {distance}")
        last = got[-1].float().view(heads, dim)
        assert (last.mean() > 90) == seen, f"key at distance {distance} of window {window}: seen={seen}, output {last.mean():.2f}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_len", [1, 40])
def test_latent_form_finds_a_far_key_among_hundreds(dtype, q_len):
    """One key/value head of the latent's size whose keys are its values (one plane), many query heads:
    a key 700 positions back whose score stands out is what the output must be."""
    ops = cuda_ops(dtype)
    heads, rank, page, ctx = 6, 48, 16, 800
    g = torch.Generator().manual_seed(9)
    c = torch.randn(ctx, 1, rank, generator=g) * 0.2
    q = torch.randn(ctx, heads, rank, generator=g) * 0.2
    far = ctx - 1 - 700
    c[far] = 0.0
    c[far, 0, 5] = 3.0
    q[ctx - 1] = 0.0
    q[ctx - 1, :, 5] = 8.0
    got, want = attend_both(ops, dtype, [(q, c, c, q_len)], page, heads, 1, rank, 1.0, None, None, None, shared_plane=True)
    close(got, want, TOL[dtype], "latent form")
    assert (got[-1].float().view(heads, rank)[:, 5] > 2.9).all()
