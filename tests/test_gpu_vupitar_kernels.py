"""Each mechanism of the Vupitar parts alone on the GPU, against the plain functions of
`tests/plain/plain_vupitar.py` in float64: the tanh norm that adds pending sums (one norm, two, gathered
rows), the scaled embedding with its second copy, the clamped gate (alone and in the tensor-core
product's epilogue), queries, keys and values with per-head norms and a partial rotation, paged
attention over chunks of positions with keys planted at a chunk's edges, at page borders and far back,
the matrix memory (whole, in portions, token by token, on slots that had other owners), the router and
the experts' weighted activation."""

import math

import pytest
import torch

from tests.gpu_common import cuda_ops
from tests.plain import plain_vupitar as pv
from tests.test_gpu_sadodra_kernels import close, paged, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


# ------------------------------------------------------------------ tanh norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,partials", [(3, 96, 1), (5, 70, 3), (300, 320, 1), (2, 4096, 8), (70, 1030, 2)])
def test_tanh_norm_adds_pending_sums_and_norms_twice(dtype, n, width, partials):
    ops = cuda_ops(dtype)
    resid = rnd(n, width, seed=1, scale=2.0)
    first, second = rnd(partials, n, width, seed=2), rnd(n, width, seed=3)
    row = rnd(width, seed=4)
    weights = {"a": 1.0 + 0.1 * rnd(width, seed=5), "a.b": 0.2 * rnd(width, seed=6), "a.alpha": torch.tensor(0.7),
               "b": 1.0 + 0.1 * rnd(width, seed=7), "b.b": 0.2 * rnd(width, seed=8), "b.alpha": torch.tensor(1.9)}
    summed = resid.double() + 0.8 * first.double().sum(0) - 1.3 * second.double() + row.double()
    x = resid.to(DEV)
    outs = [torch.empty(n, width, dtype=dtype, device=DEV) for _ in range(2)]
    stack = first.to(DEV) if partials > 1 else first[0].contiguous().to(DEV)
    dev = {k: v.float().to(DEV) for k, v in weights.items()}
    ops.tanh_norm(x, [(stack, 0.8), (second.to(DEV), -1.3)], row_add=row.to(DEV),
                  norms=[(0.7, dev["a"], dev["a.b"], outs[0]), (1.9, dev["b"], dev["b.b"], outs[1])])
    close(x, summed, 2e-5, "residual")
    for name, out in zip("ab", outs):
        close(out, pv.tanh_norm(summed, weights, name), TOL[dtype], f"norm {name}")
    # gathered rows: the residual stays, the pending sum is still added for the rows that are normed
    rows = torch.tensor([n - 1, 0, n // 2, 0], dtype=torch.int32)
    before = x.clone()
    few = torch.empty(4, width, dtype=dtype, device=DEV)
    ops.tanh_norm(x, [(second.to(DEV), 2.0)], rows=rows.to(DEV), norms=[(0.7, dev["a"], dev["a.b"], few)])
    assert torch.equal(x, before), "the residual was written"
    close(few, pv.tanh_norm((summed + 2.0 * second.double())[rows.long()], weights, "a"), TOL[dtype], "gathered rows")
    ops.tanh_norm(x, [], row_add=row.to(DEV))       # no norm at all: a pass entry
    close(x, summed + row.double(), 3e-5, "row added")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_scales_its_rows_and_keeps_a_copy(dtype):
    ops = cuda_ops(dtype)
    table = rnd(50, 72, seed=1).to(dtype)
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    keep = torch.full((5, 72), float("nan"), dtype=torch.float32, device=DEV)
    ops.embed(ids.to(DEV), table.to(DEV), out, None, scale=1.7, keep=keep)
    close(out, table.double()[ids.long()] * 1.7, 1e-6, "scaled rows")
    assert torch.equal(out, keep)


# ------------------------------------------------------------------ clamped gate
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,inter,limit", [(5, 179, 0.8), (3, 176, 7.0), (300, 320, 1.0)])
def test_clamped_gate(dtype, n, inter, limit):
    ops = cuda_ops(dtype)
    gate_up = (rnd(n, 2 * inter, seed=8, scale=2.5)).to(dtype)
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops.act_mul(gate_up.to(DEV), out, 0, "clamped_swish", limit=limit)
    g, u = gate_up.double()[:, :inter].clamp(max=limit), gate_up.double()[:, inter:].clamp(-limit, limit)
    close(out, g * torch.sigmoid(1.702 * g) * (u + 1.0), 1e-5 if dtype == torch.float32 else 6e-2, "clamped gate")
    with pytest.raises(Exception):
        ops.act_mul(gate_up.to(DEV), out, 0, "clamped_swish")     # no limit


@pytest.mark.parametrize("tokens,inter,k", [(1, 64, 64), (8, 176, 192), (33, 320, 240)])
def test_clamped_gate_in_the_product_epilogue_equals_the_separate_kernel(tokens, inter, k):
    ops = cuda_ops(torch.bfloat16)
    run = ops.gated_rows
    weights = {"m.gate": rnd(inter, k, seed=1, scale=0.3).bfloat16(), "m.up": rnd(inter, k, seed=2, scale=0.3).bfloat16(),
               "m.down": torch.eye(inter)}
    x = rnd(tokens, k, seed=3).bfloat16()
    mixed = torch.stack([weights["m.gate"].view(inter // run, run, k), weights["m.up"].view(inter // run, run, k)], dim=1)
    mixed = mixed.reshape(2 * inter, k).contiguous().to(DEV)
    fused = torch.empty(tokens, inter, dtype=torch.bfloat16, device=DEV)
    assert ops.linear_gated(x.to(DEV), mixed, fused, "clamped_swish", limit=0.9)
    both = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device=DEV)
    ops.linear(x.to(DEV), mixed, both)
    stepwise = torch.empty_like(fused)
    ops.act_mul(both, stepwise, run, "clamped_swish", limit=0.9)
    ops.check_status()
    assert torch.equal(fused, stepwise)
    close(fused, pv.dense_ff(x.double(), weights, "m", {"limit": 0.9}, False), 5e-2, "against float64")


# ------------------------------------------------------------------ queries, keys, values
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,partials,normed", [(4, 2, 32, 16, 16, 1, True), (3, 3, 16, 48, 2, 3, True),
                                                                        (5, 1, 64, 64, 64, 2, True), (2, 2, 24, 8, 0, 1, False),
                                                                        (2, 1, 128, 128, 64, 1, True)])
def test_heads_are_normed_rotated_and_stored(dtype, heads, kv_heads, dim, vdim, rot, partials, normed):
    ops = cuda_ops(dtype)
    padded = -(-max(dim, vdim) // 16) * 16
    positions = torch.tensor([0, 1, 7, 300, 1113, 5, 64, 2, 9], dtype=torch.int32)
    n = len(positions)
    total = heads * dim + kv_heads * (dim + vdim) + heads
    fused = rnd(partials, n, total, seed=3, scale=0.7)
    bias = 0.3 * rnd(total, seed=9)
    bias[-heads:] = 0.0
    q_weight, k_weight = 1.0 + 0.2 * rnd(dim, seed=4), 1.0 + 0.2 * rnd(dim, seed=5)
    base = 10000.0
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64) if rot else None
    page, pages = 4, 6
    keys = torch.full((pages, page, kv_heads, padded), float("nan"), dtype=dtype, device=DEV)
    values = torch.full_like(keys, float("nan"))
    slots = torch.tensor([5, 0, 9, 23, 11, 2, 7, 8, -1], dtype=torch.int32)
    q_out = torch.full((n, heads * padded), float("nan"), dtype=dtype, device=DEV)
    gate = torch.full((n, heads), float("nan"), dtype=torch.float32, device=DEV)
    stack = fused.to(DEV) if partials > 1 else fused[0].contiguous().to(DEV)
    ops.head_prep(stack, bias.to(DEV), positions.to(DEV), None if inv_freq is None else inv_freq.float().to(DEV), rot,
                  q_weight.to(DEV) if normed else None, k_weight.to(DEV) if normed else None, 1e-5, q_out, keys, values,
                  slots.to(DEV), gate, heads, kv_heads, dim, vdim, padded)
    x = fused.double().sum(0) + bias.double()
    q = x[:, : heads * dim].view(n, heads, dim)
    k = x[:, heads * dim: (heads + kv_heads) * dim].view(n, kv_heads, dim)
    v = x[:, (heads + kv_heads) * dim: (heads + kv_heads) * dim + kv_heads * vdim].view(n, kv_heads, vdim)
    if normed:
        q, k = pv.rms_unit(q, 1e-5) * q_weight.double(), pv.rms_unit(k, 1e-5) * k_weight.double()
    if rot:
        q, k = pv.rotate_partial(q, positions, rot, base), pv.rotate_partial(k, positions, rot, base)
    # the angle is position * frequency in 32-bit: at position 1113 its rounding alone moves a component by about 1e-4
    tol = 4e-4 if dtype == torch.float32 else 4e-2
    got_q = q_out.view(n, heads, padded)
    close(got_q[:, :, :dim], q, tol, "queries")
    assert (got_q[:, :, dim:] == 0).all()
    close(gate, torch.sigmoid(x[:, -heads:]), 1e-6, "head gates")
    flat_k, flat_v = keys.view(-1, kv_heads, padded), values.view(-1, kv_heads, padded)
    for row, slot in enumerate(slots.tolist()):
        if slot >= 0:
            close(flat_k[slot, :, :dim], k[row], tol, f"keys of token {row}")
            close(flat_v[slot, :, :vdim], v[row], tol, f"values of token {row}")
            assert (flat_k[slot, :, dim:] == 0).all() and (flat_v[slot, :, vdim:] == 0).all()
    assert torch.isnan(flat_k[1].float()).all(), "a slot nobody named was written"


# ------------------------------------------------------------------ attention over chunks
def attend_both(ops, dtype, sequences, page, heads, kv_heads, dim, scale, chunk):
    case = paged(dtype, sequences, page, kv_heads, dim)
    out = torch.empty_like(case["q"])
    ops.paged_attention(case["q"], case["keys"], case["values"], case["table"], case["q_start"], case["ctx_len"], case["seq_of"],
                        heads, kv_heads, dim, scale, None, out, max_q_len=max(case["q_lens"]), max_ctx_len=max(case["ctx_lens"]),
                        min_q_len=min(case["q_lens"]), q_lens=case["q_lens"], chunk=chunk)
    want = []
    for q, k, v, q_len in sequences:
        ctx = len(k)
        r = lambda t: t.to(dtype).double()   # noqa: E731  the oracle sees the stored values
        want.append(pv.attend(r(q[ctx - q_len:]), r(k), r(v), scale, chunk, first_position=ctx - q_len))
    return out, torch.cat(want).reshape(out.shape)


def random_sequences(shapes, heads, kv_heads, dim, seed):
    sequences = []
    for s, (ctx, q_len) in enumerate(shapes):
        g = torch.Generator().manual_seed(seed + s)
        sequences.append((torch.randn(ctx, heads, dim, generator=g) * 1.5, torch.randn(ctx, kv_heads, dim, generator=g),
                          torch.randn(ctx, kv_heads, dim, generator=g), q_len))
    return sequences


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,page,chunk", [(4, 2, 32, 8, 20), (3, 3, 32, 5, 37), (8, 2, 64, 16, 70), (6, 2, 48, 16, 5),
                                                           (20, 1, 16, 4, 1), (2, 1, 128, 16, 130), (2, 2, 64, 32, 64), (4, 1, 96, 16, 1000)])
def test_chunked_keys_in_single_tokens_and_portions(dtype, heads, kv_heads, dim, page, chunk):
    ops = cuda_ops(dtype)
    shapes = [(1, 1), (40, 1), (130, 1), (21, 2), (100, 37), (300, 129), (64, 64), (33, 1), (200, 3), (chunk + 1, 1), (2 * chunk, 2)]
    sequences = random_sequences(shapes, heads, kv_heads, dim, 50)
    got, want = attend_both(ops, dtype, sequences, page, heads, kv_heads, dim, dim ** -0.5 * 2, chunk)
    ops.check_status()
    close(got, want, TOL[dtype], "attention over chunks")
    singles = [(q, k, v, 1) for q, k, v, _ in sequences]     # the single-token kernel alone (other split and cluster shapes)
    got, want = attend_both(ops, dtype, singles, page, heads, kv_heads, dim, dim ** -0.5 * 2, chunk)
    close(got, want, TOL[dtype], "single tokens only")


@pytest.mark.parametrize("tensor_core,splits", [(True, 0), (True, 3), (False, 0)])
@pytest.mark.parametrize("heads,kv_heads,dim,page,chunk", [(6, 2, 64, 16, 150), (4, 1, 128, 16, 136), (2, 2, 128, 8, 300), (3, 3, 64, 32, 64)])
def test_chunked_keys_on_the_tensor_core_portions_kernel(heads, kv_heads, dim, page, chunk, tensor_core, splits):
    ops = cuda_ops(torch.bfloat16)
    ops.tensor_core_attention, ops.portion_splits = tensor_core, splits
    sequences = random_sequences([(700, 700), (130, 1), (500, 129), (300, 300), (64, 2), (1000, 37)], heads, kv_heads, dim, 70)
    got, want = attend_both(ops, torch.bfloat16, sequences, page, heads, kv_heads, dim, dim ** -0.5 * 3, chunk)
    ops.check_status()
    close(got, want, TOL[torch.bfloat16], "portions on the tensor cores")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_len", [1, 2, 50])
@pytest.mark.parametrize("page,chunk,dim", [(16, 48, 32), (8, 20, 32), (5, 37, 32), (16, 16, 64), (16, 112, 64), (16, 33, 128)])
def test_a_key_at_the_chunks_edge_decides(dtype, q_len, page, chunk, dim):
    """The last query's direction is planted in one key: the first key of the query's own chunk (seen, and the
    output is that key's value), the last key of the chunk before (not seen: the output must not hold a trace of
    it), and the query's own key when it opens a chunk (it then sees nothing else)."""
    ops = cuda_ops(dtype)
    heads = kv_heads = 2
    for ctx in (3 * chunk + chunk // 2 + 1, 2 * chunk + 1, 4 * chunk):
        last = ctx - 1
        start = last // chunk * chunk
        for key, seen in ((start, True), (start - 1, False), (last, True)):
            if key < 0:
                continue
            g = torch.Generator().manual_seed(key)
            q, k, v = (torch.randn(ctx, heads, dim, generator=g) * 0.3 for _ in range(3))
            direction = torch.nn.functional.normalize(torch.randn(dim, generator=g), dim=0)
            q[last] = direction * 12.0
            k[key] = direction * 12.0
            v[key] = 100.0
            got, want = attend_both(ops, dtype, [(q, k, v, min(q_len, ctx))], page, heads, kv_heads, dim, 1.0, chunk)
            close(got, want, TOL[dtype] * 100, f"key {key} of context {ctx}")
            out = got[-1].float().view(heads, dim)
            assert (out.mean() > 90) == seen, f"chunk {chunk}, context {ctx}, key {key}: seen={seen}, output {out.mean():.2f}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_len", [1, 40])
def test_a_far_key_of_a_long_chunk_is_found_among_hundreds(dtype, q_len):
    ops = cuda_ops(dtype)
    heads, kv_heads, dim, page, ctx, chunk = 4, 1, 64, 16, 1500, 800
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(ctx, n, dim, generator=g) * 0.2 for n in (heads, kv_heads, kv_heads))
    far = 801                          # the second key of the last query's chunk, 698 positions back
    k[far] = 0.0
    k[far, 0, 5] = 3.0
    v[far] = 7.0
    q[ctx - 1] = 0.0
    q[ctx - 1, :, 5] = 8.0
    got, want = attend_both(ops, dtype, [(q, k, v, q_len)], page, heads, kv_heads, dim, 1.0, chunk)
    close(got, want, TOL[dtype] * 10, "far key")
    assert (got[-1].float() > 6.8).all()


# ------------------------------------------------------------------ matrix memory
def memory_case(heads, dim, vdim, cap, n, seed):
    """Weights and inputs whose gates move: forget gates between keeping all and nearly nothing."""
    width = 40
    names = {"q": heads * dim, "k": heads * dim, "v": heads * vdim, "g": heads * vdim, "i": heads, "f": heads}
    weights = {f"m.{name}": rnd(rows, width, seed=seed + i, scale=0.5) for i, (name, rows) in enumerate(names.items())}
    weights["m.i"] *= 3.0
    weights["m.f"] *= 3.0
    weights["m.i.b"], weights["m.f.b"] = rnd(heads, seed=seed + 7), rnd(heads, seed=seed + 8) + 1.0
    weights["m.norm"] = 1.0 + 0.2 * rnd(heads * vdim, seed=seed + 9)
    weights["m.o"] = torch.eye(heads * vdim)
    h = rnd(n, width, seed=seed + 10)
    spec = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    fused = torch.cat([h.double() @ weights[f"m.{name}"].double().T for name in names], dim=1).float()
    return weights, h, spec, fused


def run_memory(ops, dtype, fused, weights, spec, cuts, state, slot, partials=1, walk=False):
    heads, dim, vdim = spec["heads"], spec["dim"], spec["vdim"]
    outs, position = [], 0
    bias = torch.cat([weights["m.i.b"], weights["m.f.b"]]).float().to(DEV)
    for cut in cuts:
        piece = fused[position: position + cut].contiguous().to(DEV)
        if partials > 1:
            piece = torch.stack([piece * 0.5] + [piece * (0.5 / (partials - 1))] * (partials - 1)).contiguous()
        out = torch.empty(cut, heads * vdim, dtype=dtype, device=DEV)
        num = torch.empty(cut, heads * vdim, dtype=torch.float32, device=DEV)
        den = torch.empty(cut, heads, dtype=torch.float32, device=DEV)
        q_start = torch.tensor([0, cut], dtype=torch.int32, device=DEV)
        ops.matrix_memory(piece, bias, state, q_start, torch.tensor([slot], dtype=torch.int32, device=DEV), num, den,
                          weights["m.norm"].float().to(DEV), 1e-5, out, 1, heads, dim, vdim, spec["gate_cap"], 1e-6,
                          longest=0 if walk else cut)
        outs.append(out)
        position += cut
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,cap", [(2, 48, 32, 11.0), (3, 16, 24, 8.0), (1, 64, 64, 15.0), (2, 40, 8, 1.5), (3, 8, 40, 2.5),
                                                (1, 128, 256, 15.0), (2, 256, 40, 6.0), (2, 300, 70, 6.0)])
def test_matrix_memory_whole_in_portions_and_token_by_token(dtype, heads, dim, vdim, cap):
    ops = cuda_ops(dtype)
    n = 150
    weights, h, spec, fused = memory_case(heads, dim, vdim, cap, n, seed=heads * 100 + dim)
    trace = []
    want = pv.matrix_memory(h.double(), weights, "m", spec, 1e-5, False, trace=trace)
    m, S, z = trace[0]
    tol = 2e-4 if dtype == torch.float32 else 4e-2
    state = torch.zeros(3, heads, -(-(dim * vdim + dim + 1) // 4) * 4, dtype=torch.float32, device=DEV)
    state[1] = float("nan")                           # a neighbour's slot: never read, never written
    # whole (products over chunks of 64), the same as a walk token by token inside one launch, and cut into portions
    # that meet both forms and leave a chunk part full
    for slot, cuts, partials, walk in ((0, [n], 1, False), (0, [n], 1, True), (2, [1, 2, 7, 64, 3, 1, 1, 71], 3, False)):
        state[slot].zero_()
        got = run_memory(ops, dtype, fused, weights, spec, cuts, state, slot, partials, walk)
        close(got, want, tol, f"cuts {cuts}")
        held = state[slot].cpu().double()
        size = float(S.abs().max())              # the state's entries grow with the sequence: judged against their size
        close(held[:, : dim * vdim].view(heads, dim, vdim) / size, S / size, 1e-5, "S")
        close(held[:, dim * vdim: dim * vdim + dim] / float(z.abs().max()), z / float(z.abs().max()), 1e-5, "z")
        close(held[:, dim * vdim + dim], m, 1e-4, "m")
    assert torch.isnan(state[1]).all()
    state[0].zero_()                                  # the slot's next owner, token by token
    got = run_memory(ops, dtype, fused[:40], weights, spec, [1] * 40, state, 0)
    close(got, want[:40], tol, "token by token")


def test_matrix_memory_skips_padding_rows_and_leaves_them_finite():
    ops = cuda_ops(torch.float32)
    weights, h, spec, fused = memory_case(2, 16, 16, 5.0, 6, seed=3)
    state = torch.zeros(2, 2, 16 * 16 + 16 + 1, dtype=torch.float32, device=DEV)   # heads that start off a 16-byte border
    out = torch.full((6, 32), float("nan"), dtype=torch.float32, device=DEV)
    num, den = torch.full((6, 32), float("nan"), device=DEV), torch.full((6, 2), float("nan"), device=DEV)
    bias = torch.cat([weights["m.i.b"], weights["m.f.b"]]).float().to(DEV)
    ops.matrix_memory(fused.to(DEV), bias, state, torch.tensor([0, 1, 6], dtype=torch.int32, device=DEV),
                      torch.tensor([-1, 1], dtype=torch.int32, device=DEV), num, den, weights["m.norm"].float().to(DEV), 1e-5, out,
                      2, 2, 16, 16, 5.0, 1e-6)
    assert torch.isfinite(out).all() and float(state[0].abs().sum()) == 0 and float(state[1].abs().sum()) > 0
    want = pv.matrix_memory(h[1:].double(), weights, "m", spec, 1e-5, False)
    close(out[1:], want, 2e-4, "the request beside a padding row")


# ------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,width,shared", [(8, 3, 96, True), (5, 2, 70, True), (3, 3, 64, False), (6, 1, 72, True), (40, 6, 128, False)])
def test_router_picks_the_largest_and_renormalises(dtype, experts, top, width, shared):
    ops = cuda_ops(dtype)
    n = 37
    x = rnd(n, width, seed=1).to(dtype)
    weights = {"f.router": rnd(experts, width, seed=2, scale=0.6), "f.shared.sg": rnd(1, width, seed=3)}
    share = torch.full((n, experts + (1 if shared else 0)), float("nan"), dtype=torch.float32, device=DEV)
    ops.route_top(x.to(DEV), weights["f.router"].to(DEV), weights["f.shared.sg"].reshape(-1).to(DEV) if shared else None, share, top, 1e-20)
    chosen, portion = pv.route(x.double(), weights, "f", experts, top)
    want = torch.zeros(n, experts, dtype=torch.float64).scatter_(1, chosen, portion)
    close(share[:, :experts], want, 1e-5, "expert weights")
    assert ((share[:, :experts] > 0).sum(-1) == top).all()
    if shared:
        close(share[:, experts], torch.sigmoid(x.double() @ weights["f.shared.sg"].double().T)[:, 0], 1e-5, "shared gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,each,rest", [(8, 12, 16), (5, 40, 24), (3, 32, 0), (4, 7, 9)])
def test_activation_weighted_by_the_columns_expert(dtype, experts, each, rest):
    ops = cuda_ops(dtype)
    n, inter = 9, experts * each + rest
    gate_up = rnd(n, 2 * inter, seed=4, scale=1.5).to(dtype)
    gate_up[0, :each] = float("nan")                       # an expert the first token did not choose may hold anything
    share = torch.rand(n, experts + (1 if rest else 0), generator=torch.Generator().manual_seed(5))
    share[0, 0] = 0.0
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops.act_mul_blocks(gate_up.to(DEV), share.to(DEV), out, experts, each, "silu")
    g, u = gate_up.double()[:, :inter], gate_up.double()[:, inter:]
    column = torch.arange(inter)
    block = torch.where(column < experts * each, column // each, torch.full_like(column, experts))
    want = torch.nan_to_num(g * torch.sigmoid(g) * u) * share.double()[:, block]
    close(out, want, 1e-5 if dtype == torch.float32 else 6e-2, "weighted activation")
