"""Causal softmax attention over a cached low-rank latent.

Per token only the latent c = RMS(Wdkv x) * weight is cached (`latent_rank` numbers, one plane of
pages).  Head h's keys and values are k = Wuk_h c and v = Wuv_h c, its score scale * q_h.k.  Neither
k nor v is ever formed for a cached token: the key projection is moved to the query and the value
projection to the output,

    q_h . (Wuk_h c_j) = (Wuk_h^T q_h) . c_j        sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j),

so the layer is attention with ONE key/value head of size `latent_rank` whose keys and values are
the same cached rows, between two small per-head products; it runs on the engine's paged attention
kernels as they are.  A layer without a latent of its own reads the pages another layer's run wrote
(the run order names the cache) with its own Wuk, Wuv, queries and output.  An optional gate
multiplies head h's output by sigmoid(Wg x)_h; it is applied to the attended latent, before the
value projection, which is linear.  Query, latent and gate come from one fused product.
"""

from __future__ import annotations

import torch

from .attention import padded_head
from .base import KVNeed, ParamSpec, register_part


class LatentAttention:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out = spec.num_heads * spec.head_dim
        v_out = spec.num_heads * spec.value_dim
        params = {"q_proj.weight": ParamSpec((q_out, spec.width), "matrix")}
        if spec.own_latent:
            params["kv_down.weight"] = ParamSpec((spec.latent_rank, spec.width), "matrix")
            params["kv_norm.weight"] = ParamSpec((spec.latent_rank,), "norm")
        params["k_up.weight"] = ParamSpec((q_out, spec.latent_rank), "matrix")
        params["v_up.weight"] = ParamSpec((v_out, spec.latent_rank), "matrix")
        if spec.gated:
            params["gate.weight"] = ParamSpec((spec.num_heads, spec.width), "matrix")
        params["o_proj.weight"] = ParamSpec((spec.width, v_out), "matrix")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        return [KVNeed(1, padded_head(spec.latent_rank), None, planes=1)]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        heads, dim, vdim, rank = spec.num_heads, spec.head_dim, spec.value_dim, spec.latent_rank
        self.padded = padded_head(rank)
        ops.check_head_dim(self.padded)
        rows = [tensors.pop("q_proj.weight")]
        self.latent_weight = None
        if spec.own_latent:
            rows.append(tensors.pop("kv_down.weight"))
            self.latent_weight = tensors.pop("kv_norm.weight").to(torch.float32).contiguous()
        if spec.gated:
            rows.append(tensors.pop("gate.weight"))
        self.w_in = torch.cat(rows).contiguous()
        k_up, v_up = tensors.pop("k_up.weight"), tensors.pop("v_up.weight")
        # per head: [padded rank, dim] takes a query to the latent space, [vdim, padded rank] brings the
        # attended latent back; the padding columns and rows are zero
        self.w_absorb = k_up.new_zeros(heads, self.padded, dim)
        self.w_absorb[:, :rank] = k_up.view(heads, dim, rank).transpose(1, 2)
        self.w_expand = v_up.new_zeros(heads, vdim, self.padded)
        self.w_expand[:, :, :rank] = v_up.view(heads, vdim, rank)
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.q_width = heads * dim
        self.in_width = self.w_in.shape[0]

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        heads, dim, vdim, padded = spec.num_heads, spec.head_dim, spec.value_dim, self.padded
        n = x.shape[0]
        fused = rt.buffer("qkv", (n, self.in_width), torch.float32)
        fused = ops.linear(x, self.w_in, fused, allow_partials=True)
        group, latents, _ = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, self.q_width), rt.act_dtype)
        gate = rt.buffer("head_gate", (n, heads), torch.float32) if spec.gated else None
        writes = spec.own_latent and run.writes_cache
        ops.latent_store(fused, self.latent_weight, spec.eps, q, latents if writes else None, view.slot_mapping, gate,
                         self.q_width, spec.latent_rank if spec.own_latent else 0, padded, heads if spec.gated else 0)
        q_latent = rt.buffer("q_latent", (n, heads, padded), rt.act_dtype)
        ops.head_linear(q.view(n, heads, dim), self.w_absorb, q_latent)
        attended = rt.buffer("attn_out", (n, heads * padded), rt.act_dtype)
        ops.paged_attention(
            q_latent.view(n, heads * padded), latents, latents, view.block_table, ctx.q_start, ctx.ctx_len,
            ctx.seq_of_token, heads, 1, padded, spec.scale, None, attended,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
        )
        if spec.gated:
            ops.head_scale(attended, gate, heads, padded)
        out = rt.buffer("head_out", (n, heads, vdim), rt.act_dtype)
        ops.head_linear(attended.view(n, heads, padded), self.w_expand, out)
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(out.view(n, heads * vdim), self.w_o, delta, allow_partials=True)


register_part("mixer", "latent_attention", LatentAttention)
