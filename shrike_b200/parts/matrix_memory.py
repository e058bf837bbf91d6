"""A recurrent mixer whose state is a matrix per head (the mLSTM cell of xLSTM).

Per head, with q scaled by dim^(-1/2), log gates a_t = cap tanh((w_i x + b_i) / cap) and
f_t = logsigmoid(cap tanh((w_f x + b_f) / cap)), and a running maximum m (m_0 = 0):

    m_t = max(f_t + m_(t-1), a_t)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T        (z_t likewise with k_t alone)
    o_t = S_t^T q_t / (max(|z_t . q_t|, exp(-m_t)) + floor)

Each head's o_t is divided by its root mean square; the heads, side by side, are scaled by one
weight, gated by sigmoid(Wg x) and projected.  S, z and m of every head are the request's state: one
float32 slot `[heads, dim * vdim + dim + 1 (rounded up to four)]`, zeroed by the step function when the request is opened
(so m_0 = 0 needs nothing of its own), read and left updated by the scan kernel, whatever the cut of
the prompt.  All six projections are one matrix product; gates, decays and the state are 32-bit.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, StateNeed, register_part


def padded_rows(matrix: torch.Tensor, multiple: int = 16) -> torch.Tensor:
    """`matrix` with rows of zeros added up to a multiple: a fused projection whose output rows are a whole
    number of 64 bytes gets the library's aligned product kernels."""
    extra = -matrix.shape[0] % multiple
    if extra:
        matrix = torch.cat([matrix, matrix.new_zeros(extra, matrix.shape[1])])
    return matrix.contiguous()


class MatrixMemory:
    capture_safe = True   # it reads the batch's metadata on the device only and skips rows whose state slot is -1

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        qk, v = spec.num_heads * spec.head_dim, spec.num_heads * spec.value_dim
        return {
            "q_proj.weight": ParamSpec((qk, spec.width), "matrix"),
            "k_proj.weight": ParamSpec((qk, spec.width), "matrix"),
            "v_proj.weight": ParamSpec((v, spec.width), "matrix"),
            "gate.weight": ParamSpec((v, spec.width), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, v), "matrix"),
            "norm.weight": ParamSpec((v,), "norm"),
            "input_gate.weight": ParamSpec((spec.num_heads, spec.width), "matrix"),
            "input_gate.bias": ParamSpec((spec.num_heads,), "bias"),
            "forget_gate.weight": ParamSpec((spec.num_heads, spec.width), "matrix"),
            "forget_gate.bias": ParamSpec((spec.num_heads,), "bias"),
        }

    @staticmethod
    def state_shape(spec) -> tuple:
        floats = spec.head_dim * spec.value_dim + spec.head_dim + 1      # S, z and m of a head
        return (spec.num_heads, -(-floats // 4) * 4)                      # every head starts on a 16-byte border

    @staticmethod
    def cache_needs(spec) -> list:
        return [StateNeed(MatrixMemory.state_shape(spec), "float32")]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        first = tensors["q_proj.weight"]
        rows = [tensors.pop(name) for name in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate.weight")]
        rows += [tensors.pop("input_gate.weight").to(first.dtype), tensors.pop("forget_gate.weight").to(first.dtype)]
        self.w_fused = padded_rows(torch.cat(rows))
        self.total = self.w_fused.shape[0]
        self.gate_bias = torch.cat([tensors.pop("input_gate.bias"), tensors.pop("forget_gate.bias")]).to(torch.float32).contiguous()
        self.norm_weight = tensors.pop("norm.weight").to(torch.float32).contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.out_width = spec.num_heads * spec.value_dim

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        if not run.writes_cache:
            raise NotImplementedError("a matrix memory owns its state: no run can read another run's")
        n = x.shape[0]
        fused = rt.buffer("memory_in", (n, self.total), torch.float32)
        fused = ops.linear(x, self.w_fused, fused, allow_partials=True)
        numerator = rt.buffer("memory_num", (n, self.out_width), torch.float32)
        denominator = rt.buffer("memory_den", (n, spec.num_heads), torch.float32)
        out = rt.buffer("memory_out", (n, self.out_width), rt.act_dtype)
        ops.matrix_memory(fused, self.gate_bias, ctx.storage.state[run.cache], ctx.q_start, ctx.state_slot, numerator,
                          denominator, self.norm_weight, spec.eps, out, ctx.num_seqs, spec.num_heads, spec.head_dim,
                          spec.value_dim, spec.gate_cap, spec.denominator_floor, longest=ctx.max_q_len)
        delta = rt.buffer("memory_delta", (n, spec.width), torch.float32)
        return ops.linear(out, self.w_o, delta, allow_partials=True)


register_part("mixer", "matrix_memory", MatrixMemory)
