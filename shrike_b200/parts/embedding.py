"""Token embedding and output head: how ids enter the residual stream and how it leaves as logits.

The embedding copies one table row per token into the float32 residual
(shrike/models/qwen.py:161); the head multiplies the final norm's output at the wanted
rows by a [vocab, width] matrix, the embedding's own table when the model ties them
(qwen.py:192,211-212), into float32 logits.  Both are parts like the others, chosen by the
`kind` of `ModelConfig.embedding` and `ModelConfig.head`: an architecture that scales its
embedding, adds a learned position table or caps its logits registers a part of its own
instead of changing the model class.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, PendingSum, register_part


class TokenEmbedding:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "table")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.table = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        resid = self.runtime.buffer("resid", (ctx.num_tokens, self.spec.width), torch.float32)
        keep = ctx.carried.get("embedding_copy")   # a pass entry may ask for a second copy of what leaves here
        scale = getattr(self.spec, "scale", 1.0)
        if keep is None and scale == 1.0:
            self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens)
        else:
            self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens, scale=scale, keep=keep)
            if keep is not None:
                ctx.carried["embedding_copied"] = True
        return resid


class PassEntry:
    """What entering pass t over a run of repeated layers does to the residual: the embedding's output is
    added again (every pass but the first) and the learned vector step[t], in 32-bit, in the kernel that
    also adds whatever branch outputs are still pending."""

    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"step": ParamSpec((spec.passes, spec.width), "bias")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.step = tensors["step"].to(torch.float32).contiguous()
        self._kept = None

    def before_embedding(self, ctx) -> None:
        self._kept = None
        if self.spec.add_embedding and self.spec.passes > 1:
            self._kept = self.runtime.buffer("embedding_out", (ctx.num_tokens, self.spec.width), torch.float32)
            ctx.carried["embedding_copy"] = self._kept

    def begin(self, resid, ctx) -> None:
        if self._kept is not None and not ctx.carried.get("embedding_copied"):
            self._kept.copy_(resid)   # an embedding part that does not write the copy itself

    def forward(self, resid, delta, ctx, number: int):
        if not 0 <= number < self.spec.passes:
            raise ValueError(f"pass {number} of {self.spec.passes}")
        terms = PendingSum.of(delta)
        if number > 0 and self._kept is not None:
            terms.append((self._kept, 1.0))
        while len(terms) > 4:
            self.ops.tanh_norm(resid, terms[:4])
            terms = terms[4:]
        self.ops.tanh_norm(resid, terms, row_add=self.step[number])
        return resid, None


class TokenPositionEmbedding:
    """Token row plus the learned vector of the token's position, summed in 32-bit."""

    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "table"),
                "positions": ParamSpec((spec.max_positions, spec.width), "table")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.table = tensors["weight"]
        self.position_table = tensors["positions"].to(self.table.dtype).contiguous()

    def forward(self, ctx) -> torch.Tensor:
        resid = self.runtime.buffer("resid", (ctx.num_tokens, self.spec.width), torch.float32)
        self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens,
                       position_table=self.position_table, positions=ctx.positions)
        return resid


class LMHead:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "matrix")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.weight = tensors["weight"]

    def forward(self, hidden) -> torch.Tensor:
        logits = self.runtime.buffer("logits", (hidden.shape[0], self.spec.vocab), torch.float32)
        if hidden.shape[0]:
            self.ops.linear(hidden, self.weight, logits)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "token_position_embedding", TokenPositionEmbedding)
register_part("head", "lm_head", LMHead)
register_part("pass_entry", "pass_entry", PassEntry)
