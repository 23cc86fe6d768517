"""Token embedding and output head.

Embedding: a row gather without scaling (ampere_kv/runner.py:282) into the float32 residual
stream.  Head: ``logits = x W^T`` on the rows that were asked for, float32 out
(runner.py:297); a tied head reads the embedding matrix.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, CacheSpec, Embedding, Head, ParamSpec, build_part, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``tensor`` (the matrix's name under the prefix, default ``weight``), ``scale`` (the
    row is multiplied by it, default 1), ``position_tensor`` and ``max_positions`` (a learned table
    [max_positions, hidden] whose row of the token's position is added, unscaled; default none), ``pair_table`` (None,
    or ``tensor``, ``buckets``, ``mul_prev``, ``mul_cur``: a table [buckets + 1, hidden] whose row
    ``(previous token * mul_prev + token * mul_cur) mod buckets`` is added, unscaled, and its last row for a
    sequence's first token; the previous token of a step's first row is kept per request, as a state of one int32
    that the cache manager holds with the request's state slot)."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.vocab_size = int(spec.params["vocab_size"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.scale = float(spec.params.get("scale", 1.0))
        self.position_tensor = spec.params.get("position_tensor")
        self.max_positions = int(spec.params.get("max_positions") or 0)
        if self.position_tensor is not None and self.max_positions <= 0:
            raise ValueError("token_embedding: a position table needs 'max_positions'")
        self.pair_table = spec.params.get("pair_table")
        if self.pair_table is not None:
            self.pair_tensor = str(self.pair_table["tensor"])
            self.buckets, self.mul_prev, self.mul_cur = (int(self.pair_table[k]) for k in ("buckets", "mul_prev", "mul_cur"))
            if self.buckets <= 0:
                raise ValueError("token_embedding: a pair table needs a positive number of buckets")
        self.weight: torch.Tensor | None = None
        self.position_rows: torch.Tensor | None = None
        self.pair_rows: torch.Tensor | None = None

    def param_specs(self):
        specs = {self.tensor: ParamSpec((self.vocab_size, self.hidden_size))}
        if self.position_tensor is not None:
            specs[str(self.position_tensor)] = ParamSpec((self.max_positions, self.hidden_size))
        if self.pair_table is not None:
            specs[self.pair_tensor] = ParamSpec((self.buckets + 1, self.hidden_size))
        return specs

    def cache_spec(self) -> CacheSpec:
        # the request's newest token, as the bits of one float32 state entry
        return CacheSpec(kind="none", state_shape=(1,)) if self.pair_table is not None else CacheSpec()

    def load(self, tensors):
        self.weight = tensors[self.tensor].contiguous()
        if self.position_tensor is not None:
            self.position_rows = tensors[str(self.position_tensor)].contiguous()
        if self.pair_table is not None:
            self.pair_rows = tensors[self.pair_tensor].contiguous()

    def forward(self, token_ids: torch.Tensor, ctx, cache=None) -> torch.Tensor:
        hidden = ops.embedding(token_ids, self.weight, status=getattr(ctx, "status", None),
                               sampled=getattr(ctx, "sampled", None), scale=self.scale,
                               positions=ctx.positions if self.position_rows is not None else None,
                               position_rows=self.position_rows)
        if self.pair_rows is None:
            return hidden
        if cache is None or cache.state is None:
            raise ValueError("token_embedding: a pair table needs the request's state (its previous token)")
        return ops.pair_rows_add(hidden, token_ids, ctx.positions, ctx.cu_q, ctx.state_slots,
                                 cache.state.view(torch.int32), self.pair_rows, vocab=self.vocab_size,
                                 buckets=self.buckets, mul_prev=self.mul_prev, mul_cur=self.mul_cur,
                                 sampled=getattr(ctx, "sampled", None))


@register_embedding("normed_token_embedding")
class NormedTokenEmbedding(TokenEmbedding):
    """A row gather followed by a norm: the residual stream starts as the normed row.  params: those of
    ``token_embedding`` and ``norm`` (a PartSpec of a registered norm kind)."""

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.norm = build_part(NORMS, spec.params["norm"], hidden_size=self.hidden_size, dtype=torch.float32,
                               device=self.device)

    def children(self):
        return (self.norm,)

    def forward(self, token_ids: torch.Tensor, ctx, cache=None) -> torch.Tensor:
        rows = super().forward(token_ids, ctx, cache)
        # the norm part, asked for float32 activations, hands back the stream itself
        return self.norm.forward(rows, None, ctx)


@register_head("linear_head")
class LinearHead(Head):
    """params: ``vocab_size``, ``tied`` (read the embedding's matrix instead of one's own), ``tensor`` (the
    matrix's name under the prefix, default ``weight``), ``softcap`` (the logits become ``cap * tanh(logits / cap)``;
    default none).  A tied checkpoint may
    still carry the head's tensor: it is accepted if it equals the embedding's and refused if it differs."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.vocab_size = int(spec.params["vocab_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.softcap = float(spec.params["softcap"]) if spec.params.get("softcap") else 0.0
        if self.softcap < 0:
            raise ValueError("linear_head: softcap must be positive")
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {self.tensor: ParamSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors[self.tensor].contiguous()
        else:
            self._stored = tensors.get(self.tensor)

    def tie(self, embedding) -> None:
        if not self.tied:
            return
        if getattr(embedding, "weight", None) is None or tuple(embedding.weight.shape) != (self.vocab_size,
                                                                                           self.hidden_size):
            raise ValueError("a tied head needs an embedding with a [vocab, hidden] matrix named 'weight'")
        stored = getattr(self, "_stored", None)
        if stored is not None and not torch.equal(stored, embedding.weight):
            from ..weights.loader import WeightError
            name = f"{self.spec.prefix}.{self.tensor}" if self.spec.prefix else self.tensor
            raise WeightError(f"the checkpoint ties the head to the embedding but carries a different {name} "
                              f"(largest difference {float((stored.float() - embedding.weight.float()).abs().max()):.3g})")
        self._stored = None
        self.weight = embedding.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, out_dtype=torch.float32)
        return ops.softcap_(logits, self.softcap) if self.softcap else logits
