"""Token embedding and the output table (src/model/qwen3.cpp:75,92-100,213,255-259): x[t] = table[id],
logits = last . W^T in float32, W = the embedding table when the model ties them."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import Embedding, OutputHead, register_part, to_compute


class TokenEmbedding(Embedding):
    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = spec["name"]
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.dtype = dtype
        self.table = None

    def needs(self):
        return {self.name: TensorNeed((self.vocab, self.hidden))}

    def bind(self, get):
        # Kept the way a matrix product streams it best (in k-blocks, for the tensor-core kernels): an output head
        # that shares the table multiplies by this very tensor (`product`), and a row of it is as cheap to gather.
        self.product = ops.bound_gemm(to_compute(get(self.name), self.dtype).contiguous())
        self.table = self.product.w

    def forward(self, tokens, x):
        ops.embed(self.table, tokens, x)


class NormedTokenEmbedding(TokenEmbedding):
    """x[t] = norm(table[id]): the looked-up rows pass a norm part (`norm`, a PartSpec of the norm family) before they
    become the residual stream."""

    def __init__(self, spec, dtype, prefix: str = ""):
        super().__init__(spec, dtype, prefix)
        from .base import build_part
        self.norm = build_part("norm", spec["norm"], torch.float32)

    def needs(self):
        return {**super().needs(), **self.norm.needs()}

    def bind(self, get):
        super().bind(get)
        self.norm.bind(get)

    def forward(self, tokens, x):
        ops.embed(self.table, tokens, x)
        self.norm.rows(x, x)            # float32 rows, in place


class PairHashEmbedding(TokenEmbedding):
    """x[t] = table[id] + pairs[row]: a second table is indexed by a hash of the pair (previous token, token),
    row = (prev * mul_prev + id * mul_cur) mod buckets; a sequence's first token takes the table's last row (`buckets`). The sum is
    float32. The previous token of a request is per-request state (one int32 in its state slot), so that a prompt may be cut
    anywhere. params beside `TokenEmbedding`'s: `pairs` = {"name", "buckets", "mul_prev", "mul_cur"}."""

    def __init__(self, spec, dtype, prefix: str = ""):
        super().__init__(spec, dtype, prefix)
        pairs = spec["pairs"]
        self.pairs_name = pairs["name"]
        self.buckets, self.mul_prev, self.mul_cur = int(pairs["buckets"]), int(pairs["mul_prev"]), int(pairs["mul_cur"])
        if self.buckets <= 0:
            raise InvalidArgument(f"a pair table needs a positive number of buckets, got {self.buckets}")
        self.pairs = None

    def needs(self):
        return {**super().needs(), self.pairs_name: TensorNeed((self.buckets + 1, self.hidden))}

    def bind(self, get):
        super().bind(get)
        self.pairs = to_compute(get(self.pairs_name), self.dtype).contiguous()

    def state_need(self):
        from .base import StateNeed
        return StateNeed((), torch.int32)

    def forward(self, tokens, x):
        raise InvalidArgument("this embedding reads the token before each token: it is called with the step (`forward_step`)")

    def forward_step(self, ctx, x, state):
        if state is None:
            raise InvalidArgument("the pair-hash embedding keeps a request's last token in a state slot: none was given")
        ops.embed(self.table, ctx.tokens, x)
        ops.pair_hash_add(x, self.pairs, ctx.tokens, ctx.positions, ctx.seq_of_row, ctx.query_start, ctx.state_slots, state,
                          self.buckets, self.mul_prev, self.mul_cur)


class SinusoidTokenEmbedding(TokenEmbedding):
    """x[t] = table[id] + e(position): e[2i] = sin(p * base^(-2i/hidden)), e[2i+1] = cos of the same angle, positions counted
    from 0 in each sequence. The sum is float32. params beside `TokenEmbedding`'s: `base` (10000 when absent)."""

    def __init__(self, spec, dtype, prefix: str = ""):
        super().__init__(spec, dtype, prefix)
        self.base = float(spec.params.get("base", 10000.0))

    def forward(self, tokens, x):
        raise InvalidArgument("this embedding reads each token's position: it is called with the step (`forward_step`)")

    def forward_step(self, ctx, x, state):
        ops.embed(self.table, ctx.tokens, x)
        ops.sinusoid_add(x, ctx.positions, self.base)


class LMHead(OutputHead):
    def __init__(self, spec, dtype, embedding: TokenEmbedding | None = None, prefix: str = ""):
        self.name = spec["name"]
        self.tied = bool(spec["tied"])
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.logit_scale = float(spec.params.get("logit_scale", 1.0))      # a constant factor on the float32 logits
        self.dtype = dtype
        self.embedding = embedding
        self.weight = None

    def needs(self):
        # A tied checkpoint may still carry a duplicate output table; it is accepted and ignored.
        return {self.name: TensorNeed((self.vocab, self.hidden), optional=self.tied)}

    def bind(self, get):
        if self.tied:
            if getattr(self.embedding, "product", None) is None:
                raise InvalidArgument("a tied output head needs an embedding part that offers the `product` with its table")
            self.product = self.embedding.product
        else:
            self.product = ops.bound_gemm(to_compute(get(self.name), self.dtype).contiguous())
        self.weight = self.product.w

    def forward(self, last, logits):
        self.product(last, logits)
        if self.logit_scale != 1.0:
            ops.scale_rows(logits, self.logit_scale)


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("embedding", "normed_token_embedding", NormedTokenEmbedding, replace=True)
register_part("embedding", "pair_hash_embedding", PairHashEmbedding, replace=True)
register_part("embedding", "sinusoid_token_embedding", SinusoidTokenEmbedding, replace=True)
register_part("head", "lm_head", LMHead, replace=True)
