"""Parts that rewrite the residual stream ahead of a run entry's layer (`RunEntry.before`).

`concat_projection`: x <- W [x; origin], one product over the stream and the embedding part's output side by side
(W is [hidden, 2 hidden], the stream's columns first). A model that runs a span of its layers several times puts one
ahead of each pass, so that every pass starts from the stream mixed with the embedding again. The pending delta of
the layer before is added first, in float32; the product reads both halves in the compute dtype and writes the float32
stream.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorNeed
from .base import StreamInput, register_part, to_compute


class ConcatProjection(StreamInput):
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = prefix + spec["name"]
        self.hidden = int(spec["hidden_size"])
        self.dtype = dtype

    def needs(self):
        return {self.name: TensorNeed((self.hidden, 2 * self.hidden))}

    def bind(self, get):
        self.product = ops.bound_gemm(to_compute(get(self.name), self.dtype).contiguous(), split_many=False)
        self.weight = self.product.w

    def forward(self, x, pending, origin, ctx):
        T, D = x.shape
        if isinstance(pending, ops.NormedDelta):
            raise NotImplementedError("concat_projection takes a plain delta or partial sums, not one that still has a norm to pass")
        both = ctx.ws.rows("stream.concat", T, 2 * D, self.dtype)
        ops.add_concat(x, pending, origin, both)
        self.product(both, x)
        return None


class PassVector(StreamInput):
    """x[t] += vectors[index]: one learned vector joins every row of the stream (float32) ahead of a pass over a span
    of layers; `vectors` is [passes, hidden] and every pass names its own row. params: `name`, `index`, `passes`,
    `hidden_size`."""
    launches_only = True
    reads_origin = False        # the model need not keep the embedding's output for it

    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = prefix + spec["name"]
        self.index, self.passes, self.hidden = int(spec["index"]), int(spec["passes"]), int(spec["hidden_size"])
        self.vector = None

    def needs(self):
        return {self.name: TensorNeed((self.passes, self.hidden))}

    def bind(self, get):
        self.vector = get(self.name)[self.index].to(torch.float32).contiguous()

    def forward(self, x, pending, origin, ctx):
        if pending is not None:
            raise NotImplementedError("pass_vector stands behind layers that leave the stream complete")
        ops.add_row_vector(x, self.vector)
        return None


register_part("stream_input", "concat_projection", ConcatProjection, replace=True)
register_part("stream_input", "pass_vector", PassVector, replace=True)
