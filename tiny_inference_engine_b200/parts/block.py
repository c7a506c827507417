"""Pre-norm arrangement of a layer: x += mixer(norm(x)); x += ffn(norm(x))
(src/model/qwen3.cpp:214-239). Each residual add is fused with the norm that follows it, so
the feed-forward's output is handed on as a pending delta that the next layer's first norm
(or the final norm) adds."""
from __future__ import annotations

import torch

from .base import Block, build_part, register_part


class PreNormBlock(Block):
    launches_only = True

    def __init__(self, layer_spec, dtype, prefix: str = ""):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, dtype)
        self.mixer = build_part("mixer", layer_spec.mixer, dtype)
        self.has_ffn = layer_spec.ffn is not None          # a layer may be a mixer alone
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm, dtype) if self.has_ffn else None
        self.ffn = build_part("feed_forward", layer_spec.ffn, dtype) if self.has_ffn else None
        self.dtype = dtype
        self.parts = (self.mixer_norm, self.mixer) + ((self.ffn_norm, self.ffn) if self.has_ffn else ())

    def needs(self):
        n = {}
        for p in self.parts:
            n.update(p.needs())
        return n

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def forward(self, x, pending, ctx, cache, state):
        """`pending` and what the parts return may be tensors [T, D] or ops.SplitSum (a split product
        whose partial sums the next add+norm adds up itself)."""
        h = ctx.ws.rows("block.normed", x.shape[0], x.shape[1], self.dtype)
        self.mixer_norm.add_norm(x, as_delta(pending, self.mixer_norm, ctx, "block.delta"), h)
        mixed = self.mixer.forward(h, ctx, cache, state)
        if not self.has_ffn:
            return mixed
        self.ffn_norm.add_norm(x, as_delta(mixed, self.ffn_norm, ctx, "block.delta"), h)
        return self.ffn.forward(h, ctx)


def as_delta(delta, norm, ctx, name):
    """A SplitSum stays one for norms that add the splits themselves (`takes_split_sum`), else it is added up first;
    likewise a ScaledSum (sublayer outputs with a factor each) for norms that say `takes_scaled_sum`."""
    from .. import ops
    if isinstance(delta, ops.SplitSum) and not getattr(norm, "takes_split_sum", False):
        return delta.materialize(ctx.ws.rows(name, delta.M, delta.N, ctx.ws_dtype))
    if isinstance(delta, ops.ScaledSum) and not getattr(norm, "takes_scaled_sum", False):
        first = delta.terms[0][0]
        M, N = (first.M, first.N) if isinstance(first, ops.SplitSum) else first.shape
        return delta.materialize(ctx.ws.rows(name, M, N, ctx.ws_dtype))
    return delta


class SandwichNormBlock(Block):
    """A norm before and after each sublayer, and a factor on what joins the residual stream:

        x += mult * norm_b(mixer(norm_a(x)));   x += mult * norm_d(ffn(norm_c(x)))

    A layer may have no feed-forward (`LayerSpec.ffn` None): then it is the first line alone. A sublayer's output
    is handed on as an `ops.NormedDelta` (the raw output, the weight and eps of the norm it still has to pass, the
    factor, and a bias of the sublayer's last product where it has one: a mixer says so with an `output_bias`
    attribute, float32 [D]); the add+norm ahead of the next sublayer (or the model's final norm) finishes it, all in
    float32. params: `residual_mult`."""
    launches_only = False

    def __init__(self, layer_spec, dtype, prefix: str = ""):
        self.mult = float(layer_spec.block.params.get("residual_mult", 1.0))
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, dtype)
        self.mixer = build_part("mixer", layer_spec.mixer, dtype)
        self.mixer_post_norm = build_part("norm", layer_spec.mixer_post_norm, dtype)
        self.has_ffn = layer_spec.ffn is not None
        self.parts = (self.mixer_norm, self.mixer, self.mixer_post_norm)
        if self.has_ffn:
            self.ffn_norm = build_part("norm", layer_spec.ffn_norm, dtype)
            self.ffn = build_part("feed_forward", layer_spec.ffn, dtype)
            self.ffn_post_norm = build_part("norm", layer_spec.ffn_post_norm, dtype)
            self.parts += (self.ffn_norm, self.ffn, self.ffn_post_norm)
        self.dtype = dtype

    def needs(self):
        n = {}
        for p in self.parts:
            n.update(p.needs())
        return n

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def _normed(self, delta, norm, bias=None):
        from .. import ops
        return ops.NormedDelta(delta, norm.weight, norm.eps, self.mult, bias)

    def forward(self, x, pending, ctx, cache, state):
        h = ctx.ws.rows("block.normed", x.shape[0], x.shape[1], self.dtype)
        self.mixer_norm.add_norm(x, as_delta(pending, self.mixer_norm, ctx, "block.delta"), h)
        mixed = self._normed(self.mixer.forward(h, ctx, cache, state), self.mixer_post_norm,
                             getattr(self.mixer, "output_bias", None))
        if not self.has_ffn:
            return mixed
        self.ffn_norm.add_norm(x, mixed, h)
        return self._normed(self.ffn.forward(h, ctx), self.ffn_post_norm)


SIDE_PRODUCT_ROWS = 256      # from this many rows of a step on, a parallel block's token side input runs as two matrix products


class ParallelBlock(Block):
    """Both sublayers read the same stream, side by side, and join it with one factor:

        h1 = in1(norm1(x)),  h2 = in2(norm2(x)),  x += mult * (mixer(h1) + ffn(h2))

    `in` is an optional short causal convolution over time per channel that is ADDED to what it reads:
    in(h)_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j), zeros ahead of the sequence (`taps`, tensors
    `<prefix><conv_names[0|1]>` of shape [hidden, taps]). The norms are RMS norms over groups of a row (`grouped_rmsnorm`;
    one group is the plain norm) with one eps and one number of groups, so that both sublayers' inputs come from the same
    unit rows u = x / rms: norm(x) = u * w, and the convolution runs over u with the norm's weight outside. The last
    taps - 1 unit rows of a request are its state in this layer (float32 [taps - 1, hidden], by position mod taps - 1),
    one state per run entry; both sublayers read that one ring.

    Then, optionally (`side`), a token input of the layer: e = table[token] (a slice of `side.table`, `side.dim` wide,
    at column `side.index * side.dim`), g = gelu_tanh(W_gate x) * e, y = W_proj g,
    x += mult * y / sqrt(mean(y^2) + eps) * w_norm, on the stream as the sublayers left it.

    Few rows (decoding) take the side input in the kernel that also adds the sublayers' outputs; from `SIDE_PRODUCT_ROWS` rows on
    its two products are matrix products (the stream's copy in the compute dtype times W_gate, g times W_proj into float32)
    between three small kernels.

    A layer may have no feed-forward. The stream, its sums, the norms and the convolution are float32. The block leaves
    the stream complete (it hands on no pending delta). params: `residual_mult`, `taps`, `conv_names`, `side`
    ({"table", "index", "dim", "gate", "proj", "norm", "eps"}), `hidden_size`."""
    launches_only = False
    graph_safe = True        # reads the step through device tensors only; padding sequences have no slot and no ring

    def __init__(self, layer_spec, dtype, prefix: str = ""):
        from ..errors import InvalidArgument
        p = layer_spec.block.params
        self.prefix = layer_spec.prefix
        self.hidden = int(p["hidden_size"])
        self.mult = float(p.get("residual_mult", 1.0))
        self.taps = int(p.get("taps") or 0)
        self.conv_names = tuple(p.get("conv_names") or ("conv1", "conv2"))
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, dtype)
        self.mixer = build_part("mixer", layer_spec.mixer, dtype)
        self.has_ffn = layer_spec.ffn is not None
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm, dtype) if layer_spec.ffn_norm is not None else None
        self.ffn = build_part("feed_forward", layer_spec.ffn, dtype) if self.has_ffn else None
        norms = [self.mixer_norm] + ([self.ffn_norm] if self.has_ffn else [])
        for n in norms:
            if not all(hasattr(n, a) for a in ("groups", "eps", "size")):
                raise InvalidArgument("a parallel block takes RMS norms over groups of a row (`grouped_rmsnorm`)")
        if len({(n.groups, n.eps) for n in norms}) != 1:
            raise InvalidArgument("the norms of a parallel block share one eps and one number of groups")
        if self.taps < 0 or self.taps > 8:
            raise InvalidArgument(f"a sublayer's input convolution has 0 to 8 taps, got {self.taps}")
        if self.mixer.state_need() is not None:
            raise InvalidArgument("a parallel block keeps the state of its input convolutions: its mixer may keep none")
        self.groups, self.eps = self.mixer_norm.groups, self.mixer_norm.eps
        side = p.get("side")
        self.side_spec = dict(side) if side else None
        self.side = None
        self.dtype = dtype
        self.parts = tuple(x for x in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if x is not None)
        self.taps_a = self.taps_b = None

    def needs(self):
        from ..weights.loader import TensorNeed
        n = {}
        for part in self.parts:
            n.update(part.needs())
        if not self.has_ffn and self.ffn_norm is not None:     # a checkpoint may carry the unused norm: accepted, not required
            n.update({k: TensorNeed(v.shape, v.role, optional=True) for k, v in self.ffn_norm.needs().items()})
        if self.taps > 0:
            n[self.prefix + self.conv_names[0]] = TensorNeed((self.hidden, self.taps))
            n[self.prefix + self.conv_names[1]] = TensorNeed((self.hidden, self.taps), optional=not self.has_ffn)
        if self.side_spec is not None:
            s = self.side_spec
            n[s["table"]] = TensorNeed((int(s["vocab_size"]), int(s["table_width"])))
            n[self.prefix + s["gate"]] = TensorNeed((int(s["dim"]), self.hidden))
            n[self.prefix + s["proj"]] = TensorNeed((self.hidden, int(s["dim"])))
            n[self.prefix + s["norm"]] = TensorNeed((self.hidden,), "norm")
        return n

    def bind(self, get):
        from .base import to_compute
        for part in self.parts:
            if part is self.ffn_norm and not self.has_ffn:
                continue
            part.bind(get)
        f32 = lambda name: get(name).to(torch.float32).contiguous()
        if self.taps > 0:
            by_tap = lambda name: get(name).to(torch.float32).t().contiguous()      # [taps, hidden]: a tap of every channel side by side
            self.taps_a = by_tap(self.prefix + self.conv_names[0])
            self.taps_b = by_tap(self.prefix + self.conv_names[1]) if self.has_ffn else None
        if self.side_spec is not None:
            s = self.side_spec
            dim, at = int(s["dim"]), int(s["index"]) * int(s["dim"])
            table = to_compute(get(s["table"])[:, at:at + dim], self.dtype).contiguous()
            self.side = (table, to_compute(get(self.prefix + s["gate"]), self.dtype).contiguous(),
                         to_compute(get(self.prefix + s["proj"]), self.dtype).contiguous(), f32(self.prefix + s["norm"]))
            self.side_eps = float(s.get("eps", self.eps))
            from .. import ops
            # the same two weights for the many-row path (a second copy: a few hundred KB a layer)
            self.gemm_gate = ops.bound_gemm(self.side[1].clone(), split_many=False)
            self.gemm_proj = ops.bound_gemm(self.side[2].clone(), split_many=False)

    def state_need(self):
        from .base import StateNeed
        return StateNeed((self.taps - 1, self.hidden), torch.float32) if self.taps > 1 else None

    def state_part(self):
        return self

    def forward(self, x, pending, ctx, cache, state):
        from .. import ops
        T, D = x.shape
        if pending is not None:          # what an earlier layer of another arrangement left to add
            ops.parallel_finish(x, 1.0, pending, None, self.dtype)
        h1 = ctx.ws.rows("pblock.h1", T, D, self.dtype)
        h2 = ctx.ws.rows("pblock.h2", T, D, self.dtype) if self.has_ffn else None
        ring = state if self.taps > 1 else None
        if self.taps > 1 and ring is None:
            from ..errors import InvalidArgument
            raise InvalidArgument("a parallel block with an input convolution keeps rows per request: no state slots were given")
        unit = ctx.ws.rows("pblock.unit", T, D, torch.float32) if ring is not None else None
        ops.group_norm_taps(x, self.groups, self.eps, self.mixer_norm.weight, h1, self.ffn_norm.weight if self.has_ffn else None, h2,
                            self.taps_a, self.taps_b, ctx=ctx, unit=unit, ring=ring)
        mixed = self.mixer.forward(h1, ctx, cache, None)
        fed = self.ffn.forward(h2, ctx) if self.has_ffn else None
        if self.side is not None and T >= SIDE_PRODUCT_ROWS:
            n = self.side[1].shape[0]
            copy = ctx.ws.rows("pblock.copy", T, D, self.dtype)
            ops.parallel_sum(x, self.mult, mixed, fed, copy)
            pre = ctx.ws.rows("pblock.side.pre", T, n, torch.float32)
            self.gemm_gate(copy, pre)
            g = ctx.ws.rows("pblock.side.g", T, n, self.dtype)
            ops.side_gate_act(pre, self.side[0], ctx.tokens, g)
            y = ctx.ws.rows("pblock.side.y", T, D, torch.float32)
            self.gemm_proj(g, y)
            ops.side_finish(x, y, self.mult, self.side_eps, self.side[3], ctx=ctx, unit=unit, ring=ring)
            return None
        ops.parallel_finish(x, self.mult, mixed, fed, self.dtype, ctx=ctx, side=self.side,
                            eps=self.side_eps if self.side is not None else 0.0, unit=unit, ring=ring)
        return None


register_part("block", "prenorm", PreNormBlock, replace=True)
register_part("block", "sandwich_norm", SandwichNormBlock, replace=True)
register_part("block", "parallel", ParallelBlock, replace=True)
