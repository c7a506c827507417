"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)), silu(g) = g / (1 + exp(-g))
(src/model/qwen3.cpp:235-238, src/backend/cpu/cpu_backend.cpp:195-207). Gate and up are
stacked into one weight so that one product reads h once."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorNeed
from .base import FeedForward, register_part, to_compute


class SwiGLU(FeedForward):
    launches_only = True

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.dtype = dtype
        self.w_gate_up = self.w_down = None

    def needs(self):
        return {self.prefix + "gate_proj.weight": TensorNeed((self.inter, self.hidden)),
                self.prefix + "up_proj.weight": TensorNeed((self.inter, self.hidden)),
                self.prefix + "down_proj.weight": TensorNeed((self.hidden, self.inter))}

    def bind(self, get):
        gate = to_compute(get(self.prefix + "gate_proj.weight"), self.dtype)
        up = to_compute(get(self.prefix + "up_proj.weight"), self.dtype)
        # On the tensor-core path gate and up rows are interleaved in blocks of 16 and SiLU * up
        # happens in the product's epilogue; else they are stacked and a kernel of its own does it.
        self.fused = self.dtype == torch.bfloat16 and self.inter % 16 == 0 and self.hidden % 8 == 0
        self.gate_up = ops.bound_gemm(ops.interleave_gate_up(gate, up) if self.fused else torch.cat([gate, up], dim=0).contiguous(),
                                      silu=self.fused)
        del gate, up
        self.down = ops.bound_gemm(to_compute(get(self.prefix + "down_proj.weight"), self.dtype).contiguous())
        self.w_gate_up, self.w_down = self.gate_up.w, self.down.w      # as the products keep them (in k-blocks when they stream them)
        self._partial_capacity = None

    def forward(self, h, ctx):
        T = h.shape[0]
        act = ctx.ws.rows("ffn.act", T, self.inter, self.dtype)
        if self.fused:
            self.gate_up(h, act)
        else:
            gu = ctx.ws.rows("ffn.gate_up", T, 2 * self.inter, self.dtype)
            self.gate_up(h, gu)
            ops.silu_mul(gu, act)
        out = ctx.ws.rows("ffn.out", T, self.hidden, self.dtype)
        if self._partial_capacity is None:
            self._partial_capacity = ops.partial_capacity(ctx.ws.max_rows, self.down.N, self.down.K)
        return self.down(act, out, lambda n: ctx.ws.flat("ffn.out.partial", n, torch.float32, self._partial_capacity))


class ClampedGLU(FeedForward):
    """A gated unit with clamped branches: g = min(gate(h), limit), u = clamp(up(h), -limit, limit),
    y = g * sigmoid(slope * g) * (u + up_shift), then down(y). params: `hidden_size`, `intermediate_size`, `limit`,
    `slope`, `up_shift`, and the three tensors' names (`gate`, `up`, `down`) after `prefix`."""
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.limit, self.slope, self.up_shift = float(p["limit"]), float(p.get("slope", 1.0)), float(p.get("up_shift", 0.0))
        self.names = tuple(self.prefix + p.get(k, k) for k in ("gate", "up", "down"))
        self.dtype = dtype
        self._partial_capacity = None

    def needs(self):
        return {self.names[0]: TensorNeed((self.inter, self.hidden)), self.names[1]: TensorNeed((self.inter, self.hidden)),
                self.names[2]: TensorNeed((self.hidden, self.inter))}

    def bind(self, get):
        gate, up = (to_compute(get(n), self.dtype) for n in self.names[:2])
        self.gate_up = ops.bound_gemm(torch.cat([gate, up], dim=0).contiguous(), split_many=False)
        del gate, up
        self.down = ops.bound_gemm(to_compute(get(self.names[2]), self.dtype).contiguous())
        self.w_gate_up, self.w_down = self.gate_up.w, self.down.w

    def forward(self, h, ctx):
        T = h.shape[0]
        gu = ctx.ws.rows("ffn.gate_up", T, 2 * self.inter, self.dtype)
        self.gate_up(h, gu)
        act = ctx.ws.rows("ffn.act", T, self.inter, self.dtype)
        ops.glu_clamped(gu, act, self.limit, self.slope, self.up_shift)
        out = ctx.ws.rows("ffn.out", T, self.hidden, self.dtype)
        if self._partial_capacity is None:
            self._partial_capacity = ops.partial_capacity(ctx.ws.max_rows, self.down.N, self.down.K)
        return self.down(act, out, lambda n: ctx.ws.flat("ffn.out.partial", n, torch.float32, self._partial_capacity))


class BiasedGLU(FeedForward):
    """A gated unit whose three products have biases: down(act(gate(h) + b_gate) * (up(h) + b_up)) + b_down, with `act`
    "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))). Gate and up are one stacked product; their
    biases and the activation are one float kernel behind it. The down bias rides in the product: the unit's output
    gets a column of ones (and zeros up to a multiple of 8) and the weight the bias as that column, so it is added
    inside the float accumulator and split products still hand on partial sums. params: `hidden_size`,
    `intermediate_size`, `activation`, and the tensors' names (`gate`, `up`, `down`; biases `<name>.b`) after `prefix`."""
    launches_only = False
    ACTIVATIONS = {"silu": ops.ACT_SILU, "gelu_tanh": ops.ACT_GELU_TANH}

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        act = p.get("activation", "silu")
        if act not in self.ACTIVATIONS:
            from ..errors import UnsupportedError
            raise UnsupportedError(f"no activation '{act}' (known: {', '.join(sorted(self.ACTIVATIONS))})")
        self.act = self.ACTIVATIONS[act]
        self.names = tuple(self.prefix + p.get(k, k) for k in ("gate", "up", "down"))
        self.padded = (self.inter + 1 + 7) // 8 * 8          # the unit, the column of ones, zeros
        self.dtype = dtype
        self._partial_capacity = None

    def needs(self):
        g, u, d = self.names
        return {g: TensorNeed((self.inter, self.hidden)), u: TensorNeed((self.inter, self.hidden)),
                d: TensorNeed((self.hidden, self.inter)), g + ".b": TensorNeed((self.inter,), "norm"),
                u + ".b": TensorNeed((self.inter,), "norm"), d + ".b": TensorNeed((self.hidden,), "norm")}

    def bind(self, get):
        g, u, d = self.names
        gate, up = (to_compute(get(n), self.dtype) for n in (g, u))
        self.gate_up = ops.bound_gemm(torch.cat([gate, up], dim=0).contiguous(), split_many=False)
        del gate, up
        down = to_compute(get(d), self.dtype)
        wide = torch.zeros((self.hidden, self.padded), dtype=self.dtype, device=down.device)
        wide[:, :self.inter] = down
        wide[:, self.inter] = to_compute(get(d + ".b"), self.dtype)
        self.down = ops.bound_gemm(wide)
        self.w_gate_up, self.w_down = self.gate_up.w, self.down.w
        self.bias_gate, self.bias_up = (get(n + ".b").to(torch.float32).contiguous() for n in (g, u))

    def forward(self, h, ctx):
        T = h.shape[0]
        gu = ctx.ws.rows("ffn.gate_up", T, 2 * self.inter, self.dtype)
        self.gate_up(h, gu)
        act = ctx.ws.rows("ffn.act1", T, self.padded, self.dtype)
        ops.glu_biased(gu, self.bias_gate, self.bias_up, act, self.act)
        out = ctx.ws.rows("ffn.out", T, self.hidden, self.dtype)
        if self._partial_capacity is None:
            self._partial_capacity = ops.partial_capacity(ctx.ws.max_rows, self.down.N, self.down.K)
        return self.down(act, out, lambda n: ctx.ws.flat("ffn.out.partial", n, torch.float32, self._partial_capacity))


class TwoBranchMLP(FeedForward):
    """One hidden layer without a gate: down(act(up(h))), with an activation in two branches that meet at zero with the
    slope 1/2 and whose curvatures are learned, two numbers a layer (`<prefix>act` = [a_pos, a_neg]):

        z > 0:  softplus(a_pos) z^2 + z / 2;      z <= 0:  (1/2 + softplus(a_neg)) (exp(z) - 1 - z) + z / 2

    The two softplus are formed once, in float64, when the tensor is bound. params: `hidden_size`, `intermediate_size`, and
    the tensors' names (`up`, `down`, `act`) after `prefix`."""
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.names = tuple(self.prefix + p.get(k, k) for k in ("up", "down", "act"))
        self.dtype = dtype
        self._partial_capacity = None

    def needs(self):
        u, d, a = self.names
        return {u: TensorNeed((self.inter, self.hidden)), d: TensorNeed((self.hidden, self.inter)), a: TensorNeed((2,), "norm")}

    def bind(self, get):
        u, d, a = self.names
        self.up = ops.bound_gemm(to_compute(get(u), self.dtype).contiguous(), split_many=False)
        self.down = ops.bound_gemm(to_compute(get(d), self.dtype).contiguous())
        self.w_up, self.w_down = self.up.w, self.down.w
        a_pos, a_neg = (float(v) for v in get(a).to(torch.float64).cpu().reshape(-1)[:2])
        softplus = lambda v: float(torch.nn.functional.softplus(torch.tensor(v, dtype=torch.float64)))
        self.c_pos, self.c_neg = softplus(a_pos), 0.5 + softplus(a_neg)

    def forward(self, h, ctx):
        T = h.shape[0]
        z = ctx.ws.rows("ffn.gate_up", T, self.inter, self.dtype)
        self.up(h, z)
        act = ctx.ws.rows("ffn.act", T, self.inter, self.dtype)
        ops.two_branch_unit(z, act, self.c_pos, self.c_neg)
        out = ctx.ws.rows("ffn.out", T, self.hidden, self.dtype)
        if self._partial_capacity is None:
            self._partial_capacity = ops.partial_capacity(ctx.ws.max_rows, self.down.N, self.down.K)
        return self.down(act, out, lambda n: ctx.ws.flat("ffn.out.partial", n, torch.float32, self._partial_capacity))


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("feed_forward", "two_branch_mlp", TwoBranchMLP, replace=True)
register_part("feed_forward", "biased_glu", BiasedGLU, replace=True)
register_part("feed_forward", "clamped_glu", ClampedGLU, replace=True)
