"""A recurrent mixer that blends every input with the token before and reads its matrix state before it writes it.

With h' the row of the token before (zeros ahead of a sequence's first token), each of five inputs is a blend of its own,
x_s = h + (h' - h) * mu_s for s in r, k, v, g, w. Then, per head of `dim` key and value channels,

    r, k, v = x_r Wr^T, x_k Wk^T, x_v Wv^T;   gate = silu(x_g Wg^T)
    w       = exp(-exp(tanh(x_w W1^T) W2^T + w0))                        a decay per head and key channel, in (0, 1)
    o_t     = (S + diag(u) k_t v_t^T)^T r_t                              u: a weight per head and key channel on the token's own write
    S      <- diag(w_t) S + k_t v_t^T                                    S float32 [dim, dim], zero at the start of a sequence
    out     = ((o / sqrt(mean(o^2) + eps) per head) * norm * gate) Wo^T   `norm` has a weight per head and channel

A request's state is one float32 row in a state slot: S of every head, then the last row of h it has seen. The blends,
the decay from its raw projection on, S and the read-out's norm are float32 in either compute dtype. The recurrence is the
engine's plain recurrence kernel in its read-first mode. The inner size of the decay projection comes from its tensors'
shapes (`decay_rank`).
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import Mixer, StateNeed, register_part, to_compute

BLENDS = ("r", "k", "v", "g", "w")


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class TokenShiftRecurrence(Mixer):
    launches_only = False
    graph_safe = True       # the kernels read the step from device tensors only and skip sequences without a slot

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden, self.heads, self.dim = int(p["hidden_size"]), int(p["num_heads"]), int(p["head_dim"])
        self.rank = int(p["decay_rank"])
        self.eps = float(p.get("eps", 1e-6))
        if min(self.heads, self.rank) <= 0 or not 0 < self.dim <= 256:
            raise InvalidArgument(f"token-shift recurrence: bad sizes heads={self.heads} dim={self.dim} (1 to 256) decay rank={self.rank}")
        self.dtype = dtype
        self.n = self.heads * self.dim
        self.rank8 = _up8(self.rank)
        self.state_floats = self.heads * self.dim * self.dim       # S of every head; the kept row of h follows

    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D, n, name = self.hidden, self.n, self._name
        t = {name("mu." + s): TensorNeed((D,), "norm") for s in BLENDS}
        t.update({name(s): TensorNeed((n, D)) for s in ("r", "k", "v", "g")})
        t.update({name("w1"): TensorNeed((self.rank, D)), name("w2"): TensorNeed((n, self.rank)), name("w0"): TensorNeed((n,), "norm"),
                  name("u"): TensorNeed((self.heads, self.dim), "norm"), name("norm"): TensorNeed((n,), "norm"), name("o"): TensorNeed((D, n))})
        return t

    def bind(self, get):
        name = self._name
        f32 = lambda leaf: get(name(leaf)).to(torch.float32).contiguous()
        self.mu = torch.stack([f32("mu." + s) for s in BLENDS]).contiguous()
        self.gemms = [ops.bound_gemm(to_compute(get(name(s)), self.dtype).contiguous(), split_many=False) for s in ("r", "k", "v", "g")]
        w1 = to_compute(get(name("w1")), self.dtype)
        w1p = torch.zeros((self.rank8, self.hidden), dtype=self.dtype, device=w1.device)       # rows padded: tanh(0) = 0 meets zero columns
        w1p[:self.rank] = w1
        self.gemm_w1 = ops.bound_gemm(w1p, split_many=False)
        w2 = to_compute(get(name("w2")), self.dtype)
        w2p = torch.zeros((self.n, self.rank8), dtype=self.dtype, device=w2.device)
        w2p[:, :self.rank] = w2
        self.gemm_w2 = ops.bound_gemm(w2p, split_many=False)
        self.gemm_o = ops.bound_gemm(to_compute(get(name("o")), self.dtype).contiguous(), split_many=True)
        self.w0, self.bonus, self.norm_w = f32("w0"), f32("u").reshape(-1).contiguous(), f32("norm")
        self._capacity = None

    def state_need(self):
        return StateNeed((self.state_floats + self.hidden,), torch.float32)

    def forward(self, h, ctx, cache, state):
        T, D, n = h.shape[0], self.hidden, self.n
        if state is None:
            raise InvalidArgument("the token-shift recurrence needs state slots (make the cache with `make_cache`)")
        blends = ctx.ws.rows("tmix.blends", T, len(BLENDS) * D, self.dtype)
        ops.token_shift_mix(h, self.mu, state, self.state_floats, ctx, blends)
        proj = [ctx.ws.rows("tmix.proj." + s, T, n, self.dtype) for s in BLENDS[:4]]
        for i, gemm in enumerate(self.gemms):
            gemm(blends[:, i * D:(i + 1) * D], proj[i])
        inner = ctx.ws.rows("tmix.inner", T, self.rank8, torch.float32)
        self.gemm_w1(blends[:, 4 * D:5 * D], inner)
        inner_act = ctx.ws.rows("tmix.inner.act", T, self.rank8, self.dtype)
        ops.tanh_rows(inner, inner_act)
        decay = ctx.ws.rows("tmix.decay", T, n, torch.float32)
        self.gemm_w2(inner_act, decay)
        rn, kn, vn = (ctx.ws.rows("tmix." + s, T, n, torch.float32) for s in ("rn", "kn", "vn"))
        ops.time_mix_prep(proj[0], proj[1], proj[2], self.w0, rn, kn, vn, decay)
        o = ctx.ws.rows("tmix.o", T, n, torch.float32)
        ops.delta_rule_bonus(rn, kn, vn, decay, self.bonus, state, ctx, self.heads, self.dim, o)
        gated = ctx.ws.rows("tmix.gated", T, n, self.dtype)
        ops.time_mix_out(o, proj[3], self.norm_w, self.eps, gated, self.heads, self.dim, h, state, self.state_floats, ctx)
        out = ctx.ws.rows("tmix.mixed", T, D, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(gated, out, lambda m: ctx.ws.flat("tmix.mixed.partial", m, torch.float32, self._capacity))


class MixerSum(Mixer):
    """Mixers side by side on the same input, summed with one factor each: sum_i scale_i * mixer_i(h). At most one of them
    keeps pages and at most one keeps state, which become this mixer's own. The sum is handed on as an `ops.ScaledSum`:
    the residual add that follows forms it in float32. params: `parts` = [(PartSpec of a mixer, factor), ...] (two)."""
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        from .base import build_part
        self.parts = [(build_part("mixer", ps, dtype, prefix=prefix), float(c)) for ps, c in spec["parts"]]
        if len(self.parts) != 2:
            raise InvalidArgument(f"a sum of mixers has two of them, got {len(self.parts)}")
        if sum(m.cache_need() is not None for m, _ in self.parts) > 1 or sum(m.state_need() is not None for m, _ in self.parts) > 1:
            raise InvalidArgument("a sum of mixers: at most one of them keeps pages and at most one keeps state")
        self.mixers = tuple(m for m, _ in self.parts)
        self.graph_safe = all(m.graph_safe for m in self.mixers if m.state_need() is not None)

    def needs(self):
        n = {}
        for m in self.mixers:
            n.update(m.needs())
        return n

    def bind(self, get):
        for m in self.mixers:
            m.bind(get)

    def cache_need(self):
        return next((m.cache_need() for m in self.mixers if m.cache_need() is not None), None)

    def state_need(self):
        return next((m.state_need() for m in self.mixers if m.state_need() is not None), None)

    def forward(self, h, ctx, cache, state):
        return ops.ScaledSum([(m.forward(h, ctx, cache if m.cache_need() is not None else None,
                                         state if m.state_need() is not None else None), c) for m, c in self.parts])


register_part("mixer", "token_shift_recurrence", TokenShiftRecurrence, replace=True)
register_part("mixer", "mixer_sum", MixerSum, replace=True)
