"""A recurrent mixer that blends every input with the token before and reads its matrix state before it writes it.

With h' the row of the token before (zeros ahead of a sequence's first token), each of five inputs is a blend of its own,
x_s = h + (h' - h) * mu_s for s in r, k, v, g, w. Then, per head of `dim` key and value channels,

    r, k, v = x_r Wr^T, x_k Wk^T, x_v Wv^T;   gate = silu(x_g Wg^T)
    w       = exp(-exp(tanh(x_w W1^T) W2^T + w0))                        a decay per head and key channel, in (0, 1)
    o_t     = (S + diag(u) k_t v_t^T)^T r_t                              u: a weight per head and key channel on the token's own write
    S      <- diag(w_t) S + k_t v_t^T                                    S float32 [dim, dim], zero at the start of a sequence
    out     = ((o / sqrt(mean(o^2) + eps) per head) * norm * gate) Wo^T   `norm` has a weight per head and channel

A request's state is one float32 row in a state slot: S of every head, then the last row of h it has seen. The decay from
its raw projection on, S and the read-out's norm are float32 in either compute dtype. The engine never forms the blends: with
W (1 - mu) and W mu, the columns of W scaled by the blend's factors (in float32, once, when the weights are bound),
x_s W^T = [h | h'] [W (1 - mu_s) | W mu_s]^T, so the five projections are ONE matrix product over the rows [h | h'], the
weights stacked; the second step of the decay's projection, over its few inner channels, runs in the kernel that forms the decays. The recurrence is the
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
        name, D, n = self._name, self.hidden, self.n
        f32 = lambda leaf: get(name(leaf)).to(torch.float32).contiguous()
        n8 = _up8(n)
        self.offs = {s: i * n8 for i, s in enumerate(("r", "k", "v", "g"))}       # columns of the stacked product
        self.inner_off = 4 * n8
        self.width = self.inner_off + self.rank8
        stacked = torch.zeros((self.width, 2 * D), dtype=torch.float32, device=get(name("r")).device)
        for s, leaf, off, rows in [(s, s, self.offs[s], n) for s in ("r", "k", "v", "g")] + [("w", "w1", self.inner_off, self.rank)]:
            w, mu = f32(leaf), f32("mu." + s)
            stacked[off:off + rows, :D] = w * (1.0 - mu)[None, :]
            stacked[off:off + rows, D:] = w * mu[None, :]
        self.gemm_in = ops.bound_gemm(stacked.to(self.dtype).contiguous(), split_many=False)
        self.w2t = f32("w2").t().contiguous()                 # [inner, n]: a thread a decay channel reads it coalesced
        self.gemm_o = ops.bound_gemm(to_compute(get(name("o")), self.dtype).contiguous(), split_many=True)
        self.w0, self.bonus, self.norm_w = f32("w0"), f32("u").reshape(-1).contiguous(), f32("norm")
        self._capacity = None

    def state_need(self):
        return StateNeed((self.state_floats + self.hidden,), torch.float32)

    def forward(self, h, ctx, cache, state):
        T, D, n = h.shape[0], self.hidden, self.n
        if state is None:
            raise InvalidArgument("the token-shift recurrence needs state slots (make the cache with `make_cache`)")
        pair = ctx.ws.rows("tmix.pair", T, 2 * D, self.dtype)
        ops.token_shift_concat(h, state, self.state_floats, ctx, pair)
        proj = ctx.ws.rows("tmix.proj", T, self.width, self.dtype)
        self.gemm_in(pair, proj)
        rn, kn, vn, decay = (ctx.ws.rows("tmix." + s, T, n, torch.float32) for s in ("rn", "kn", "vn", "decay"))
        ops.time_mix_prep(proj, self.offs["r"], self.offs["k"], self.offs["v"], self.inner_off, self.w2t, self.w0, rn, kn, vn, decay)
        o = ctx.ws.rows("tmix.o", T, n, torch.float32)
        ops.delta_rule_bonus(rn, kn, vn, decay, self.bonus, state, ctx, self.heads, self.dim, o)
        gated = ctx.ws.rows("tmix.gated", T, n, self.dtype)
        ops.time_mix_out(o, proj[:, self.offs["g"]:self.offs["g"] + n], self.norm_w, self.eps, gated, self.heads, self.dim, h, state, self.state_floats, ctx)
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
