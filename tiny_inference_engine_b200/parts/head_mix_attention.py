"""Grouped-query attention whose scores are mixed across heads before the softmax:

    q, k, v = h Wq^T, h Wk^T, h Wv^T                 one product, the three weights stacked; keys of `head_dim`,
                                                     values of `value_dim`
    q, k    = pairs (2i, 2i+1) of the first `rotary_dim` dimensions of each head turned by position * theta^(-2i/rotary_dim)
    q, k    = x / sqrt(mean(x^2) + eps) per head     (`unit_qk`; no weight)
    k, v   -> cache pages
    s[g]    = scale * q_g . k_(kv head of g)         every query head g, float32
    s'[h]   = sum_g M[h, g] s[g]                     (`head_mix`: M is the tensor `<prefix>talk`, [heads, heads])
    p[h, j] = exp(s'[h, j]) / (sink + sum_j' exp(s'[h, j']))    `sink`: one more key of score 0 without a value
    out     = (p v) Wo^T

Rotation, unit norm, scores, mix and softmax are float32 whatever the compute dtype. Every size and constant is a
parameter; each of the rotation, the unit norm, the mix and the sink can be left out. The rotation's frequencies come from
the position part (`rope`: a table of inverse frequencies), which this mixer applies to neighbouring pairs.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .attention import MAX_SPLITS, NUM_SMS, SPLIT_KEYS
from .base import CacheNeed, Mixer, build_part, register_part, to_compute


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class HeadMixAttention(Mixer):
    launches_only = True

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.eps = float(p.get("eps", 1e-6))
        self.unit_qk = bool(p.get("unit_qk", False))
        self.head_mix = bool(p.get("head_mix", False))
        self.sink = bool(p.get("sink", False))
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise InvalidArgument(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.head_dim % 2:
            raise InvalidArgument(f"heads of {self.head_dim} cannot be rotated in pairs")
        self.dtype = dtype
        self.position = build_part("position", p["position"], dtype, prefix=self.prefix) if p.get("position") else None
        if self.position is not None and not self.position.is_identity:
            self.scale *= float(self.position.score_scale())
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.value_dim
        self.o_dim = self.heads * self.value_dim
        # columns of the stacked product, each section starting at a multiple of 8 (16 bytes of bfloat16)
        self.q_off = 0
        self.k_off = _up8(self.q_dim)
        self.v_off = self.k_off + _up8(self.k_dim)
        self.width = self.v_off + _up8(self.v_dim)
        self.mix = None

    def _name(self, leaf):
        return self.prefix + leaf

    def needs(self):
        D = self.hidden
        n = {self._name("q"): TensorNeed((self.q_dim, D)), self._name("k"): TensorNeed((self.k_dim, D)),
             self._name("v"): TensorNeed((self.v_dim, D)), self._name("o"): TensorNeed((D, self.o_dim))}
        if self.head_mix:
            n[self._name("talk")] = TensorNeed((self.heads, self.heads), "norm")
        if self.position is not None:
            n.update(self.position.needs())
        return n

    def bind(self, get):
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=get(self._name("q")).device)
        for leaf, off, n in (("q", self.q_off, self.q_dim), ("k", self.k_off, self.k_dim), ("v", self.v_off, self.v_dim)):
            stacked[off:off + n] = to_compute(get(self._name(leaf)), self.dtype)
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w
        self.gemm_o = ops.bound_gemm(to_compute(get(self._name("o")), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        self.mix = get(self._name("talk")).to(torch.float32).contiguous() if self.head_mix else None
        if self.position is not None:
            self.position.bind(get)
        self._capacity = None
        self._tensor_cores = None       # whether prompts of this geometry run on the tensor cores: asked at first use

    def cache_need(self):
        return CacheNeed("full", self.kv_heads, self.head_dim, 0, value_dim=0 if self.value_dim == self.head_dim else self.value_dim)

    def forward(self, h, ctx, cache, state):
        T = h.shape[0]
        H, G, Dk, Dv = self.heads, self.kv_heads, self.head_dim, self.value_dim
        g = ctx.groups[cache.group]
        if not cache.writes:
            raise InvalidArgument("this attention computes its own keys and values: it cannot read another entry's cache")
        proj = ctx.ws.rows("hmattn.proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        table = None
        if self.position is not None and not self.position.is_identity:
            table = self.position.fused_table()
            if table is None:
                raise InvalidArgument("this attention takes a rotation by a frequency table (or none) as its position encoding")
        ops.rope_pairs_unit_append(proj, self.q_off, self.k_off, self.v_off, table, self.unit_qk, self.eps, ctx.positions, g.slots,
                                   cache.k, cache.v, H, G, Dk, Dv)
        attn = ctx.ws.rows("hmattn.out", T, self.o_dim, self.dtype)
        q = proj[:, :self.q_dim]
        arrays = (ctx.seq_of_row, ctx.query_start, ctx.context_lens, g.block_tables)
        if self._tensor_cores is None:
            self._tensor_cores = self.dtype == torch.bfloat16 and ops.attention_mixed_tc_takes(H, G, Dk, Dv)
        if ctx.multi_rows > 0:
            if self._tensor_cores:
                ops.attention_mixed_tc(q, cache.k, cache.v, attn, self.mix, ctx.query_start, ctx.context_lens, g.block_tables,
                                       ctx.multi_seqs, ctx.multi_max_queries, H, G, Dk, Dv, self.scale, self.sink)
            else:
                ops.attention_mixed(q, cache.k, cache.v, attn, self.mix, arrays, ctx.multi_rows, H, G, Dk, Dv, self.scale, self.sink)
        if ctx.single_count > 0:
            # one block serves all heads of a split: enough splits to fill the SMs, none shorter than SPLIT_KEYS
            longest = ctx.single_max_context
            want = max(1, (2 * NUM_SMS) // max(1, ctx.single_count))
            split_keys = max(SPLIT_KEYS, -(-math.ceil(longest / want) // 64) * 64)
            while math.ceil(longest / split_keys) > MAX_SPLITS:
                split_keys *= 2
            max_splits = max(1, math.ceil(longest / split_keys))
            scratch = ctx.ws.flat("hmattn.split", ops.attention_split_scratch_floats(ctx.max_seqs, H, Dv, MAX_SPLITS), torch.float32)
            if self._tensor_cores:
                ops.attention_mixed_tc(q, cache.k, cache.v, attn, self.mix, ctx.query_start, ctx.context_lens, g.block_tables,
                                       ctx.single_count, 1, H, G, Dk, Dv, self.scale, self.sink, seq_list=ctx.single_seqs,
                                       split_keys=split_keys, max_splits=max_splits, scratch=scratch)
            else:
                ops.attention_mixed(q, cache.k, cache.v, attn, self.mix, arrays, 0, H, G, Dk, Dv, self.scale, self.sink,
                                    seq_list=ctx.single_seqs, n_list=ctx.single_count, split_keys=split_keys, max_splits=max_splits,
                                    scratch=scratch)
        out = ctx.ws.rows("mixer.out", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(attn, out, lambda m: ctx.ws.flat("mixer.out.partial", m, torch.float32, self._capacity))


register_part("mixer", "head_mix_attention", HeadMixAttention, replace=True)
