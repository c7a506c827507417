"""Two kinds of attention whose query heads read slices of wider cached key rows, with float32 scores, softmax and
outputs on the kernels of `ops.attention_maps_*`.

`differential_attention`: two score maps a head over the same values.

    q [H, 2, dim], k [G, 2, dim], v [G, vdim] = h Wq^T, h Wk^T, h Wv^T      head by head as [map 1 | map 2] in the checkpoint;
                                                                             the engine keeps the rows of Wq map by map
    q, k   = (x / sqrt(mean(x^2) + eps)) * w      per head and map over dim, one weight for all of them (`q.norm`, `k.norm`)
    k, v  -> cache pages (a key row holds both maps of a kv head)
    a_m    = softmax(scale q_m k_m^T over the visible keys) v            m = 1, 2, each a softmax of its own
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                      one number a layer
    o      = a_1 - lambda a_2;  o <- (o / sqrt(mean(o^2) + eps)) * (1 - diff)     per head over vdim, no weight
    out    = (o * sigmoid(h Wg^T)) Wo^T                                   (`output_gate`)

`chunk` > 0: position i sees the keys j <= i with i // chunk == j // chunk, chunks counted from position 0 of the
sequence; 0: every j <= i. An entry that reads another entry's cache (`RunEntry.cache_of`) has no k, v and k.norm
tensors and computes its queries only.

`talking_heads_attention`: softmax weights mixed across heads before they meet the values.

    q [H, dim], k [G, dim], v [G, vdim] = h Wq^T, h Wk^T, h Wv^T
    s_g    = scale q_g . k_(g // (H/G));  s_g <- cap tanh(s_g / cap) (`softcap`);  s_g -= r1_g ln(1 + r2_g (i - j))  (`distance_bias`)
    p_g    = softmax(s_g over j <= i)
    p'_h   = sum_g M[h, g] p_g                                            M = `<prefix>talk` [H, H]
    out    = (p'_h v_(h // (H/G)))_h Wo^T

The engine never forms p': sum_j (sum_g M[h, g] p_g[j]) v_c[j] = sum_g M[h, g] (sum_j p_g[j] v_c[j]), so every head's
weights meet the values of EVERY kv head (a cached row holds all kv heads' keys, another all their values), each head
with an online softmax of its own, and the mix is a small product over the H x G results per token.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .attention import MAX_SPLITS, NUM_SMS, SPLIT_KEYS
from .base import CacheNeed, Mixer, register_part, to_compute


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class _SliceAttention(Mixer):
    """What both kinds share: the stacked product, the step into the cache, the attention calls, the output product."""
    launches_only = False

    def _sizes(self, p, prefix):
        self.prefix = prefix + p.get("prefix", "")
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("value_dim") or self.dim)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim)
        self.eps = float(p.get("eps", 1e-6))
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads or min(self.dim, self.vdim) <= 0:
            raise InvalidArgument(f"{self.heads} heads of {self.dim} (values of {self.vdim}) over {self.kv_heads} kv heads: impossible sizes")

    def _name(self, leaf):
        return self.prefix + leaf

    def _stack(self, get, sections, reorder=None):
        """sections: (leaf, column offset, rows); `reorder`: {leaf: function on the weight} for rows that are kept in another order."""
        first = get(self._name(sections[0][0]))
        stacked = torch.zeros((self.width, self.hidden), dtype=self.dtype, device=first.device)
        for leaf, off, n in sections:
            w = to_compute(get(self._name(leaf)), self.dtype)
            stacked[off:off + n] = reorder[leaf](w) if reorder and leaf in reorder else w
        self.gemm_in = ops.bound_gemm(stacked, split_many=False)
        self.w_in = self.gemm_in.w
        self.gemm_o = ops.bound_gemm(to_compute(get(self._name("o")), self.dtype).contiguous(), split_many=True)
        self.w_o = self.gemm_o.w
        self._capacity = None

    def _attend(self, q, cache, ctx, g, width, q_heads, group, sub_div, sub_count, tensor_cores=None, chunk=0, softcap=0.0, r1=None, r2=None):
        """The step's rows through attention into one float32 buffer [T, width]. Rows of sequences that bring several tokens come first;
        they go through `tensor_cores(out)` where the caller gives it, else through the CUDA-core kernel. Sequences that bring one
        token go through the split kernel."""
        T, m = q.shape[0], ctx.multi_rows
        out = ctx.ws.rows(self.tag + ".attended", T, width, torch.float32)
        if m > 0 and tensor_cores is not None:
            tensor_cores(out)
        elif m > 0:
            ops.attention_maps_rows(q, cache.k, cache.v, out, ctx.seq_of_row, ctx.query_start, ctx.context_lens, g.block_tables,
                                    m, q_heads, self.dim, group, sub_div, sub_count, self.scale, chunk=chunk, softcap=softcap, r1=r1, r2=r2)
        if ctx.single_count > 0:
            longest = ctx.single_max_context if chunk <= 0 else min(ctx.single_max_context, chunk)
            # splits enough to fill the SMs four times over with blocks, none shorter than 32 keys; the split size follows from
            # the step's longest context and its count of single rows, so a row's sums depend on the batch by their order only
            want = max(1, (4 * NUM_SMS) // max(1, ctx.single_count * cache.k.shape[1]))       # a block per (sequence, cached head, split)
            split_keys = max(32, -(-math.ceil(longest / want) // 32) * 32)
            while math.ceil(longest / split_keys) > MAX_SPLITS:
                split_keys *= 2
            max_splits = max(1, math.ceil(longest / split_keys))
            scratch = ctx.ws.flat(self.tag + ".split", ops.attention_split_scratch_floats(ctx.max_seqs, q_heads, cache.v.shape[3], MAX_SPLITS),
                                  torch.float32)
            ops.attention_maps_split(q, cache.k, cache.v, out, ctx.query_start, ctx.context_lens, g.block_tables, q_heads, self.dim,
                                     group, sub_div, sub_count, self.scale, ctx.single_seqs, ctx.single_count, split_keys, max_splits, scratch,
                                     chunk=chunk, softcap=softcap, r1=r1, r2=r2)
        return out

    def _project_out(self, heads_out, ctx):
        T = heads_out.shape[0]
        out = ctx.ws.rows(self.tag + ".mixed", T, self.hidden, self.dtype)
        if self._capacity is None:
            self._capacity = ops.partial_capacity(ctx.ws.max_rows, self.gemm_o.N, self.gemm_o.K)
        return self.gemm_o(heads_out, out, lambda m: ctx.ws.flat(self.tag + ".mixed.partial", m, torch.float32, self._capacity))


class DifferentialAttention(_SliceAttention):
    tag = "dattn"

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self._sizes(p, prefix)
        self.chunk = int(p.get("chunk") or 0)
        # how far back the cache is read by this entry and by the entries that read its cache (0: all the way)
        self.cache_span = int(p["cache_span"]) if p.get("cache_span") is not None else self.chunk
        self.diff = float(p["diff"])
        self.output_gate = bool(p.get("output_gate", True))
        self.own_kv = bool(p.get("own_kv", True))        # False: the entry reads another entry's cache
        self.dtype = dtype
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        self.q_dim, self.k_dim, self.v_dim, self.o_dim = H * 2 * dim, G * 2 * dim, G * vdim, H * vdim
        self.q_off = 0
        self.k_off = _up8(self.q_dim)
        self.v_off = self.k_off + (_up8(self.k_dim) if self.own_kv else 0)
        self.g_off = self.v_off + (_up8(self.v_dim) if self.own_kv else 0)
        self.width = self.g_off + (_up8(self.o_dim) if self.output_gate else 0)

    def needs(self):
        D, n = self.hidden, self._name
        t = {n("q"): TensorNeed((self.q_dim, D)), n("q.norm"): TensorNeed((self.dim,), "norm"), n("o"): TensorNeed((D, self.o_dim))}
        if self.own_kv:
            t.update({n("k"): TensorNeed((self.k_dim, D)), n("v"): TensorNeed((self.v_dim, D)), n("k.norm"): TensorNeed((self.dim,), "norm")})
        for leaf in ("lq1", "lk1", "lq2", "lk2"):
            t[n(leaf)] = TensorNeed((self.dim,), "norm")
        if self.output_gate:
            t[n("g")] = TensorNeed((self.o_dim, D))
        return t

    def bind(self, get):
        sections = [("q", self.q_off, self.q_dim)]
        if self.own_kv:
            sections += [("k", self.k_off, self.k_dim), ("v", self.v_off, self.v_dim)]
        if self.output_gate:
            sections.append(("g", self.g_off, self.o_dim))
        H, dim = self.heads, self.dim
        # queries map by map, [2, H, dim]: the heads that share a key slice are then neighbours, as the attention kernels want them
        self._stack(get, sections, {"q": lambda w: w.view(H, 2, dim, -1).transpose(0, 1).reshape(2 * H * dim, -1)})
        f32 = lambda leaf: get(self._name(leaf)).to(torch.float32).contiguous()
        self.wq = f32("q.norm")
        self.wk = f32("k.norm") if self.own_kv else None
        f64 = lambda leaf: get(self._name(leaf)).to(torch.float64).cpu()
        self.lam = float(torch.exp((f64("lq1") * f64("lk1")).sum()) - torch.exp((f64("lq2") * f64("lk2")).sum()) + self.diff)

    def cache_need(self):
        # a chunk never reaches further back than its own length: pages behind that go back like a window's
        return CacheNeed("window" if self.cache_span > 0 else "full", self.kv_heads, 2 * self.dim, self.cache_span, value_dim=self.vdim)

    def forward(self, h, ctx, cache, state):
        T, H = h.shape[0], self.heads
        g = ctx.groups[cache.group]
        if cache.writes != self.own_kv:
            raise InvalidArgument("differential attention: a layer with key and value projections writes its cache, one without reads another's")
        proj = ctx.ws.rows(self.tag + ".proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        ops.slice_norm_append(proj, self.q_off, 2 * H, self.k_off, 2 * self.kv_heads, self.v_off, self.v_dim, self.dim, self.wq, self.wk,
                              self.eps, g.slots if self.own_kv else None, cache.k if self.own_kv else None, cache.v if self.own_kv else None)
        q = proj[:, :self.q_dim]
        per = H // self.kv_heads
        tensor_cores = None
        if ctx.multi_rows > 0 and self.dim == self.vdim and per <= 16 and ops.attention_prompt_maps_takes(q, cache.k, cache.v, self.dim):
            tensor_cores = lambda out: ops.attention_prompt_maps(q, cache.k, cache.v, out, ctx.query_start, ctx.context_lens, g.block_tables,
                                                                 ctx.multi_seqs, ctx.multi_max_queries, 2 * H, 2 * self.kv_heads, self.dim,
                                                                 self.scale, chunk=self.chunk)
        heads_out = ctx.ws.rows(self.tag + ".heads", T, self.o_dim, self.dtype)
        maps = self._attend(q, cache, ctx, g, 2 * H * self.vdim, 2 * H, per, H, 2, tensor_cores, chunk=self.chunk)
        gate = proj[:, self.g_off:self.g_off + self.o_dim] if self.output_gate else None
        ops.diff_combine(maps, gate, self.lam, 1.0 - self.diff, self.eps, heads_out, H, self.vdim)
        return self._project_out(heads_out, ctx)


class TalkingHeadsAttention(_SliceAttention):
    tag = "talk"

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self._sizes(p, prefix)
        self.softcap = float(p.get("softcap") or 0.0)
        self.distance_bias = bool(p.get("distance_bias", True))
        self.head_mix = bool(p.get("head_mix", True))
        self.dtype = dtype
        H, G, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        self.q_dim, self.k_dim, self.v_dim, self.o_dim = H * dim, G * dim, G * vdim, H * vdim
        self.q_off = 0
        self.k_off = _up8(self.q_dim)
        self.v_off = self.k_off + _up8(self.k_dim)
        self.width = self.v_off + _up8(self.v_dim)

    def needs(self):
        D, n, H = self.hidden, self._name, self.heads
        t = {n("q"): TensorNeed((self.q_dim, D)), n("k"): TensorNeed((self.k_dim, D)), n("v"): TensorNeed((self.v_dim, D)),
             n("o"): TensorNeed((D, self.o_dim))}
        if self.distance_bias:
            t.update({n("r1"): TensorNeed((H,), "norm"), n("r2"): TensorNeed((H,), "norm")})
        if self.head_mix:
            t[n("talk")] = TensorNeed((H, H), "norm")
        return t

    def bind(self, get):
        self._stack(get, [("q", self.q_off, self.q_dim), ("k", self.k_off, self.k_dim), ("v", self.v_off, self.v_dim)])
        f32 = lambda leaf: get(self._name(leaf)).to(torch.float32).contiguous()
        self.r1, self.r2 = (f32("r1"), f32("r2")) if self.distance_bias else (None, None)
        self.mix = f32("talk") if self.head_mix else torch.eye(self.heads, dtype=torch.float32, device=self.w_in.device)

    def cache_need(self):
        # one cached head: a key row holds the keys of all kv heads, a value row all their values
        return CacheNeed("full", 1, self.k_dim, 0, value_dim=self.v_dim)

    def forward(self, h, ctx, cache, state):
        T, H, G = h.shape[0], self.heads, self.kv_heads
        g = ctx.groups[cache.group]
        if not cache.writes:
            raise InvalidArgument("this attention computes its own keys and values: it cannot read another entry's cache")
        proj = ctx.ws.rows(self.tag + ".proj", T, self.width, self.dtype)
        self.gemm_in(h, proj)
        ops.slice_norm_append(proj, self.q_off, H, self.k_off, G, self.v_off, self.v_dim, self.dim, None, None, self.eps, g.slots,
                              cache.k, cache.v)
        q = proj[:, :self.q_dim]
        tensor_cores = None
        if ctx.multi_rows > 0 and self.dim == self.vdim and H // G <= 16 and ops.attention_prompt_maps_takes(q, cache.k, cache.v, self.dim):
            def tensor_cores(out):      # one call per distance between a head's own kv head and the kv head whose values it weights
                for shift in range(G):
                    ops.attention_prompt_maps(q, cache.k, cache.v, out, ctx.query_start, ctx.context_lens, g.block_tables, ctx.multi_seqs,
                                              ctx.multi_max_queries, H, G, self.dim, self.scale, v_shift=shift, softcap=self.softcap,
                                              r1=self.r1, r2=self.r2)
        heads_out = ctx.ws.rows(self.tag + ".heads", T, self.o_dim, self.dtype)
        pairs = self._attend(q, cache, ctx, g, H * self.v_dim, H, H // G, H // G, G, tensor_cores, softcap=self.softcap, r1=self.r1,
                             r2=self.r2)       # [T, H, G, vdim]
        ops.head_talk(pairs, self.mix, heads_out, H, G, self.vdim)
        return self._project_out(heads_out, ctx)


register_part("mixer", "differential_attention", DifferentialAttention, replace=True)
register_part("mixer", "talking_heads_attention", TalkingHeadsAttention, replace=True)
