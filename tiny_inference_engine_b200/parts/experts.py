"""A feed-forward of many small experts of which each token uses a few.

    s      = softmax(h Wr^T) over all experts, or sigmoid(h Wr^T) each (`score`: "softmax" | "sigmoid")   float32
    c      = s + correction                                         (`correction`: a tensor `<prefix>correction` [experts]; else c = s)
    chosen = the `top` experts with the largest c among the experts of the `group_keep` best of `group_count` equal
             blocks of consecutive experts (a block's score is the sum of its `group_top` largest c, 1: its best
             member's; ties go to the lower index; experts of other blocks count as minus infinity)
    weight = s[chosen] / (sum of s[chosen] + 1e-20), or s[chosen] as it is (`renorm` false), times `weight_scale`
    out    = sum over chosen of weight * expert(h)
    expert = down(g * sigmoid(slope * g) * (u + up_shift)),  g = min(gate(h), limit), u = clamp(up(h), -limit, limit)
             (`limit` None: no clamps; with slope 1 and up_shift 0 that is silu(gate(h)) * up(h))

The router's product writes float32; routing (softmax, groups, top-k, weights) is one float kernel. Tokens are then
listed by expert on the device (nothing of a step's routing reaches the host, so decode steps stay captured graphs),
and two grouped products run over that list, the clamped unit between them. The second product writes
weight * result as float32 partial sums [top, tokens, hidden], which the block's next residual add sums in order:
the weighted sum over experts happens in float32 in the residual add itself. What a token computes depends on its
own experts only, never on what else is in the step. params: `hidden_size`, `intermediate_size`, `num_experts`, `top`,
`group_count`, `group_keep`, `group_top`, `score`, `correction`, `renorm`, `weight_scale`, `limit`, `slope`, `up_shift`; tensors `<prefix>router` and `<prefix>e<i>.gate|up|down`.
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import InvalidArgument
from ..weights.loader import TensorNeed
from .base import FeedForward, register_part, to_compute


ROUTER_SIMT_ROWS = 16      # up to this many tokens the router's product runs on the CUDA cores (it is a few hundred KB)


class RoutedExperts(FeedForward):
    launches_only = False

    def __init__(self, spec, dtype, prefix: str = ""):
        p = spec.params
        self.prefix = prefix + p.get("prefix", "")
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.experts, self.top = int(p["num_experts"]), int(p["top"])
        self.group_count, self.group_keep = int(p.get("group_count", 1)), int(p.get("group_keep", 1))
        self.limit = float(p["limit"]) if p.get("limit") is not None else float("inf")
        self.slope, self.up_shift = float(p.get("slope", 1.0)), float(p.get("up_shift", 0.0))
        self.weight_scale = float(p.get("weight_scale", 1.0))
        score = p.get("score", "softmax")
        if score not in ("softmax", "sigmoid"):
            raise InvalidArgument(f"experts: a router scores by 'softmax' or 'sigmoid', got '{score}'")
        self.score_fn = ops.ROUTE_SIGMOID if score == "sigmoid" else ops.ROUTE_SOFTMAX
        self.group_top, self.renorm = int(p.get("group_top", 1)), bool(p.get("renorm", True))
        self.has_correction = bool(p.get("correction", False))
        self.correction = None
        E, G = self.experts, self.group_count
        if min(E, self.top, G, self.group_keep, self.inter) <= 0 or E % G or self.group_keep > G or \
                self.top > self.group_keep * (E // G) or self.top > 32:
            raise InvalidArgument(f"experts: cannot choose {self.top} (at most 32) of {E} experts in {G} groups of which "
                                  f"{self.group_keep} are kept")
        self.dtype = dtype

    def _expert(self, e: int, leaf: str) -> str:
        return f"{self.prefix}e{e}.{leaf}"

    def needs(self):
        n = {self.prefix + "router": TensorNeed((self.experts, self.hidden))}
        if self.has_correction:
            n[self.prefix + "correction"] = TensorNeed((self.experts,))
        for e in range(self.experts):
            n[self._expert(e, "gate")] = TensorNeed((self.inter, self.hidden))
            n[self._expert(e, "up")] = TensorNeed((self.inter, self.hidden))
            n[self._expert(e, "down")] = TensorNeed((self.hidden, self.inter))
        return n

    def bind(self, get):
        E = self.experts
        router = to_compute(get(self.prefix + "router"), self.dtype)
        rows = (E + 7) // 8 * 8
        padded = torch.zeros((rows, self.hidden), dtype=self.dtype, device=router.device)
        padded[:E] = router
        self.router = ops.bound_gemm(padded, split_many=False, pack=False)     # row-major: few tokens read it on the CUDA cores
        self.w_router = self.router.w
        self.router_rows = rows
        if self.has_correction:
            self.correction = get(self.prefix + "correction").to(torch.float32).contiguous()
        # [experts, 2 * inter, hidden]: an expert's gate rows, then its up rows; [experts, hidden, inter]
        w_gate_up = torch.stack([torch.cat([to_compute(get(self._expert(e, "gate")), self.dtype),
                                            to_compute(get(self._expert(e, "up")), self.dtype)], dim=0) for e in range(E)]).contiguous()
        w_down = torch.stack([to_compute(get(self._expert(e, "down")), self.dtype) for e in range(E)]).contiguous()
        # bfloat16 with sizes in whole 16-byte vectors: the experts' rows one after the other in k-blocks, the layout
        # that the tensor-core product streams (prompts) and that the few-rows kernel reads as well (decode)
        self.in_blocks = self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0 and w_down.is_cuda
        if self.in_blocks:
            w_gate_up = ops.pack_k_blocks(w_gate_up.view(E * 2 * self.inter, self.hidden))
            w_down = ops.pack_k_blocks(w_down.view(E * self.hidden, self.inter))
        self.w_gate_up, self.w_down = w_gate_up, w_down

    def forward(self, h, ctx):
        T, E, top, I, D = h.shape[0], self.experts, self.top, self.inter, self.hidden
        logits = ctx.ws.rows("moe.logits", T, self.router_rows, torch.float32)
        if T <= ROUTER_SIMT_ROWS:
            ops.gemm_simt(h, self.w_router, logits)         # a warp per expert streams its row: a few microseconds
        else:
            self.router(h, logits)
        ids = ctx.ws.rows("moe.ids", T, top, torch.int32)
        weights = ctx.ws.rows("moe.weights", T, top, torch.float32)
        ops.moe_route(logits[:, :E], top, self.group_count, self.group_keep, ids, weights, score_fn=self.score_fn,
                      correction=self.correction, group_top=self.group_top, renorm=self.renorm, weight_scale=self.weight_scale)
        pairs = T * top
        few = pairs <= 8 * E      # an expert has a few rows: a warp per output column streams its weights once
        if self.in_blocks:
            block_m = 4 if few else ops.GROUPED_TILE
        elif few and D % 4 == 0 and I % 4 == 0 and self.dtype == torch.float32:
            block_m = 4
        else:
            block_m = 16 if pairs <= 16 * E else 64
        rows_cap = ctx.ws.max_rows * top
        tiles_cap = max(ops.moe_max_tiles(rows_cap, E, 4), 1)
        sorted_pairs = ctx.ws.flat("moe.sorted", max(ops.moe_max_tiles(rows_cap, E, m) * m for m in (4, 16, 64, 128)), torch.int32)
        tile_expert = ctx.ws.flat("moe.tile_expert", tiles_cap, torch.int32)
        meta = ctx.ws.flat("moe.meta", 4, torch.int32)
        ops.moe_align(ids, E, block_m, sorted_pairs, tile_expert, meta)
        max_tiles = ops.moe_max_tiles(pairs, E, block_m)
        partial = ctx.ws.flat("moe.partial", rows_cap * D, torch.float32)
        if block_m == ops.GROUPED_TILE:
            # prompts on the tensor cores: rows copied into the listed order, two grouped products over dense operands,
            # the weighted results back to their tokens
            rows = max_tiles * block_m
            cap = ops.moe_max_tiles(rows_cap, E, block_m) * block_m
            xs = ctx.ws.flat("moe.listed", cap * D, self.dtype)[:rows * D].view(rows, D)
            ops.moe_gather(h, sorted_pairs, meta, top, xs)
            gu = ctx.ws.flat("moe.listed.gate_up", cap * 2 * I, self.dtype)[:rows * 2 * I].view(rows, 2 * I)
            ops.gemm_grouped(xs, self.w_gate_up, gu, 2 * I, D, meta, tile_expert)
            act = ctx.ws.flat("moe.listed.act", cap * I, self.dtype)[:rows * I].view(rows, I)
            ops.glu_clamped(gu, act, self.limit, self.slope, self.up_shift)
            y = xs                                          # the listed inputs are done with
            ops.gemm_grouped(act, self.w_down, y, D, I, meta, tile_expert)
            ops.moe_combine(y, sorted_pairs, meta, top, weights.view(-1), partial, T)
            return ops.SplitSum(partial, top, T, D)
        gu = ctx.ws.rows("moe.gate_up", T, top * 2 * I, self.dtype).view(pairs, 2 * I)
        ops.moe_gemm(h, self.w_gate_up, gu, top, block_m, sorted_pairs, tile_expert, meta, max_tiles,
                     blocks_of=(2 * I, D) if self.in_blocks else None)
        act = ctx.ws.rows("moe.act", T, top * I, self.dtype).view(pairs, I)
        ops.glu_clamped(gu, act, self.limit, self.slope, self.up_shift)
        ops.moe_gemm(act, self.w_down, None, top, block_m, sorted_pairs, tile_expert, meta, max_tiles, second=True,
                     partial=partial, weights=weights.view(-1), blocks_of=(D, I) if self.in_blocks else None)
        return ops.SplitSum(partial, top, T, D)


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
